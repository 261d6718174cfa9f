"""Score registry: the four boundary scores as data.

Each score is a pure function of the pre-commit optimizer state and the
gradient being committed; consumers rank coordinates by ``|score|``.

  update  signed ``wd * w + U(g)``
  abs_g   ``|g|`` (on a boundary step ``g`` already is gradient + residual)
  abs_m   ``|m|`` of the pre-commit first moment
  coi     ``|U(g) - U(0)|`` (the weight-decay term cancels)

``U(g) = m_hat / (sqrt(v_hat) + eps)`` is taken after folding ``g`` into the
moments with the upcoming commit's bias corrections. Under AdamS the second
moment is rebuilt from the pre-commit first moment and there is no bias
correction. Formulas and their fp32 operation order follow
``sga/plugins/scores.py:147-269`` so the CUDA kernels (``csrc/optim.cu``) and
the CPU path agree bit for bit; every intermediate is a separately rounded
fp32 operation (no fused multiply-add).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable

import torch

OPTIMIZERS = ("adamw", "adams")


@dataclass(frozen=True)
class ScoreSpec:
    formula: Callable[..., torch.Tensor]
    doc: str
    scratch: bool = False  # the formula needs parameter-sized temporaries


_SCORES: dict = {}


def register_score(name: str, spec: ScoreSpec) -> None:
    if name in _SCORES:
        raise ValueError(f"duplicate score registration '{name}'")
    _SCORES[name] = spec


def _div(x, d):
    """True IEEE division by a scalar. PyTorch's CUDA ``tensor / python_float``
    multiplies by the reciprocal instead, which rounds differently; dividing by
    a 0-dim tensor keeps one correctly rounded division on every device."""
    if isinstance(d, torch.Tensor):
        return x / d
    if d == 1.0:
        return x
    return x / torch.tensor(d, dtype=x.dtype, device=x.device)


def moments_after(m, v, g, beta1, beta2, bc1, bc2, optimizer="adamw"):
    """(m_hat, v_hat) after folding ``g`` in, with this framework's op order."""
    if optimizer not in OPTIMIZERS:
        raise ValueError(f"Unknown SGA optimizer '{optimizer}' for the score formulas (registered: adamw, adams)")
    m_new = m * beta1 + g * (1.0 - beta1)
    g2 = (g * (1.0 - beta2)) * g
    if optimizer == "adamw":
        v_new = v * beta2 + g2
        return _div(m_new, bc1), _div(v_new, bc2)
    v_new = (m * m) * beta2 + g2
    return m_new, v_new


def u_of_g(m, v, g, beta1, beta2, eps, bc1, bc2, optimizer="adamw"):
    mh, vh = moments_after(m, v, g, beta1, beta2, bc1, bc2, optimizer)
    return mh / (torch.sqrt(vh) + eps)


def u_of_zero(m, v, beta1, beta2, eps, bc1, bc2, optimizer="adamw"):
    if optimizer == "adams":
        return (m * beta1) / (torch.sqrt((m * m) * beta2) + eps)
    return _div(m * beta1, bc1) / (torch.sqrt(_div(v * beta2, bc2)) + eps)


def _abs_g(w, m, v, g, beta1, beta2, eps, weight_decay, bc1, bc2, update_includes_wd=True, optimizer="adamw",
           scratch=None):
    return g.abs()


def _abs_m(w, m, v, g, beta1, beta2, eps, weight_decay, bc1, bc2, update_includes_wd=True, optimizer="adamw",
           scratch=None):
    return m.abs()


def _update(w, m, v, g, beta1, beta2, eps, weight_decay, bc1, bc2, update_includes_wd=True, optimizer="adamw",
            scratch=None):
    u = u_of_g(m, v, g, beta1, beta2, eps, bc1, bc2, optimizer)
    return weight_decay * w + u if update_includes_wd else u


def _coi(w, m, v, g, beta1, beta2, eps, weight_decay, bc1, bc2, update_includes_wd=True, optimizer="adamw",
         scratch=None):
    ug = u_of_g(m, v, g, beta1, beta2, eps, bc1, bc2, optimizer)
    u0 = u_of_zero(m, v, beta1, beta2, eps, bc1, bc2, optimizer)
    return (ug - u0).abs()


def register_default_scores() -> None:
    _SCORES.setdefault("update", ScoreSpec(_update, "signed weight update wd*w + U(g); ranked by magnitude", True))
    _SCORES.setdefault("abs_g", ScoreSpec(_abs_g, "|g| of the committed, fully synced gradient"))
    _SCORES.setdefault("abs_m", ScoreSpec(_abs_m, "|m| of the pre-commit first moment"))
    _SCORES.setdefault("coi", ScoreSpec(_coi, "counterfactual optimizer impact |U(g) - U(0)|", True))


def get_score_spec(name: str) -> ScoreSpec:
    register_default_scores()
    try:
        return _SCORES[name]
    except KeyError:
        raise ValueError(f"Unknown SGA score '{name}'. Registered: {score_names()}") from None


def score_names():
    register_default_scores()
    return sorted(_SCORES)


def compute_score(name, w, m, v, g, *, beta1, beta2, eps, weight_decay, bc1, bc2, update_includes_wd=True,
                  optimizer="adamw"):
    return get_score_spec(name).formula(w, m, v, g, beta1, beta2, eps, weight_decay, bc1, bc2,
                                        update_includes_wd=update_includes_wd, optimizer=optimizer)


# Code the CUDA optimizer kernel uses for "which score to write into the grad
# buffer on a full step" (-1 = none, i.e. a sparse step).
EMIT_CODES = {None: -1, "update": 0, "abs_g": 1, "abs_m": 2, "coi": 3}

register_default_scores()
