"""Offline replay core: trace discovery, scores, exact top-k, ranking metrics
and the from-specification replay of one configuration (the oracle that the
fused engine must reproduce bit for bit on one shard).

Replay contract for a window of W logged steps after a branch point ``t0``
(``sga/replay.py:538-1172``, specification ``tests/test_replay_cycle.py:140-229``):

* the trace logs post-clip gradients; the pre-clip gradient is
  ``g = g_logged / coef_dense`` with ``coef_dense = min(1, clip / (norm + 1e-6))``;
* boundary steps (``si % T == 0``): with ``fold`` and ``si > 0`` the residual
  is first divided by ``T``; ``q = (g + res) * min(1, clip / (|g + res| + 1e-6))``;
  for ``0 < si < W - 1`` a new support is selected from ``score(q)`` on the
  pre-commit state; the residual is cleared;
* other steps: ``q = g * sel * min(1, clip / (|g * sel| + 1e-6))`` and
  ``res += g * (1 - sel)``;
* the commit is Adam with step count ``t0 + si + 1`` in the form
  ``w * (1 - lr * wd) - lr * u``; a boundary dual lr applies ``lr * scale``
  outside the outgoing support;
* ``distortion(H) = |w_sparse(H) - w_dense(H)| / |w_dense(H) - w0|``.

Every fp32 operation below is written as its own rounded step; the CUDA
kernels of ``csrc/replay.cu`` follow the same order (``-fmad=false``), so a
one-shard fused run equals this per-configuration replay bit for bit.
"""
from __future__ import annotations

import hashlib
import math
import os
import re
from dataclasses import dataclass, field
from typing import Optional

import torch

from ..plugins.scores import _div, compute_score

REPLAY_SEMANTIC_VERSION = 3
_G = re.compile(r"^step_(\d{6})_g\.pt$")
_S = re.compile(r"^step_(\d{6})_state\.pt$")


# ------------------------------------------------------------------ trace IO
@dataclass
class TraceInfo:
    dir: str
    names: list
    shapes: list
    groups: list
    g_dtype: str
    branch_points: list
    g_steps: list
    offsets: list = field(default_factory=list)
    numel: int = 0

    def window(self, t0: int, want: int) -> list:
        """Contiguous g steps starting at ``t0`` (a gap ends the window)."""
        have = set(self.g_steps)
        out = []
        t = t0
        while t in have and len(out) < want:
            out.append(t)
            t += 1
        return out


def discover_trace(trace_dir: str) -> TraceInfo:
    cat_path = os.path.join(trace_dir, "catalog.pt")
    if not os.path.exists(cat_path):
        raise FileNotFoundError(f"{trace_dir}: no catalog.pt")
    cat = torch.load(cat_path, weights_only=False)
    names = list(cat["catalog"].keys())
    shapes = [tuple(cat["catalog"][n]["shape"]) for n in names]
    groups = [int(cat["catalog"][n].get("param_group", 0)) for n in names]
    bps, gs = [], []
    for f in os.listdir(trace_dir):
        m = _S.match(f)
        if m:
            bps.append(int(m.group(1)))
        m = _G.match(f)
        if m:
            gs.append(int(m.group(1)))
    info = TraceInfo(trace_dir, names, shapes, groups, cat.get("g_dtype", "fp32"), sorted(bps), sorted(gs))
    off = 0
    for sh in shapes:
        info.offsets.append(off)
        off += int(math.prod(sh)) if sh else 1
    info.numel = off
    return info


def flatten(payload: dict, info: TraceInfo, dtype=torch.float32, lo: int = 0, hi: Optional[int] = None):
    """Catalog-ordered flat vector (or its ``[lo, hi)`` slice) of a ``{name: tensor}`` payload."""
    hi = info.numel if hi is None else hi
    out = torch.empty(hi - lo, dtype=dtype)
    for name, off, sh in zip(info.names, info.offsets, info.shapes):
        n = int(math.prod(sh)) if sh else 1
        a, b = max(off, lo), min(off + n, hi)
        if a < b:
            out[a - lo:b - lo] = payload[name].reshape(-1)[a - off:b - off].to(dtype)
    return out


def load_state(info: TraceInfo, t0: int):
    blob = torch.load(os.path.join(info.dir, f"step_{t0:06d}_state.pt"), weights_only=False)
    return blob["meta"], blob["payload"]


def load_g(info: TraceInfo, t: int, mmap: bool = True):
    """``mmap``: tensors are file-backed, so a caller that slices reads only its slice from disk."""
    blob = torch.load(os.path.join(info.dir, f"step_{t:06d}_g.pt"), weights_only=False, mmap=mmap)
    return blob["meta"], blob["payload"]


def group_vector(info: TraceInfo, per_group: list, lo: int = 0, hi: Optional[int] = None) -> torch.Tensor:
    """Per-element value of a per-group hyper-parameter."""
    hi = info.numel if hi is None else hi
    out = torch.empty(hi - lo, dtype=torch.float32)
    for off, sh, gi in zip(info.offsets, info.shapes, info.groups):
        n = int(math.prod(sh)) if sh else 1
        a, b = max(off, lo), min(off + n, hi)
        if a < b:
            out[a - lo:b - lo] = per_group[gi]
    return out


# ------------------------------------------------------------ exact selection
def abs_key(x: torch.Tensor) -> torch.Tensor:
    return x.contiguous().view(torch.int32) & 0x7FFFFFFF


def select_topk_flat(score: torch.Tensor, k: int) -> torch.Tensor:
    """Exactly ``k`` coordinates by ``|score|``: everything strictly above the
    k-th magnitude, then ties in flat index order. Returns a bool mask."""
    n = score.numel()
    k = max(0, min(int(k), n))
    sel = torch.zeros(n, dtype=torch.bool, device=score.device)
    if k == 0:
        return sel
    key = abs_key(score.float())
    thr = torch.kthvalue(key, n - k + 1).values
    gt = key > thr
    sel |= gt
    need = k - int(gt.sum())
    if need > 0:
        ties = torch.nonzero(key == thr, as_tuple=False).view(-1)[:need]
        sel[ties] = True
    return sel


def k_for(n: int, ratio_percent: float) -> int:
    return max(1, int(round(n * ratio_percent / 100.0)))


# ------------------------------------------------------------ ranking metrics
def ranking_metrics(score: torch.Tensor, label: torch.Tensor, k: int) -> dict:
    """How well top-k by ``|score|`` recovers top-k by ``label`` (the realised
    dense displacement): NDCG@k, recall@k and the label / score mass missed."""
    s, lab = score.abs().double(), label.abs().double()
    sel_s = select_topk_flat(score, k)
    sel_l = select_topk_flat(label, k)
    ideal = torch.sort(lab[sel_l], descending=True).values
    got = lab[sel_s][torch.argsort(s[sel_s], descending=True)]
    disc = 1.0 / torch.log2(torch.arange(2, k + 2, dtype=torch.float64, device=score.device))
    idcg = float((ideal * disc).sum())
    ndcg = float((got * disc).sum()) / idcg if idcg > 0 else 0.0
    tot_l, tot_s = float(lab.sum()), float(s.sum())
    return {"ndcg_at_k": ndcg, "recall_at_k": float((sel_s & sel_l).sum()) / max(k, 1),
            "missed_label_mass": float(lab[~sel_s].sum()) / tot_l if tot_l > 0 else 0.0,
            "missed_score_mass": float(s[~sel_s].sum()) / tot_s if tot_s > 0 else 0.0}


# ------------------------------------------------------------------- commits
@dataclass
class Hyper:
    wd: object              # per-element fp32 tensor (per-group weight decay) or a float
    lr: float = 0.0         # unused placeholder: the per-step lr comes from the trace meta
    beta1: float = 0.9
    beta2: float = 0.95
    eps: float = 1e-8
    clip: float = 1.0


def f32(x: float) -> float:
    return float(torch.tensor(x, dtype=torch.float32))


def adam_commit_torch(w, m, v, q, lr, wd, beta1, beta2, eps, count, optimizer="adamw", inactive=None, dual_lr=1.0,
                      label=None):
    """In-place commit in the replay form ``w * (1 - lr * wd) - lr * u``. ``label``
    (optional) accumulates the squared gradient-driven step ``(lr * u)^2``."""
    adams = optimizer == "adams"
    bc1 = 1.0 if adams else 1.0 - beta1 ** count
    bc2 = 1.0 if adams else 1.0 - beta2 ** count
    m1 = m * beta1 + q * (1.0 - beta1)
    g2 = (q * (1.0 - beta2)) * q
    v1 = ((m * m) * beta2 if adams else v * beta2) + g2
    mh, vh = (m1, v1) if adams else (_div(m1, bc1), _div(v1, bc2))
    u = mh / (torch.sqrt(vh) + eps)
    lr_t = lr if isinstance(lr, torch.Tensor) else torch.full_like(w, lr)
    if label is not None:
        step = lr_t * u
        label.add_(step * step)
    if inactive is not None and dual_lr != 1.0:
        # boundary dual lr (sga/replay.py:674-684): the whole displacement, decay term included, times the
        # lane's step size -- at every lane of the boundary commit, so the rounding differs from the form below
        lr_in = lr_t * dual_lr if isinstance(lr, torch.Tensor) else torch.full_like(w, lr * dual_lr)
        step_t = torch.where(inactive, lr_in, lr_t)
        w.copy_(w - (w * wd + u) * step_t)
    else:
        w.copy_(w * (1.0 - lr_t * wd) - lr_t * u)
    m.copy_(m1)
    v.copy_(v1)


def clip_coef(sumsq: float, clip: float) -> float:
    if clip <= 0.0:
        return 1.0
    return min(1.0, clip / (math.sqrt(sumsq) + 1.0e-6))


def coef_dense_for(gmeta: dict):
    """``(coefficient, flag)``: the clip coefficient the trainer applied to a logged gradient, from the step's
    own metadata (``min(1, clip / (norm + 1e-6))``), or 1.0 with the reason nobody clipped
    (``sga/replay.py:628-645``)."""
    clip = float(gmeta.get("clip_grad", 0.0))
    norm = float(gmeta.get("grad_norm", float("nan")))
    if clip <= 0.0:
        return 1.0, "clipping_disabled"
    if not math.isfinite(norm) or norm <= 0.0:
        return 1.0, "grad_norm_unavailable"
    return min(clip / (norm + 1.0e-6), 1.0), None


REPLAY_ONLY_SCORES = ("abs_g_step",)


def replay_score(name, w, m, v, q, hp: Hyper, count, optimizer="adamw", g_step=None):
    """Registry score on the pre-commit state in fp64, stored as fp32. ``abs_g_step`` exists only
    in the replay: ``|g|`` of the step's own gradient, without the residual a boundary adds to it
    (``g_step``; at the branch point, where there is no residual yet, it equals ``abs_g``)."""
    if name == "abs_g_step":
        return (q if g_step is None else g_step).abs().float()
    if name == "abs_g":   # the two magnitude scores need no fp64 copies of the whole state
        return q.abs().float()
    if name == "abs_m":
        return m.abs().float()
    adams = optimizer == "adams"
    bc1 = 1.0 if adams else 1.0 - hp.beta1 ** count
    bc2 = 1.0 if adams else 1.0 - hp.beta2 ** count
    wd = hp.wd.double() if isinstance(hp.wd, torch.Tensor) else hp.wd
    return compute_score(name, w.double(), m.double(), v.double(), q.double(), beta1=hp.beta1, beta2=hp.beta2,
                         eps=hp.eps, weight_decay=wd, bc1=bc1, bc2=bc2, optimizer=optimizer).float()


@dataclass(frozen=True)
class CycleConfig:
    score: str
    ratio_percent: float
    cycle_len: int
    optimizer: str = "adamw"
    fold: bool = False
    dual_lr: float = 1.0

    def key(self, multi: dict) -> str:
        k = self.score
        if multi.get("cycle_len") and self.cycle_len > 0:
            k += f"@T{self.cycle_len}"
        if multi.get("optimizer"):
            k += f"@{self.optimizer}"
        if multi.get("fold") and self.fold:
            k += "@fold"
        if multi.get("dual_lr"):
            k += f"@dl{self.dual_lr:g}"
        return k


def dense_replay(w0, m0, v0, logged, lrs, hp: Hyper, t0, optimizer="adamw", horizons=(), label_out=None):
    """The dense trajectory: the logged (already clipped) gradients as committed.
    Returns ``{h: w at horizon h}`` (h counts commits, 1-based). With ``label_out`` (a zeroed
    tensor like ``w0``) it also accumulates the ranking label of the reference's front block: the
    per-coordinate sum over the window of the squared gradient-driven step ``(lr * u)^2``
    (``sga/replay.py:646-668,790-812``; weight decay does not enter it)."""
    w, m, v = w0.clone(), m0.clone(), v0.clone()
    snaps = {}
    for si, g in enumerate(logged):
        lr = lrs[si]
        adam_commit_torch(w, m, v, g.to(w.device).float(), lr, hp.wd, hp.beta1, hp.beta2, hp.eps, t0 + si + 1,
                          optimizer, label=label_out)
        if si + 1 in horizons:
            snaps[si + 1] = w.clone()
    return snaps


def reference_cycle(w0, m0, v0, logged, grad_norms, lrs, hp: Hyper, t0, cfg: CycleConfig, branch_grad,
                    horizons=(), reselect=True):
    """One configuration replayed from the specification. Returns
    ``({h: w_sparse}, per_step records)``."""
    n = w0.numel()
    k = k_for(n, cfg.ratio_percent)
    w, m, v = w0.clone(), m0.clone(), v0.clone()
    res = torch.zeros_like(w0)
    sel = select_topk_flat(replay_score(cfg.score, w, m, v, branch_grad.float(), hp, t0 + 1, cfg.optimizer), k)
    T, W = cfg.cycle_len, len(logged)
    snaps, per_step = {}, []
    for si, g_logged in enumerate(logged):
        count = t0 + si + 1
        coef_dense = f32(clip_coef(grad_norms[si] ** 2, hp.clip)) if hp.clip > 0 else 1.0
        g = _div(g_logged.float(), coef_dense)
        boundary = T > 0 and si % T == 0  # cycle length 0: zerofill, the support stays frozen and nothing merges
        out_sel = None
        if boundary:
            if cfg.fold and si > 0:
                res = _div(res, float(T))
            q_pre = g + res
            coef = f32(clip_coef(float((q_pre.double() ** 2).sum()), hp.clip))
            q = q_pre * coef if coef != 1.0 else q_pre
            out_sel = sel
            if reselect and 0 < si < W - 1:
                sel = select_topk_flat(replay_score(cfg.score, w, m, v, q, hp, count, cfg.optimizer, g_step=g), k)
            res = torch.zeros_like(res)
        else:
            zero = torch.zeros_like(g)
            q_pre = torch.where(sel, g, zero)
            coef = f32(clip_coef(float((q_pre.double() ** 2).sum()), hp.clip))
            q = q_pre * coef if coef != 1.0 else q_pre
            res = res + torch.where(sel, zero, g)
        lr = lrs[si]
        adam_commit_torch(w, m, v, q, lr, hp.wd, hp.beta1, hp.beta2, hp.eps, count, cfg.optimizer,
                          inactive=(~out_sel if (boundary and cfg.dual_lr != 1.0) else None), dual_lr=cfg.dual_lr)
        per_step.append({"si": si, "boundary": boundary, "coef": coef, "selected": int(sel.sum())})
        if si + 1 in horizons:
            snaps[si + 1] = w.clone()
    return snaps, per_step


def distortion(w_s, w_d, w0) -> float:
    num = float(((w_s.double() - w_d.double()) ** 2).sum())
    den = float(((w_d.double() - w0.double()) ** 2).sum())
    return math.sqrt(num) / math.sqrt(den) if den > 0 else float("nan")


# ---------------------------------------------------------------- dense cache
def cache_ident(trace_dir, t0, W, horizons, replay_dtype, trace_dtype, engine, optimizer) -> dict:
    return {"semantic_version": REPLAY_SEMANTIC_VERSION, "trace_dir": os.path.abspath(trace_dir), "t0": int(t0),
            "window": int(W), "horizons": [int(h) for h in horizons], "replay_dtype": replay_dtype,
            "trace_dtype": trace_dtype, "engine": engine, "optimizer": optimizer}


def cache_path(cache_dir: str, ident: dict) -> str:
    h = hashlib.sha1(repr(sorted(ident.items())).encode()).hexdigest()[:16]
    return os.path.join(cache_dir, f"dense_{h}.pt")


def save_cache(cache_dir: str, ident: dict, blob: dict) -> str:
    os.makedirs(cache_dir, exist_ok=True)
    path = cache_path(cache_dir, ident)
    tmp = f"{path}.tmp.{os.getpid()}"
    torch.save(dict(blob, ident=ident), tmp)
    os.replace(tmp, path)
    return path


def load_cache(cache_dir: str, ident: dict):
    path = cache_path(cache_dir, ident)
    if not os.path.exists(path):
        return None
    blob = torch.load(path, weights_only=False)
    if blob.get("ident") != ident:
        raise ValueError(f"dense cache {path} was written for a different replay (ident mismatch)")
    return blob
