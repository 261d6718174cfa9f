"""PyTorch reference of the residual-aware Adam step (AdamW and AdamS).

``grad_correct_torch`` is both the CPU execution path (gloo runs, unit tests)
and the oracle the CUDA kernel (``csrc/optim.cu``) is compared with, bit for
bit: every line below is one separately rounded fp32 operation, in the order
the kernel uses. Contract (``sga/plugins/optimizer/adamw_torch.py:31-93``,
``adams_torch.py:33-85``):

* ``emit_score=None``: sparse step. With a mask, masked-out lanes see
  ``g = 0``; ``coeff`` multiplies ``g`` at active lanes; ``clear`` zeroes the
  active lanes of ``grad`` after use; ``fold`` divides ``grad`` by
  ``interval`` afterwards.
* ``emit_score=<name>``: full step. The named score is written into ``grad``.
* ``inactive_lr_scale != 1``: full-step dual lr. The commit and the score are
  mask-blind; only the applied step splits (``lr`` at active lanes,
  ``lr * scale`` elsewhere).
* m and v advance at every lane on every step; the weight always moves by
  ``lr * (wd * w + m_hat / (sqrt(v_hat) + eps))``.
"""
from __future__ import annotations

import torch

from ..scores import _div, compute_score


def grad_correct_torch(param, grad, m, v, lr, beta1, beta2, eps, weight_decay, bias_correction1, bias_correction2,
                       mask, emit_score, coeff=1.0, clear=False, fold=False, interval=1.0, inactive_lr_scale=1.0,
                       optimizer="adamw", model_param=None) -> None:
    adams = optimizer == "adams"
    bc1 = 1.0 if adams else bias_correction1
    bc2 = 1.0 if adams else bias_correction2
    active = (mask > 0) if mask is not None else None
    if inactive_lr_scale != 1.0:
        assert active is not None, "dual lr needs the outgoing support mask"
        g = grad
        lr_apply = torch.where(active, torch.full_like(param, lr), torch.full_like(param, lr) * inactive_lr_scale)
    elif active is not None:
        g = torch.where(active, grad, torch.zeros_like(grad))
        lr_apply = lr
    else:
        g = grad
        lr_apply = lr
    if coeff != 1.0:
        # the dual-lr boundary commits every lane, so the clip coefficient reaches every lane too
        g = torch.where(active, g * coeff, g) if (active is not None and inactive_lr_scale == 1.0) else g * coeff
    m_new = m * beta1 + g * (1.0 - beta1)
    g2 = (g * (1.0 - beta2)) * g
    if adams:
        v_new = (m * m) * beta2 + g2
        mh, vh = m_new, v_new
    else:
        v_new = v * beta2 + g2
        mh, vh = _div(m_new, bc1), _div(v_new, bc2)
    u = mh / (torch.sqrt(vh) + eps)
    update = weight_decay * param + u
    if emit_score is None:
        score = None
    elif emit_score == "update":
        score = update
    else:
        score = compute_score(emit_score, param, m, v, g, beta1=beta1, beta2=beta2, eps=eps,
                              weight_decay=weight_decay, bc1=bc1, bc2=bc2, optimizer=optimizer)
    m.copy_(m_new)
    v.copy_(v_new)
    if score is not None:
        grad.copy_(score)
    else:
        if clear:
            if active is not None:
                grad.masked_fill_(active, 0.0)
            else:
                grad.zero_()
        if fold:
            grad.copy_(_div(grad, float(interval)))
    param.sub_(lr_apply * update)
    if model_param is not None:
        model_param.copy_(param)


def bias_corrections(beta1, beta2, step):
    return 1.0 - beta1 ** step, 1.0 - beta2 ** step
