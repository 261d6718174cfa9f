"""Read-only boundary scoring for shadow runs.

A shadow run commits with the stock dense step; at cycle boundaries the
configured score is evaluated from the pre-commit state (weights, moments and
the clipped synced gradient) with the bias corrections of the commit that is
about to happen, without writing to any of it. ``sga/shadow.py:30-95``.
"""
from __future__ import annotations

from ..plugins.scores import compute_score


def readonly_score(rec, score_name: str, optimizer_name: str = "adamw"):
    step = rec.step
    bc1 = 1.0 - rec.beta1 ** step
    bc2 = 1.0 - rec.beta2 ** step
    if optimizer_name == "adams":
        bc1 = bc2 = 1.0
    return compute_score(score_name, rec.main_param, rec.m, rec.v, rec.grad, beta1=rec.beta1, beta2=rec.beta2,
                         eps=rec.eps, weight_decay=rec.weight_decay, bc1=bc1, bc2=bc2, update_includes_wd=True,
                         optimizer=optimizer_name)
