"""Optimizer plugin protocol: the per-parameter record and the per-step context.

A template exposes ``emit_score``, ``ensure_state(bucket_states)``,
``full_step(ctx)``, ``sparse_step(ctx)`` and ``reset(ctx, was_full)``
(``sga/plugins/optimizer/__init__.py:20-87``). On CUDA a step is one
multi-tensor launch over the flat arena (``ctx.arena``); the records are the
per-parameter view of the same memory used by the CPU path, the trace
collector and the shadow scorer.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional


@dataclass
class ParamRecord:
    model_param: object
    main_param: object
    bucket_state: object
    start: int            # element span inside the bucket
    end: int
    lr: float
    beta1: float
    beta2: float
    eps: float
    weight_decay: float
    step: int
    name: str = ""
    grad: object = None   # fp32 main-grad view (the synced gradient; the score after a full step)
    m: object = None
    v: object = None
    group: int = 0

    def mask_u8(self):
        bs = self.bucket_state
        if bs is None or bs.active_mask_u8 is None:
            return None
        return bs.active_mask_u8[self.start:self.end]


@dataclass
class OptContext:
    records: list
    phase: str                         # 'full' | 'sparse'
    support: object = None
    bucket_states: list = None
    fold_window: int = 1
    next_step_is_full: bool = False
    apply_coeff: object = 1.0          # float, or a device scalar tensor (no host round trip)
    compact_values: Optional[dict] = None
    arena: object = None               # FlatArena for the one-launch CUDA path
    optimizer: object = None           # FlatOptimizer (hyper-parameters, step)
    mask_arena: object = None          # uint8 [arena.numel]: active support mask of every bucket
    grad_source: str = "grad"          # 'grad' | 'comm' (rank-local index mode reads the staging arena)
    emit: bool = True                  # full step: write the score into the grad buffer
    sharded: object = None             # ShardedStep: every rank updates the bucket slices it owns and pushes
                                       # the bf16 parameters to its peers (None: replicated update)
