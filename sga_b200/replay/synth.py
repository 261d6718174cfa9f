"""Synthetic trace generator (no training run needed): per-step gradient dumps
of a flat parameter vector drawn ``N(0, sigma_t^2)`` with
``sigma_t = 1e-3 * (1 + 0.5 * sin(step / 8))`` and 1 % of the coordinates
scaled x20 (heavy tails), plus an fp32 AdamW state snapshot at the branch
point. The files follow the trace format exactly, so every replay path can
consume them. Used by the replay benchmark and the tests.
"""
from __future__ import annotations

import math
import os

import torch


def make_synthetic_trace(out_dir: str, sizes=(400000, 300000, 170000), steps: int = 64, t0: int = 0,
                         g_dtype: str = "bf16", seed: int = 0, lr: float = 3e-4, clip: float = 1.0,
                         groups=None) -> str:
    os.makedirs(out_dir, exist_ok=True)
    names = [f"decoder.layers.{i}.weight" for i in range(len(sizes))]
    groups = list(groups) if groups is not None else [i % 2 for i in range(len(sizes))]
    gen = torch.Generator().manual_seed(seed)
    pg = [{"lr": lr, "weight_decay": 0.1, "adam_beta1": 0.9, "adam_beta2": 0.95, "adam_eps": 1e-8},
          {"lr": lr, "weight_decay": 0.0, "adam_beta1": 0.9, "adam_beta2": 0.95, "adam_eps": 1e-8}]

    def meta(step, norm):
        return {"step": step, "phase": "shadow", "lr": [lr, lr], "grad_norm": float(norm), "clip_grad": clip,
                "weight_decay": 0.1, "adam_beta1": 0.9, "adam_beta2": 0.95, "adam_eps": 1e-8, "param_groups": pg}

    def grad(step):
        sigma = 1e-3 * (1 + 0.5 * math.sin(step / 8.0))
        raw, sq = {}, 0.0
        for n, sz in zip(names, sizes):
            g = torch.randn(sz, generator=gen) * sigma
            heavy = torch.rand(sz, generator=gen) < 0.01
            g = torch.where(heavy, g * 20.0, g)
            raw[n] = g
            sq += float((g.double() ** 2).sum())
        norm = math.sqrt(sq)
        coef = min(1.0, clip / (norm + 1e-6)) if clip > 0 else 1.0
        return {n: (g * coef) for n, g in raw.items()}, norm   # the trace logs post-clip gradients

    catalog = {n: {"shape": [sz], "dtype": "torch.float32", "param_group": gi} for n, sz, gi in
               zip(names, sizes, groups)}
    torch.save({"meta": meta(t0, 0.0), "catalog": catalog, "g_dtype": g_dtype}, os.path.join(out_dir, "catalog.pt"))
    dt = torch.bfloat16 if g_dtype == "bf16" else torch.float32
    for si in range(steps):
        step = t0 + si
        g, norm = grad(step)
        gq = {n: t.to(dt) for n, t in g.items()}
        if si == 0:
            state = {"w": {n: torch.randn(sz, generator=gen) * 0.02 for n, sz in zip(names, sizes)},
                     "m": {n: torch.randn(sz, generator=gen) * 1e-6 for n, sz in zip(names, sizes)},
                     "v": {n: (torch.randn(sz, generator=gen) * 1e-6).abs() for n, sz in zip(names, sizes)},
                     "g": {n: t.float() for n, t in gq.items()}}
            m = meta(step, norm)
            m["state_absent"] = False
            torch.save({"meta": m, "payload": state}, os.path.join(out_dir, f"step_{step:06d}_state.pt"))
        torch.save({"meta": meta(step, norm), "payload": gq}, os.path.join(out_dir, f"step_{step:06d}_g.pt"))
    return out_dir
