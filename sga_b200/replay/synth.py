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


class SyntheticSource:
    """The synthetic trace at full size without files: state snapshot and per-step gradients of a
    flat ``numel``-element vector generated on the replay device, block by block, from a seed.

    A dump of the 1.24 B-element vector is 2.5 GB per step in bf16 (159 GB for 64 steps), more than a
    benchmark box should be asked to write and read back; generated values are the same distribution
    (``sigma_t = 1e-3 * (1 + 0.5 * sin(t / 8))``, 1 % of the coordinates x20, state ``m ~ N(0, 1e-6^2)``,
    ``v = |N(0, 1e-6^2)|``, ``w ~ N(0, 0.02^2)``). Every 4 Mi-element block has its own generator seeded
    by (seed, array, step, block), so any sharding of the vector sees the same numbers and a step can be
    produced again whenever a pass needs it. Gradients are logged unclipped (``clip_grad`` 0)."""

    BLOCK = 1 << 22

    def __init__(self, numel: int, steps: int = 64, seed: int = 0, lr: float = 3e-4, g_dtype: str = "bf16"):
        self.numel, self.steps, self.seed, self.lr, self.g_dtype = int(numel), int(steps), int(seed), float(lr), g_dtype
        self.offsets, self.shapes = [0], [(int(numel),)]

    def __repr__(self):
        return f"synthetic(numel={self.numel}, steps={self.steps}, seed={self.seed}, g={self.g_dtype})"

    # ---- the parts of a trace the fused engine reads
    def window(self, t0: int, want: int) -> list:
        return list(range(t0, min(t0 + want, self.steps)))

    def meta(self, step: int) -> dict:
        pg = [{"lr": self.lr, "weight_decay": 0.1, "adam_beta1": 0.9, "adam_beta2": 0.95, "adam_eps": 1e-8}]
        return {"step": step, "phase": "shadow", "lr": [self.lr], "grad_norm": float("nan"), "clip_grad": 0.0,
                "weight_decay": 0.1, "adam_beta1": 0.9, "adam_beta2": 0.95, "adam_eps": 1e-8, "param_groups": pg,
                "state_absent": False}

    def _block(self, what: int, step: int, b: int, device) -> torch.Tensor:
        gen = torch.Generator(device=device)
        gen.manual_seed((self.seed * 1000003 + what * 7919 + step * 104729 + b * 15485863) % (2 ** 63 - 1))
        x = torch.randn(self.BLOCK, generator=gen, device=device)
        if what == 0:   # gradient of `step`
            sigma = 1e-3 * (1 + 0.5 * math.sin(step / 8.0))
            heavy = torch.rand(self.BLOCK, generator=gen, device=device) < 0.01
            return torch.where(heavy, x * (20.0 * sigma), x * sigma)
        if what == 1:
            return x * 0.02
        if what == 2:
            return x * 1e-6
        return (x * 1e-6).abs()

    def slice(self, what: str, step: int, lo: int, hi: int, device, dtype=torch.float32) -> torch.Tensor:
        """Elements ``[lo, hi)`` of array ``what`` ('g' of ``step``, or the snapshot's 'w' / 'm' / 'v')."""
        code = {"g": 0, "w": 1, "m": 2, "v": 3}[what]
        out = torch.empty(hi - lo, dtype=dtype, device=device)
        for b in range(lo // self.BLOCK, (hi + self.BLOCK - 1) // self.BLOCK if hi > lo else 0):
            b0 = b * self.BLOCK
            a, e = max(lo, b0), min(hi, b0 + self.BLOCK)
            out[a - lo:e - lo] = self._block(code, step if code == 0 else 0, b, device)[a - b0:e - b0].to(dtype)
        return out

    def gradients(self, steps, lo: int, hi: int, device):
        """Lazy sequence of this shard's logged gradients: element ``i`` is generated when it is read."""
        src, dt = self, (torch.bfloat16 if self.g_dtype == "bf16" else torch.float32)

        class _Lazy:
            def __len__(self):
                return len(steps)

            def __getitem__(self, i):
                return src.slice("g", steps[i], lo, hi, device, dt)

            def __iter__(self):
                return (self[i] for i in range(len(steps)))

        return _Lazy()
