"""Hyper-parameters, step counter and checkpoint view of the flat optimizer.

The state itself lives in the arena (``exp_avg`` / ``exp_avg_sq`` / fp32
masters). ``state_dict`` / ``load_state_dict`` expose it in exactly
``torch.optim.Adam``'s layout -- ``state[i] = {"exp_avg", "exp_avg_sq"}`` per
parameter index plus ``param_groups[g]["step"]`` -- which is the layout the
reference's templates read and write (``sga/plugins/optimizer/adamw.py:849-852``,
``sga/kernels.py:329-365``). The residual (the grad arena), the active support
and the cycle position are deliberately not part of it.
"""
from __future__ import annotations

import torch


class OptimizerConfig:
    def __init__(self, lr=3e-4, weight_decay=0.1, adam_beta1=0.9, adam_beta2=0.95, adam_eps=1e-8, clip_grad=1.0,
                 log_num_zeros_in_grad=False, check_finite=False):
        self.lr = lr
        self.weight_decay = weight_decay
        self.adam_beta1 = adam_beta1
        self.adam_beta2 = adam_beta2
        self.adam_eps = adam_eps
        self.clip_grad = clip_grad
        self.log_num_zeros_in_grad = log_num_zeros_in_grad
        self.check_finite = check_finite


class FlatOptimizer:
    """Two parameter groups by construction: 0 = weight decay, 1 = no weight decay."""

    def __init__(self, arena, config: OptimizerConfig):
        self.arena = arena
        self.config = config
        self.param_groups = [
            {"lr": config.lr, "weight_decay": config.weight_decay, "betas": (config.adam_beta1, config.adam_beta2),
             "eps": config.adam_eps, "step": 0, "params": [i for i, s in enumerate(arena.slots) if s.spec.group == 0]},
            {"lr": config.lr, "weight_decay": 0.0, "betas": (config.adam_beta1, config.adam_beta2),
             "eps": config.adam_eps, "step": 0, "params": [i for i, s in enumerate(arena.slots) if s.spec.group == 1]},
        ]

    # shared Adam step counter (advanced exactly once per engine step)
    @property
    def step_count(self) -> int:
        return int(self.param_groups[0]["step"])

    def advance_step(self) -> int:
        for g in self.param_groups:
            g["step"] = int(g["step"]) + 1
        return self.step_count

    def peek_step(self) -> int:
        return self.step_count + 1

    def set_lr(self, lr: float) -> None:
        for g in self.param_groups:
            g["lr"] = lr

    def group_lr(self):
        return [g["lr"] for g in self.param_groups]

    def group_wd(self):
        return [g["weight_decay"] for g in self.param_groups]

    def prepare_grads(self) -> bool:
        """Returns found_inf (True = bad step). bf16 training has no loss scale, so
        the finite check is optional."""
        if not self.config.check_finite:
            return False
        return not bool(torch.isfinite(self.arena.main_grad.sum()).item())

    # ------------------------------------------------------ checkpoint
    def state_dict(self) -> dict:
        state = {}
        tensors = self.arena.state_dict_tensors()
        for i, s in enumerate(self.arena.slots):
            _w, m, v = tensors[s.name]
            state[i] = {"exp_avg": m.detach().cpu().clone(), "exp_avg_sq": v.detach().cpu().clone()}
        groups = [{k: (list(v) if k == "params" else v) for k, v in g.items()} for g in self.param_groups]
        fp32 = {s.name: tensors[s.name][0].detach().cpu().clone() for s in self.arena.slots}
        return {"state": state, "param_groups": groups, "fp32_from_fp16_params": fp32}

    def load_state_dict(self, sd: dict) -> None:
        tensors = self.arena.state_dict_tensors()
        for i, s in enumerate(self.arena.slots):
            w, m, v = tensors[s.name]
            st = sd["state"].get(i, sd["state"].get(str(i)))
            if st is not None:
                m.copy_(st["exp_avg"])
                v.copy_(st["exp_avg_sq"])
            if "fp32_from_fp16_params" in sd and s.name in sd["fp32_from_fp16_params"]:
                w.copy_(sd["fp32_from_fp16_params"][s.name])
        for g, sg in zip(self.param_groups, sd["param_groups"]):
            for k in ("lr", "weight_decay", "eps", "step"):
                if k in sg:
                    g[k] = sg[k]
            if "betas" in sg:
                g["betas"] = tuple(sg["betas"])
        self.arena.sync_model_from_main()
