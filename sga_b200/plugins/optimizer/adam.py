"""The residual-aware optimizer templates: ``SgaAdamW`` and ``SgaAdamS``.

A full step commits the dense-averaged gradient at every coordinate and
writes the configured score into the grad buffer (the next reselection reads
it from there); with the boundary dual lr it applies ``lr * scale`` outside
the outgoing support. A sparse step commits the communicated coordinates
only (everything else sees ``g = 0`` and keeps accumulating in the grad
buffer), multiplies the clip coefficient in-register, clears what was
communicated, and on the step before a full sync optionally folds the
residual by ``1 / fold_window``. ``reset`` zeroes the grad buffers after a
full step. AdamS differs in the second-moment recursion only.

On CUDA each step is one launch of the multi-tensor kernel over the whole
arena (``csrc/optim.cu``), which also writes the bf16 model parameters; on
CPU the PyTorch reference runs per parameter record.
Surface and semantics: ``sga/plugins/optimizer/adamw.py:795-986``,
``adams.py:657-850``.
"""
from __future__ import annotations

import torch

from ...config import get_args
from ..scores import EMIT_CODES, get_score_spec
from .reference import grad_correct_torch


class _SgaAdamBase:
    optimizer_name = "adamw"

    def __init__(self):
        args = get_args()
        self.emit_score = args.sga_score
        get_score_spec(self.emit_score)  # unknown names fail here
        self.residual_mean = bool(args.sga_optimizer_residual_mean)
        self.inactive_lr_scale = float(args.sga_optimizer_full_sync_inactive_lr_scale)

    # state lives in the arena; nothing to allocate per parameter
    def ensure_state(self, bucket_states) -> None:
        return None

    @property
    def adams(self) -> bool:
        return self.optimizer_name == "adams"

    # ------------------------------------------------------------ steps
    def full_step(self, ctx) -> None:
        lr_scale = self.inactive_lr_scale if (self.inactive_lr_scale != 1.0 and ctx.mask_arena is not None
                                              and ctx.support is not None) else 1.0
        self._run(ctx, emit=self.emit_score if ctx.emit else None, mask=ctx.mask_arena if lr_scale != 1.0 else None,
                  clear=False, fold=False, lr_scale=lr_scale, full=True)

    def sparse_step(self, ctx) -> None:
        fold = self.residual_mean and ctx.next_step_is_full
        self._run(ctx, emit=None, mask=ctx.mask_arena, clear=True, fold=fold, lr_scale=1.0, full=False)

    def reset(self, ctx, was_full: bool) -> None:
        """After a full step the grad buffers (now holding scores) are zeroed;
        a sparse step already cleared what it consumed."""
        if was_full and ctx.arena is not None:
            ctx.arena.main_grad.zero_()

    # ------------------------------------------------------------- impl
    def _run(self, ctx, *, emit, mask, clear, fold, lr_scale, full):
        opt = ctx.optimizer
        arena = ctx.arena
        step = opt.peek_step()
        g0 = opt.param_groups[0]
        beta1, beta2 = g0["betas"]
        eps = g0["eps"]
        coeff = ctx.apply_coeff
        src = arena.comm if ctx.grad_source == "comm" else arena.main_grad
        if ctx.sharded is not None:
            # Every rank holds the same gradient here (the all-reduced bucket on a full step, the
            # rank-ordered sum of all ranks' pairs on a sparse one), so the update can be cut like the
            # dense step's: 1 / W of the weights and moments per rank, bf16 copies stored to every peer.
            if emit is not None or mask is not None or lr_scale != 1.0:
                raise NotImplementedError("the sharded step covers the rank-local index mode (no score emission, "
                                          "no mask, no boundary dual lr)")
            coeff_t = coeff if isinstance(coeff, torch.Tensor) else (
                None if coeff == 1.0 else torch.tensor([coeff], dtype=torch.float32, device=arena.device))
            ctx.sharded.step(arena, src, opt, beta1=beta1, beta2=beta2, eps=eps, step=step, coeff=coeff_t,
                             adams=self.adams)
            if clear:
                src.zero_()   # the replicated kernel clears what it consumed in the same pass; here only a slice is read
            if fold:
                from ... import kernels as K

                K.scale_(arena.main_grad, None, 1.0 / float(ctx.fold_window))
        elif arena.device.type == "cuda":
            from ... import kernels as K

            coeff_t = None
            if isinstance(coeff, torch.Tensor):
                coeff_t = coeff
            elif coeff != 1.0:
                coeff_t = torch.tensor([coeff], dtype=torch.float32, device=arena.device)
            K.adam_step(arena.main_param, src, arena.exp_avg, arena.exp_avg_sq, arena.segment_table(),
                        opt.group_lr(), opt.group_wd(), beta1=beta1, beta2=beta2, eps=eps, step=step,
                        model=arena.model_param, mask=mask, coeff=coeff_t, emit=EMIT_CODES[emit], clear=clear,
                        fold=False if ctx.grad_source == "comm" else fold, interval=float(ctx.fold_window),
                        lr_scale=lr_scale, adams=self.adams)
            if fold and ctx.grad_source == "comm":
                K.scale_(arena.main_grad, None, 1.0 / float(ctx.fold_window))
        else:
            c = float(coeff.item()) if isinstance(coeff, torch.Tensor) else float(coeff)
            bc1, bc2 = 1.0 - beta1 ** step, 1.0 - beta2 ** step
            for s in arena.slots:
                sl = slice(s.start, s.end)
                grp = opt.param_groups[s.spec.group]
                grad_correct_torch(arena.main_param[sl], src[sl], arena.exp_avg[sl], arena.exp_avg_sq[sl], grp["lr"],
                                   beta1, beta2, eps, grp["weight_decay"], bc1, bc2,
                                   mask[sl] if mask is not None else None, emit, coeff=c, clear=clear,
                                   fold=False if ctx.grad_source == "comm" else fold,
                                   interval=float(ctx.fold_window), inactive_lr_scale=lr_scale,
                                   optimizer=self.optimizer_name, model_param=arena.model_param[sl])
            if fold and ctx.grad_source == "comm":
                arena.main_grad.div_(float(ctx.fold_window))
        opt.advance_step()


class SgaAdamW(_SgaAdamBase):
    optimizer_name = "adamw"


class SgaAdamS(_SgaAdamBase):
    optimizer_name = "adams"
