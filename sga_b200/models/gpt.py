"""Decoder-only transformer (Llama-3 / Qwen3 family) with a hand-scheduled
forward and backward pass over the flat parameter arena.

There is no autograd graph: ``forward_backward`` runs the layers, keeps
exactly the activations the backward needs, computes the token-mean
cross-entropy with its logit gradient in one kernel, and walks the layers in
reverse. Weight gradients are accumulated by the GEMM epilogue straight into
the fp32 ``main_grad`` arena (no bf16 gradient tensors, no separate
accumulation pass); residual joins ride the GEMM epilogue of the output and
down projections. As soon as a parameter's gradient is final the model calls
``on_param_done(slot)`` so that the data-parallel layer can start a bucket's
synchronisation while the rest of the backward pass is still running.

Architecture: pre-norm blocks, RMSNorm, rotary embedding on half-split pairs,
grouped-query causal attention, SwiGLU MLP with fused gate|up projection,
optional per-head QK RMSNorm (Qwen3), tied or untied output embedding.
The geometry presets are those of the reference's example configs
(``examples/llama3/train_1b_adamw.yaml:106-142``,
``examples/qwen3/train_q3_06b.yaml:115-165``) and of the headline benchmark.
"""
from __future__ import annotations

from dataclasses import dataclass, replace
from typing import Callable, Optional

import torch

from ..ops import attention as A
from ..ops import functional as F
from ..runtime.arena import FlatArena, ParamSpec


@dataclass(frozen=True)
class GPTConfig:
    name: str
    num_layers: int
    hidden: int
    ffn: int
    n_heads: int
    n_kv_heads: int
    head_dim: int
    vocab: int
    seq_len: int
    rope_theta: float = 500000.0
    norm_eps: float = 1e-5
    qk_norm: bool = False
    tied_embeddings: bool = True
    init_std: float = 0.02

    @property
    def qkv_dim(self) -> int:
        return (self.n_heads + 2 * self.n_kv_heads) * self.head_dim

    def num_params(self) -> int:
        per_layer = (self.qkv_dim * self.hidden + self.n_heads * self.head_dim * self.hidden
                     + 3 * self.hidden * self.ffn + 2 * self.hidden + (2 * self.head_dim if self.qk_norm else 0))
        emb = self.vocab * self.hidden * (1 if self.tied_embeddings else 2)
        return self.num_layers * per_layer + emb + self.hidden

    def flops_per_token(self) -> float:
        """Model FLOPs per trained token (forward + backward, causal attention)."""
        dense = (self.qkv_dim * self.hidden + self.n_heads * self.head_dim * self.hidden + 3 * self.hidden * self.ffn)
        attn = 2 * self.n_heads * self.head_dim * self.seq_len / 2  # QK^T and PV, causal half
        return 6.0 * (self.num_layers * (dense + attn) + self.vocab * self.hidden)


PRESETS = {
    "llama3_1b": GPTConfig("llama3_1b", 16, 2048, 8192, 32, 8, 64, 128256, 2048, 500000.0, 1e-5, False, True),
    "llama3_1b_ref": GPTConfig("llama3_1b_ref", 16, 2048, 8192, 32, 8, 64, 64320, 2048, 500000.0, 1e-5, False, False),
    "qwen3_0.6b": GPTConfig("qwen3_0.6b", 28, 1024, 3072, 16, 8, 128, 151936, 4096, 1e6, 1e-6, True, True),
    "qwen3_1.7b": GPTConfig("qwen3_1.7b", 28, 2048, 6144, 16, 8, 128, 151936, 4096, 1e6, 1e-6, True, True),
    "llama3_8b": GPTConfig("llama3_8b", 32, 4096, 14336, 32, 8, 128, 128256, 4096, 500000.0, 1e-5, False, False),
    "llama_tiny": GPTConfig("llama_tiny", 4, 512, 2048, 8, 2, 64, 32000, 512, 500000.0, 1e-5, False, False),
    "test_tiny": GPTConfig("test_tiny", 2, 128, 256, 4, 2, 32, 512, 32, 10000.0, 1e-5, False, True),
    "test_tiny_qk": GPTConfig("test_tiny_qk", 2, 128, 256, 4, 2, 32, 512, 32, 10000.0, 1e-6, True, False),
}


def get_config(name: str, **overrides) -> GPTConfig:
    if name not in PRESETS:
        raise ValueError(f"unknown model '{name}' (known: {sorted(PRESETS)})")
    return replace(PRESETS[name], **overrides) if overrides else PRESETS[name]


def param_specs(cfg: GPTConfig) -> list:
    """Parameter specs in the order their gradients become final in the backward pass."""
    std = cfg.init_std
    specs = []
    if not cfg.tied_embeddings:
        specs.append(ParamSpec("output_layer.weight", (cfg.vocab, cfg.hidden), 0, "normal", std))
    specs.append(ParamSpec("decoder.final_layernorm.weight", (cfg.hidden,), 1, "ones", tp_duplicate=True))
    for i in reversed(range(cfg.num_layers)):
        p = f"decoder.layers.{i}."
        specs.append(ParamSpec(p + "mlp.linear_fc2.weight", (cfg.hidden, cfg.ffn), 0, "normal", std))
        specs.append(ParamSpec(p + "mlp.linear_fc1.weight", (2 * cfg.ffn, cfg.hidden), 0, "normal", std))
        specs.append(ParamSpec(p + "pre_mlp_layernorm.weight", (cfg.hidden,), 1, "ones", tp_duplicate=True))
        specs.append(ParamSpec(p + "self_attention.linear_proj.weight", (cfg.hidden, cfg.n_heads * cfg.head_dim), 0,
                               "normal", std))
        if cfg.qk_norm:
            specs.append(ParamSpec(p + "self_attention.k_layernorm.weight", (cfg.head_dim,), 1, "ones",
                                   tp_duplicate=True))
            specs.append(ParamSpec(p + "self_attention.q_layernorm.weight", (cfg.head_dim,), 1, "ones",
                                   tp_duplicate=True))
        specs.append(ParamSpec(p + "self_attention.linear_qkv.weight", (cfg.qkv_dim, cfg.hidden), 0, "normal", std))
        specs.append(ParamSpec(p + "input_layernorm.weight", (cfg.hidden,), 1, "ones", tp_duplicate=True))
    specs.append(ParamSpec("embedding.word_embeddings.weight", (cfg.vocab, cfg.hidden), 0, "normal", std))
    return specs


class GPT:
    def __init__(self, cfg: GPTConfig, *, device="cpu", pool=None, bucket_elems: int = 16 * 1024 * 1024,
                 seed: int = 0, need_comm_staging: bool = False, arena: Optional[FlatArena] = None):
        self.cfg = cfg
        self.device = torch.device(device)
        self.arena = arena if arena is not None else FlatArena(
            param_specs(cfg), bucket_elems=bucket_elems, device=device, pool=pool,
            need_comm_staging=need_comm_staging)
        if arena is None:
            self.arena.init_parameters(seed)
        self.cuda = self.device.type == "cuda"
        self._rope = None
        a = self.arena.by_name
        self.emb = a["embedding.word_embeddings.weight"]
        self.head = self.emb if cfg.tied_embeddings else a["output_layer.weight"]
        self.final_norm = a["decoder.final_layernorm.weight"]
        self.layers = []
        for i in range(cfg.num_layers):
            p = f"decoder.layers.{i}."
            self.layers.append(dict(
                ln1=a[p + "input_layernorm.weight"], qkv=a[p + "self_attention.linear_qkv.weight"],
                qn=a.get(p + "self_attention.q_layernorm.weight"), kn=a.get(p + "self_attention.k_layernorm.weight"),
                proj=a[p + "self_attention.linear_proj.weight"], ln2=a[p + "pre_mlp_layernorm.weight"],
                fc1=a[p + "mlp.linear_fc1.weight"], fc2=a[p + "mlp.linear_fc2.weight"]))
        self.launches = 0  # native kernel launches issued by the model (bench bookkeeping)

    def named_parameters(self):
        for s in self.arena.slots:
            yield s.name, s.model

    # --------------------------------------------------------------- GEMMs
    def _linear(self, x, slot, residual=None):
        """y = x @ W^T (+ residual). x: [T, in] bf16, W: [out, in]."""
        W = slot.model
        if self.cuda:
            from .. import kernels as K

            out = torch.empty(x.shape[0], W.shape[0], dtype=torch.bfloat16, device=x.device)
            self.launches += 1
            if residual is not None:
                return K.gemm_bf16(x, W, out, epi=K.EPI_BF16_ADD, residual=residual)
            return K.gemm_bf16(x, W, out)
        y = x.float() @ W.float().t()
        if residual is not None:
            y = y + residual.float()
        return y.to(torch.bfloat16)

    def _dgrad(self, dy, slot):
        """dx = dy @ W. dy: [T, out]."""
        W = slot.model
        if self.cuda:
            from .. import kernels as K

            out = torch.empty(dy.shape[0], W.shape[1], dtype=torch.bfloat16, device=dy.device)
            self.launches += 1
            return K.gemm_bf16(dy, W, out, b_mn=True)
        return (dy.float() @ W.float()).to(torch.bfloat16)

    def _wgrad(self, dy, x, slot):
        """main_grad(W) += dy^T @ x, accumulated in fp32 by the GEMM epilogue."""
        if self.cuda:
            from .. import kernels as K

            self.launches += 1
            K.gemm_bf16(dy, x, slot.grad, a_mn=True, b_mn=True, epi=K.EPI_F32_ACC)
        else:
            slot.grad += dy.float().t() @ x.float()

    def _rope_tables(self):
        if self._rope is None:
            self._rope = F.rope_tables(self.cfg.seq_len, self.cfg.head_dim, self.cfg.rope_theta, self.device)
        return self._rope

    # ------------------------------------------------------------ forward
    def _layer_fwd(self, L, x, B, S):
        c = self.cfg
        T = B * S
        cs, sn = self._rope_tables()
        h1, rstd1 = F.rmsnorm_fwd(x, L["ln1"].model, c.norm_eps)
        qkv = self._linear(h1, L["qkv"])
        del h1
        nq, nkv, hd = c.n_heads, c.n_kv_heads, c.head_dim
        qk_saved = None
        if c.qk_norm:
            pre = qkv[:, :(nq + nkv) * hd].clone()
            rq = F.headnorm_fwd_(qkv, L["qn"].model, c.norm_eps, T, nq, hd, 0)
            rk = F.headnorm_fwd_(qkv, L["kn"].model, c.norm_eps, T, nkv, hd, nq * hd)
            qk_saved = (pre, rq, rk)
            self.launches += 2
        F.rope_(qkv, cs, sn, S, nq + nkv, hd, 0, +1.0)
        ctx, att_saved = A.attn_fwd(qkv, B, S, nq, nkv, hd)
        x_mid = self._linear(ctx, L["proj"], residual=x)
        h2, rstd2 = F.rmsnorm_fwd(x_mid, L["ln2"].model, c.norm_eps)
        gu = self._linear(h2, L["fc1"])
        del h2
        s = F.swiglu_fwd(gu)
        x_out = self._linear(s, L["fc2"], residual=x_mid)
        del s
        self.launches += 5
        return x_out, (x, rstd1, qkv, qk_saved, ctx, att_saved, x_mid, rstd2, gu)

    def _layer_bwd(self, L, saved, dx, B, S, done):
        c = self.cfg
        T = B * S
        x, rstd1, qkv, qk_saved, ctx, att_saved, x_mid, rstd2, gu = saved
        nq, nkv, hd = c.n_heads, c.n_kv_heads, c.head_dim
        cs, sn = self._rope_tables()
        # MLP
        s = F.swiglu_fwd(gu)
        self._wgrad(dx, s, L["fc2"])
        done(L["fc2"])
        ds = self._dgrad(dx, L["fc2"])
        del s
        dgu = F.swiglu_bwd(gu, ds)
        del ds
        h2, _ = F.rmsnorm_fwd(x_mid, L["ln2"].model, c.norm_eps, want_rstd=False)
        self._wgrad(dgu, h2, L["fc1"])
        done(L["fc1"])
        del h2
        dh2 = self._dgrad(dgu, L["fc1"])
        del dgu
        # dx (the residual stream gradient) += norm backward, in place
        F.rmsnorm_bwd(x_mid, L["ln2"].model, dh2, rstd2, dw_out=L["ln2"].grad, dx_out=dx, accumulate_dx=True)
        done(L["ln2"])
        del dh2
        # attention
        self._wgrad(dx, ctx, L["proj"])
        done(L["proj"])
        dctx = self._dgrad(dx, L["proj"])
        dqkv = A.attn_bwd(dctx, qkv, att_saved, B, S, nq, nkv, hd)
        del dctx
        F.rope_(dqkv, cs, sn, S, nq + nkv, hd, 0, -1.0)
        if c.qk_norm:
            pre, rq, rk = qk_saved
            F.headnorm_bwd_(pre, dqkv, L["kn"].model, rk, L["kn"].grad, T, nkv, hd, nq * hd, nq * hd)
            F.headnorm_bwd_(pre, dqkv, L["qn"].model, rq, L["qn"].grad, T, nq, hd, 0, 0)
            done(L["kn"])
            done(L["qn"])
            self.launches += 4
        h1, _ = F.rmsnorm_fwd(x, L["ln1"].model, c.norm_eps, want_rstd=False)
        self._wgrad(dqkv, h1, L["qkv"])
        done(L["qkv"])
        del h1
        dh1 = self._dgrad(dqkv, L["qkv"])
        del dqkv
        F.rmsnorm_bwd(x, L["ln1"].model, dh1, rstd1, dw_out=L["ln1"].grad, dx_out=dx, accumulate_dx=True)
        done(L["ln1"])
        self.launches += 9
        return dx

    def forward_backward(self, tokens: torch.Tensor, targets: torch.Tensor, *, loss_scale: float = 1.0,
                         on_param_done: Optional[Callable] = None, backward: bool = True) -> torch.Tensor:
        """One micro-batch. ``tokens`` / ``targets``: ``[B, S]`` int64. Gradients of
        ``loss_scale * mean token loss`` are accumulated into ``main_grad``.
        Returns the (unscaled) mean loss as a 0-dim fp32 tensor on the device."""
        c = self.cfg
        B, S = tokens.shape
        T = B * S
        done = on_param_done if on_param_done is not None else (lambda slot: None)
        ids = tokens.reshape(-1)
        x = F.embed_fwd(ids, self.emb.model)
        saved = []
        for L in self.layers:
            x, sv = self._layer_fwd(L, x, B, S)
            saved.append(sv)
        hf, rstd_f = F.rmsnorm_fwd(x, self.final_norm.model, c.norm_eps)
        logits = self._linear(hf, self.head)
        self.launches += 3
        loss_tok = F.cross_entropy_(logits, targets.reshape(-1), grad_scale=loss_scale / T, write_grad=backward)
        loss = loss_tok.mean()
        if not backward:
            return loss
        dlogits = logits  # overwritten in place by the loss kernel
        self._wgrad(dlogits, hf, self.head)
        if not c.tied_embeddings:
            done(self.head)
        dhf = self._dgrad(dlogits, self.head)
        del logits, dlogits, hf
        dx = F.rmsnorm_bwd(x, self.final_norm.model, dhf, rstd_f, dw_out=self.final_norm.grad)
        done(self.final_norm)
        del dhf
        for L, sv in zip(reversed(self.layers), reversed(saved)):
            dx = self._layer_bwd(L, sv, dx, B, S, done)
        saved.clear()
        F.embed_bwd(ids, dx, self.emb.grad)
        done(self.emb)
        self.launches += 4
        return loss
