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
    # small models whose head dimensions take the native attention kernels (64 and 128; grouped queries)
    "test_hd64": GPTConfig("test_hd64", 2, 256, 512, 4, 2, 64, 512, 320, 500000.0, 1e-5, False, True),
    "test_hd128_qk": GPTConfig("test_hd128_qk", 2, 256, 512, 4, 2, 128, 512, 320, 1e6, 1e-6, True, False),
}


def get_config(name: str, **overrides) -> GPTConfig:
    if name not in PRESETS:
        raise ValueError(f"unknown model '{name}' (known: {sorted(PRESETS)})")
    return replace(PRESETS[name], **overrides) if overrides else PRESETS[name]


def _rows(*ranges):
    return [(0, lo, hi) for lo, hi in ranges]


def stage_layers(num_layers: int, pp_size: int, pp_rank: int) -> range:
    """Layers of pipeline stage ``pp_rank`` (contiguous, sizes differing by at most one)."""
    base, extra = divmod(num_layers, pp_size)
    lo = pp_rank * base + min(pp_rank, extra)
    return range(lo, lo + base + (1 if pp_rank < extra else 0))


def param_specs(cfg: GPTConfig, tp_size: int = 1, tp_rank: int = 0, pp_size: int = 1, pp_rank: int = 0,
                vocab_parallel: bool = False) -> list:
    """Parameter specs in the order their gradients become final in the backward pass.

    With ``pp_size > 1`` only the parameters of stage ``pp_rank`` are returned:
    its contiguous run of layers, the embedding on the first stage, the final
    norm and the output layer on the last (untied embeddings only).

    With ``tp_size > 1`` the linear weights are this rank's shard (QKV and the
    fused gate|up projection by output rows, per head group / per half; the
    output and down projections by input columns) and carry the slices of the
    full tensor they are cut from; norm weights, the embedding and the output
    layer are replicated (activations are sharded by rows, so each rank embeds
    and scores its own tokens against the full vocabulary). ``vocab_parallel``
    shards those two by vocabulary rows instead (``vocab % tp_size == 0``)."""
    std = cfg.init_std
    tp = tp_size
    nq, nkv, hd, F_, H = cfg.n_heads, cfg.n_kv_heads, cfg.head_dim, cfg.ffn, cfg.hidden
    if tp > 1:
        assert nq % tp == 0 and nkv % tp == 0 and F_ % tp == 0, "heads and ffn must divide over tensor-parallel ranks"
    dup = tp > 1
    r = tp_rank
    nql, nkvl, Fl = nq // tp, nkv // tp, F_ // tp

    def sharded(name, full_shape, pieces):
        if tp == 1:
            return ParamSpec(name, full_shape, 0, "normal", std)
        dim = pieces[0][0]
        shape = list(full_shape)
        shape[dim] = sum(hi - lo for _, lo, hi in pieces)
        return ParamSpec(name, tuple(shape), 0, "normal", std, tp_full_shape=tuple(full_shape), tp_pieces=pieces)

    vp = vocab_parallel and tp > 1
    if vp:
        assert cfg.vocab % tp == 0, "the vocabulary must divide over the tensor-parallel ranks"
    Vl = cfg.vocab // tp

    def vocab_rows(name):
        if vp:
            return sharded(name, (cfg.vocab, H), _rows((r * Vl, (r + 1) * Vl)))
        return ParamSpec(name, (cfg.vocab, H), 0, "normal", std, tp_duplicate=dup)

    specs = []
    if not cfg.tied_embeddings:
        specs.append(vocab_rows("output_layer.weight"))
    specs.append(ParamSpec("decoder.final_layernorm.weight", (H,), 1, "ones", tp_duplicate=True))
    for i in reversed(range(cfg.num_layers)):
        p = f"decoder.layers.{i}."
        specs.append(sharded(p + "mlp.linear_fc2.weight", (H, F_), [(1, r * Fl, (r + 1) * Fl)]))
        specs.append(sharded(p + "mlp.linear_fc1.weight", (2 * F_, H),
                             _rows((r * Fl, (r + 1) * Fl), (F_ + r * Fl, F_ + (r + 1) * Fl))))
        specs.append(ParamSpec(p + "pre_mlp_layernorm.weight", (H,), 1, "ones", tp_duplicate=True))
        specs.append(sharded(p + "self_attention.linear_proj.weight", (H, nq * hd),
                             [(1, r * nql * hd, (r + 1) * nql * hd)]))
        if cfg.qk_norm:
            specs.append(ParamSpec(p + "self_attention.k_layernorm.weight", (hd,), 1, "ones", tp_duplicate=True))
            specs.append(ParamSpec(p + "self_attention.q_layernorm.weight", (hd,), 1, "ones", tp_duplicate=True))
        ko, vo = nq * hd, (nq + nkv) * hd
        specs.append(sharded(p + "self_attention.linear_qkv.weight", (cfg.qkv_dim, H),
                             _rows((r * nql * hd, (r + 1) * nql * hd), (ko + r * nkvl * hd, ko + (r + 1) * nkvl * hd),
                                   (vo + r * nkvl * hd, vo + (r + 1) * nkvl * hd))))
        specs.append(ParamSpec(p + "input_layernorm.weight", (H,), 1, "ones", tp_duplicate=True))
    specs.append(vocab_rows("embedding.word_embeddings.weight"))
    if tp > 1 or pp_size > 1:
        for i, s in enumerate(specs):
            s.init_order = i  # every parameter keeps the random stream it has in the whole model
    if pp_size > 1:
        if cfg.tied_embeddings:
            raise ValueError("pipeline stages need untied embeddings (the two uses live on different stages)")
        mine = set(stage_layers(cfg.num_layers, pp_size, pp_rank))
        first, last = pp_rank == 0, pp_rank == pp_size - 1

        def keep(name: str) -> bool:
            if name.startswith("decoder.layers."):
                return int(name.split(".")[2]) in mine
            if name.startswith("embedding."):
                return first
            return last  # final norm, output layer

        specs = [s for s in specs if keep(s.name)]
    if tp > 1:
        # shards first, replicated parameters after them (each kind keeps its backward order), so that
        # buckets never mix the two; bucket synchronisation is not overlapped under tensor parallelism
        specs = [s for s in specs if not s.tp_duplicate] + [s for s in specs if s.tp_duplicate]
    return specs


class GPT:
    def __init__(self, cfg: GPTConfig, *, device="cpu", pool=None, bucket_elems: int = 16 * 1024 * 1024,
                 seed: int = 0, need_comm_staging: bool = False, arena: Optional[FlatArena] = None, tp=None,
                 init_on_device: bool = False, pp_size: int = 1, pp_rank: int = 0, recompute: bool = False,
                 vocab_parallel: bool = False):
        self.cfg = cfg
        # False: the normalised inputs of the two column-parallel linears and the SwiGLU output are kept
        # for the backward pass (about 0.2 GB per layer at 8192 tokens; HBM is not the scarce resource);
        # True: they are recomputed from what the backward pass holds anyway
        self.recompute = recompute
        self.device = torch.device(device)
        self.tp = tp if (tp is not None and tp.world > 1) else None
        self.tp_size = self.tp.world if self.tp is not None else 1
        self.pp_size, self.pp_rank = pp_size, pp_rank
        self.first_stage, self.last_stage = pp_rank == 0, pp_rank == pp_size - 1
        self.layer_ids = stage_layers(cfg.num_layers, pp_size, pp_rank)
        # Under tensor parallelism the embedding and the output layer are replicated by default (each rank
        # embeds and scores its own rows); vocab_parallel shards both by vocabulary rows: 1 / tp of their
        # parameters, gradients and optimizer state per rank, for two library collectives per micro-batch.
        self.vocab_parallel = bool(vocab_parallel) and self.tp is not None
        self.arena = arena if arena is not None else FlatArena(
            param_specs(cfg, self.tp_size, self.tp.rank if self.tp is not None else 0, pp_size, pp_rank,
                        vocab_parallel=self.vocab_parallel),
            bucket_elems=bucket_elems, device=device, pool=pool, need_comm_staging=need_comm_staging,
            split_on_tp_duplicate=self.tp_size > 1)
        if arena is None:
            self.arena.init_parameters(seed, on_device=init_on_device)
        self.cuda = self.device.type == "cuda"
        self._rope = None
        a = self.arena.by_name
        self.emb = a.get("embedding.word_embeddings.weight")
        self.head = self.emb if cfg.tied_embeddings else a.get("output_layer.weight")
        self.final_norm = a.get("decoder.final_layernorm.weight")
        self.layers = []
        for i in self.layer_ids:
            p = f"decoder.layers.{i}."
            self.layers.append(dict(
                ln1=a[p + "input_layernorm.weight"], qkv=a[p + "self_attention.linear_qkv.weight"],
                qn=a.get(p + "self_attention.q_layernorm.weight"), kn=a.get(p + "self_attention.k_layernorm.weight"),
                proj=a[p + "self_attention.linear_proj.weight"], ln2=a[p + "pre_mlp_layernorm.weight"],
                fc1=a[p + "mlp.linear_fc1.weight"], fc2=a[p + "mlp.linear_fc2.weight"]))
        self.launches = 0  # native kernel launches issued by the model (bench bookkeeping)
        # Under tensor parallelism the gradient of a replicated parameter is summed over the group. main_grad
        # also carries the residual of earlier steps, which every rank already holds in full, so the step's
        # new gradient is accumulated in a staging buffer, summed there, and only then added to main_grad.
        self._stage = {}
        if self.tp is not None:
            dup = [sl for sl in self.arena.slots if sl.spec.tp_duplicate]
            if dup:
                lo, hi = min(sl.start for sl in dup), max(sl.end for sl in dup)
                self._stage_buf = torch.zeros(hi - lo, dtype=torch.float32, device=self.device)
                for sl in dup:
                    self._stage[id(sl)] = self._stage_buf[sl.start - lo:sl.end - lo].view(sl.spec.shape)

    def named_parameters(self):
        for s in self.arena.slots:
            yield s.name, s.model

    def _gbuf(self, slot):
        """Where this step's gradient of ``slot`` is accumulated."""
        return self._stage.get(id(slot), slot.grad)

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
            K.gemm_bf16(dy, x, self._gbuf(slot), a_mn=True, b_mn=True, epi=K.EPI_F32_ACC)
        else:
            self._gbuf(slot).add_(dy.float().t() @ x.float())

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
        if self.recompute:
            h1 = None
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
        s = F.swiglu_fwd(gu)
        x_out = self._linear(s, L["fc2"], residual=x_mid)
        if self.recompute:
            h2 = s = None
        self.launches += 5
        return x_out, (x, rstd1, qkv, qk_saved, ctx, att_saved, x_mid, rstd2, gu, h1, h2, s)

    def _layer_bwd(self, L, saved, dx, B, S, done):
        c = self.cfg
        T = B * S
        x, rstd1, qkv, qk_saved, ctx, att_saved, x_mid, rstd2, gu, h1, h2, s = saved
        nq, nkv, hd = c.n_heads, c.n_kv_heads, c.head_dim
        cs, sn = self._rope_tables()
        # MLP
        if s is None:
            s = F.swiglu_fwd(gu)
        self._wgrad(dx, s, L["fc2"])
        done(L["fc2"])
        ds = self._dgrad(dx, L["fc2"])
        del s
        dgu = F.swiglu_bwd(gu, ds)
        del ds
        if h2 is None:
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
        if h1 is None:
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

    # ------------------------------------------------- tensor-parallel layers
    # Activations between the linears are [T / tp, hidden] (this rank's rows); the
    # column-parallel linears (QKV, gate|up) gather their input rows inside the GEMM
    # kernel, the row-parallel ones (output, down) reduce-scatter their output rows
    # inside it. The gathered inputs are kept for the weight gradients.
    def _layer_fwd_tp(self, i, L, x, B, S, inflight=0):
        # The gathered inputs of the two column-parallel linears stay in per-layer symmetric buffers for
        # the backward pass. A pipeline stage holds several micro-batches between their forward and their
        # backward, so the buffers are also keyed by the micro-batch's in-flight slot.
        c, tp = self.cfg, self.tp
        T = B * S
        cs, sn = self._rope_tables()
        nq, nkv, hd = c.n_heads // tp.world, c.n_kv_heads // tp.world, c.head_dim
        g1 = tp.slot(("h1", i, inflight), T, c.hidden)
        _, rstd1 = F.rmsnorm_fwd(x, L["ln1"].model, c.norm_eps, out=g1.local)
        qkv = tp.ag_linear(g1, L["qkv"].model)
        qk_saved = None
        if c.qk_norm:
            pre = qkv[:, :(nq + nkv) * hd].clone()
            rq = F.headnorm_fwd_(qkv, L["qn"].model, c.norm_eps, T, nq, hd, 0)
            rk = F.headnorm_fwd_(qkv, L["kn"].model, c.norm_eps, T, nkv, hd, nq * hd)
            qk_saved = (pre, rq, rk)
            self.launches += 2
        F.rope_(qkv, cs, sn, S, nq + nkv, hd, 0, +1.0)
        ctx, att_saved = A.attn_fwd(qkv, B, S, nq, nkv, hd)
        x_mid = tp.linear_rs(ctx, L["proj"].model, residual=x)
        g2 = tp.slot(("h2", i, inflight), T, c.hidden)
        _, rstd2 = F.rmsnorm_fwd(x_mid, L["ln2"].model, c.norm_eps, out=g2.local)
        gu = tp.ag_linear(g2, L["fc1"].model)
        s = F.swiglu_fwd(gu)
        x_out = tp.linear_rs(s, L["fc2"].model, residual=x_mid)
        if self.recompute:
            s = None
        self.launches += 5
        return x_out, (x, rstd1, qkv, qk_saved, ctx, att_saved, x_mid, rstd2, gu, g1, g2, s)

    def _layer_bwd_tp(self, L, saved, gdx, B, S, done):
        c, tp = self.cfg, self.tp
        T = B * S
        x, rstd1, qkv, qk_saved, ctx, att_saved, x_mid, rstd2, gu, g1, g2, s = saved
        nq, nkv, hd = c.n_heads // tp.world, c.n_kv_heads // tp.world, c.head_dim
        cs, sn = self._rope_tables()
        dx = gdx.local
        # MLP: the down projection's input gradient gathers dx rows; gdx.full then feeds its weight gradient
        if s is None:
            s = F.swiglu_fwd(gu)
        ds = tp.ag_linear(gdx, L["fc2"].model, b_mn=True)
        self._wgrad(gdx.full, s, L["fc2"])
        done(L["fc2"])
        del s
        dgu = F.swiglu_bwd(gu, ds)
        del ds
        self._wgrad(dgu, g2.full, L["fc1"])
        done(L["fc1"])
        dh2 = tp.linear_rs(dgu, L["fc1"].model, b_mn=True)
        del dgu
        F.rmsnorm_bwd(x_mid, L["ln2"].model, dh2, rstd2, dw_out=self._gbuf(L["ln2"]), dx_out=dx, accumulate_dx=True)
        done(L["ln2"])
        del dh2
        # attention
        dctx = tp.ag_linear(gdx, L["proj"].model, b_mn=True)
        self._wgrad(gdx.full, ctx, L["proj"])
        done(L["proj"])
        dqkv = A.attn_bwd(dctx, qkv, att_saved, B, S, nq, nkv, hd)
        del dctx
        F.rope_(dqkv, cs, sn, S, nq + nkv, hd, 0, -1.0)
        if c.qk_norm:
            pre, rq, rk = qk_saved
            F.headnorm_bwd_(pre, dqkv, L["kn"].model, rk, self._gbuf(L["kn"]), T, nkv, hd, nq * hd, nq * hd)
            F.headnorm_bwd_(pre, dqkv, L["qn"].model, rq, self._gbuf(L["qn"]), T, nq, hd, 0, 0)
            done(L["kn"])
            done(L["qn"])
            self.launches += 4
        self._wgrad(dqkv, g1.full, L["qkv"])
        done(L["qkv"])
        dh1 = tp.linear_rs(dqkv, L["qkv"].model, b_mn=True)
        del dqkv
        F.rmsnorm_bwd(x, L["ln1"].model, dh1, rstd1, dw_out=self._gbuf(L["ln1"]), dx_out=dx, accumulate_dx=True)
        done(L["ln1"])
        self.launches += 7

    def _forward_backward_tp(self, tokens, targets, loss_scale, on_param_done, backward, reduce_replicated):
        loss, ctx = self._stage_forward_tp(tokens, targets, None, loss_scale, backward, 0)
        if backward:
            self._stage_backward_tp(ctx, None, on_param_done, reduce_replicated)
        return loss

    # One micro-batch through this stage's layers under tensor parallelism. Activations are sharded by rows
    # (sequence parallel), so what travels between stages is this rank's [T / tp, hidden] block: rank t of a
    # stage talks to rank t of its neighbours.
    def _stage_forward_tp(self, tokens, targets, x_in, loss_scale, write_grad, inflight):
        c, tp = self.cfg, self.tp
        B, S = tokens.shape
        T = B * S
        Tl = T // tp.world
        lo = tp.rank * Tl
        ids = vp_rows = None
        if self.first_stage and self.vocab_parallel:
            # every rank looks up the tokens of the whole micro-batch that fall into its vocabulary rows
            # (zeros elsewhere); the sum over the ranks, scattered by rows, is the sequence-parallel input
            Vl = c.vocab // tp.world
            all_ids = tokens.reshape(-1)
            mine = (all_ids >= tp.rank * Vl) & (all_ids < (tp.rank + 1) * Vl)
            vp_rows = torch.nonzero(mine).view(-1)
            ids = all_ids[vp_rows] - tp.rank * Vl
            part = torch.zeros(T, c.hidden, dtype=torch.bfloat16, device=self.device)
            if vp_rows.numel():
                part[vp_rows] = F.embed_fwd(ids, self.emb.model)
            x = tp.reduce_scatter_rows(part)
            del part
        elif self.first_stage:
            ids = tokens.reshape(-1)[lo:lo + Tl]
            x = F.embed_fwd(ids, self.emb.model)
        else:
            x = x_in
        saved = []
        for i, L in enumerate(self.layers):
            x, sv = self._layer_fwd_tp(i, L, x, B, S, inflight)
            saved.append(sv)
        self.launches += 1
        if not self.last_stage:
            return x, dict(B=B, S=S, ids=ids, vp_rows=vp_rows, saved=saved)
        if self.vocab_parallel:
            # the output layer holds 1 / tp of the vocabulary: gather the normalised rows, score every token
            # against the local rows, and combine the softmax statistics over the ranks
            gh = tp.slot(("hf", inflight), T, c.hidden)
            _, rstd_f = F.rmsnorm_fwd(x, self.final_norm.model, c.norm_eps, out=gh.local)
            hf = tp.gather(gh)
            logits = self._linear(hf, self.head)
            self.launches += 2
            loss_tok = self._vocab_parallel_ce_(logits, targets.reshape(-1), loss_scale / T, write_grad)
            loss = loss_tok.sum() / T   # every rank holds every token's loss
        else:
            tgt = targets.reshape(-1)[lo:lo + Tl]
            hf, rstd_f = F.rmsnorm_fwd(x, self.final_norm.model, c.norm_eps)
            logits = self._linear(hf, self.head)
            self.launches += 2
            loss_tok = F.cross_entropy_(logits, tgt, grad_scale=loss_scale / T, write_grad=write_grad)
            loss = tp.allreduce_scalar(loss_tok.sum() / T)
        return loss, dict(B=B, S=S, ids=ids, vp_rows=vp_rows, saved=saved, x=x, hf=hf, rstd_f=rstd_f, dlogits=logits)

    def _vocab_parallel_ce_(self, logits, targets, grad_scale, write_grad):
        """Cross-entropy over a vocabulary whose columns are sharded over the tensor-parallel ranks:
        ``logits`` is ``[T, vocab / tp]`` for all ``T`` tokens. Row maximum, sum of exponentials and the
        target's logit are combined over the ranks; ``logits`` is overwritten by its gradient. Returns the
        per-token loss (fp32, the same on every rank)."""
        tp = self.tp
        Vl = logits.shape[1]
        lo = tp.rank * Vl
        z = logits.float()
        m = z.max(1).values
        tp.allreduce_(m, torch.distributed.ReduceOp.MAX)
        e = torch.exp(z - m[:, None])
        ssum = e.sum(1)
        tp.allreduce_(ssum)
        local = (targets >= lo) & (targets < lo + Vl)
        col = (targets - lo).clamp(0, Vl - 1)
        zt = torch.where(local, z.gather(1, col[:, None]).squeeze(1), torch.zeros_like(m))
        tp.allreduce_(zt)
        loss = torch.log(ssum) + m - zt
        if write_grad:
            e /= ssum[:, None]
            rows = torch.nonzero(local).view(-1)
            e[rows, col[rows]] -= 1.0
            logits.copy_((e * grad_scale).to(logits.dtype))
        return loss

    def _stage_backward_tp(self, ctx, dx_out, on_param_done, reduce_replicated):
        c, tp = self.cfg, self.tp
        B, S, saved = ctx["B"], ctx["S"], ctx["saved"]
        T = B * S
        user_done = on_param_done if on_param_done is not None else (lambda slot: None)

        def done(slot):
            # a replicated parameter's gradient is final only once summed over the tensor-parallel ranks
            st = self._stage.get(id(slot))
            if st is not None:
                if not reduce_replicated:
                    return  # keeps accumulating in the staging buffer until the step's last micro-batch
                tp.allreduce_replicated(st)
                slot.grad.add_(st)
                st.zero_()
            user_done(slot)

        gdx = tp.slot("dx", T, c.hidden)
        if self.last_stage:
            dlogits, hf = ctx.pop("dlogits"), ctx.pop("hf")
            self._wgrad(dlogits, hf, self.head)
            if not c.tied_embeddings:
                done(self.head)
            dhf = self._dgrad(dlogits, self.head)
            del dlogits, hf
            if self.vocab_parallel:
                dhf = tp.reduce_scatter_rows(dhf)  # every rank's vocabulary rows contribute to every token
            F.rmsnorm_bwd(ctx.pop("x"), self.final_norm.model, dhf, ctx.pop("rstd_f"),
                          dw_out=self._gbuf(self.final_norm), dx_out=gdx.local)
            done(self.final_norm)
            del dhf
            self.launches += 3
        else:
            gdx.local.copy_(dx_out)
        for L, sv in zip(reversed(self.layers), reversed(saved)):
            self._layer_bwd_tp(L, sv, gdx, B, S, done)
        saved.clear()
        if self.first_stage:
            if self.vocab_parallel:
                rows = ctx["vp_rows"]
                if rows.numel():
                    F.embed_bwd(ctx["ids"], tp.gather(gdx)[rows].contiguous(), self._gbuf(self.emb))
                else:
                    tp.gather(gdx)  # the collective is the group's
            else:
                F.embed_bwd(ctx["ids"], gdx.local, self._gbuf(self.emb))
            done(self.emb)
            self.launches += 1
            return None
        return gdx.local.clone()  # the buffer is the next backward pass's too

    def forward_backward(self, tokens: torch.Tensor, targets: torch.Tensor, *, loss_scale: float = 1.0,
                         on_param_done: Optional[Callable] = None, backward: bool = True,
                         reduce_replicated: bool = True) -> torch.Tensor:
        """One micro-batch. ``tokens`` / ``targets``: ``[B, S]`` int64. Gradients of
        ``loss_scale * mean token loss`` are accumulated into ``main_grad``.
        Returns the (unscaled) mean loss as a 0-dim fp32 tensor on the device.
        Under tensor parallelism every rank of the group passes the same batch;
        ``reduce_replicated`` (set it on the last micro-batch of a step) sums the
        gradients of replicated parameters over the group as they become final."""
        if self.tp is not None:
            return self._forward_backward_tp(tokens, targets, loss_scale, on_param_done, backward,
                                             reduce_replicated)
        loss, ctx = self.stage_forward(tokens, targets, None, loss_scale=loss_scale, write_grad=backward)
        if backward:
            self.stage_backward(ctx, None, on_param_done)
        return loss

    # ------------------------------------------------------- pipeline stages
    # One micro-batch through this stage's layers. The first stage embeds ``tokens``; later stages take
    # the previous stage's activation ``x_in`` ``[T, hidden]``. The last stage computes the loss (and,
    # in the same kernel, the logit gradient); earlier stages return the activation to send on.
    def stage_forward(self, tokens, targets, x_in, *, loss_scale: float = 1.0, write_grad: bool = True,
                      inflight: int = 0):
        """``inflight``: which of the stage's in-flight micro-batch slots this pass uses (only tensor
        parallelism keeps per-slot buffers between a forward and its backward)."""
        if self.tp is not None:
            return self._stage_forward_tp(tokens, targets, x_in, loss_scale, write_grad, inflight)
        c = self.cfg
        B, S = tokens.shape
        T = B * S
        ids = tokens.reshape(-1) if self.first_stage else None
        x = F.embed_fwd(ids, self.emb.model) if self.first_stage else x_in
        saved = []
        for L in self.layers:
            x, sv = self._layer_fwd(L, x, B, S)
            saved.append(sv)
        self.launches += 1
        if not self.last_stage:
            return x, dict(B=B, S=S, ids=ids, saved=saved)
        hf, rstd_f = F.rmsnorm_fwd(x, self.final_norm.model, c.norm_eps)
        logits = self._linear(hf, self.head)
        self.launches += 2
        loss_tok = F.cross_entropy_(logits, targets.reshape(-1), grad_scale=loss_scale / T, write_grad=write_grad)
        # logits now holds the logit gradient (the loss kernel overwrites it in place)
        return loss_tok.mean(), dict(B=B, S=S, ids=ids, saved=saved, x=x, hf=hf, rstd_f=rstd_f, dlogits=logits)

    def stage_backward(self, ctx, dx_out, on_param_done: Optional[Callable] = None):
        """Backward of one micro-batch through this stage. ``dx_out`` is the gradient of the stage's
        output received from the next stage (``None`` on the last stage); returns the gradient of the
        stage's input (``None`` on the first stage). Under tensor parallelism the pass that is given
        ``on_param_done`` (the step's last) also sums the replicated parameters' gradients over the group."""
        if self.tp is not None:
            return self._stage_backward_tp(ctx, dx_out, on_param_done, on_param_done is not None)
        c = self.cfg
        done = on_param_done if on_param_done is not None else (lambda slot: None)
        B, S, saved = ctx["B"], ctx["S"], ctx["saved"]
        if self.last_stage:
            dlogits, hf = ctx.pop("dlogits"), ctx.pop("hf")
            self._wgrad(dlogits, hf, self.head)
            if not c.tied_embeddings:
                done(self.head)
            dhf = self._dgrad(dlogits, self.head)
            del dlogits, hf
            dx = F.rmsnorm_bwd(ctx.pop("x"), self.final_norm.model, dhf, ctx.pop("rstd_f"),
                               dw_out=self.final_norm.grad)
            done(self.final_norm)
            del dhf
            self.launches += 3
        else:
            dx = dx_out
        for L, sv in zip(reversed(self.layers), reversed(saved)):
            dx = self._layer_bwd(L, sv, dx, B, S, done)
        saved.clear()
        if self.first_stage:
            F.embed_bwd(ctx["ids"], dx, self.emb.grad)
            done(self.emb)
            self.launches += 1
            return None
        return dx
