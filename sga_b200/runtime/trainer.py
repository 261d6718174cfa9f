"""Training driver: model + data-parallel layer + optimizer + (optional) SGA
engine, one process per GPU.

``Trainer.train_step(batch)`` is the public per-step call: it splits the
rank's batch into micro-batches, runs forward/backward for each (arming
per-bucket gradient synchronisation for the last one so that communication
overlaps the backward pass), synchronises, clips, steps the optimizer and
returns the mean loss as a device scalar.

Three step flavours:

* SGA on: ``engine.grad_sync`` + ``engine.optimizer_step`` (full or sparse by
  the calendar).
* SGA off, ``dense_mode=fused``: per-bucket reduce-scatter kernels overlapped
  with the backward pass, then one kernel that runs AdamW on the slices this
  rank owns and all-gathers the bf16 parameters through peer stores.
* SGA off, ``dense_mode=allreduce`` (also the library baseline): bucket
  all-reduce, multi-tensor AdamW on the replicated state.

This is the counterpart of the reference's training entry + Megatron
``pretrain`` loop (``sga/train_gpt.py:212-252``); data is synthetic (uniform
token ids from a seed) because the headline benchmark is defined on it.
"""
from __future__ import annotations

import argparse
import os
import time
from typing import Optional

import torch
import torch.distributed as dist

from .. import config as C
from ..models.gpt import GPT, get_config
from ..plugins.optimizer import OptContext
from .builder import build_engine
from .ddp import DataParallel, DDPConfig
from .optimizer import FlatOptimizer, OptimizerConfig


def add_trainer_args(p: argparse.ArgumentParser) -> argparse.ArgumentParser:
    g = p.add_argument_group("training")
    g.add_argument("--model", type=str, default="llama3_1b")
    g.add_argument("--seq-length", type=int, default=None)
    g.add_argument("--num-layers", type=int, default=None)
    # architecture overrides on top of the --model preset, in the vocabulary of the reference's yamls
    g.add_argument("--hidden-size", type=int, default=None)
    g.add_argument("--ffn-hidden-size", type=int, default=None)
    g.add_argument("--num-attention-heads", type=int, default=None)
    g.add_argument("--num-query-groups", type=int, default=None, help="key/value heads (grouped-query attention)")
    g.add_argument("--kv-channels", type=int, default=None, help="head dimension (default hidden / heads)")
    g.add_argument("--padded-vocab-size", type=int, default=None)
    g.add_argument("--rotary-base", type=float, default=None)
    g.add_argument("--norm-epsilon", type=float, default=None)
    g.add_argument("--init-method-std", type=float, default=None)
    g.add_argument("--qk-layernorm", action="store_true", help="RMSNorm on the per-head queries and keys")
    g.add_argument("--micro-batch-size", type=int, default=4)
    g.add_argument("--global-batch-size", type=int, default=256)
    g.add_argument("--train-iters", type=int, default=10)
    g.add_argument("--lr", type=float, default=3e-4)
    g.add_argument("--min-lr", type=float, default=0.0)
    g.add_argument("--lr-decay-style", choices=("constant", "linear", "cosine"), default="constant")
    g.add_argument("--lr-warmup-iters", type=int, default=0)
    g.add_argument("--lr-warmup-fraction", type=float, default=None,
                   help="warm-up length as a fraction of --lr-decay-iters (instead of --lr-warmup-iters)")
    g.add_argument("--lr-warmup-init", type=float, default=0.0)
    g.add_argument("--exit-interval", type=int, default=0,
                   help="stop (after saving, with --save) when the iteration count is a multiple of this")
    g.add_argument("--lr-decay-iters", type=int, default=None, help="default: --train-iters")
    g.add_argument("--weight-decay", type=float, default=0.1)
    g.add_argument("--adam-beta1", type=float, default=0.9)
    g.add_argument("--adam-beta2", type=float, default=0.95)
    g.add_argument("--adam-eps", type=float, default=1e-8)
    g.add_argument("--clip-grad", type=float, default=1.0)
    g.add_argument("--seed", type=int, default=1234)
    g.add_argument("--data-seed", type=int, default=1234)
    g.add_argument("--data-path", default=None,
                   help="pre-tokenised corpus: PREFIX of an indexed-dataset .bin/.idx pair, or a flat token file; "
                        "default: synthetic uniform token ids")
    g.add_argument("--data-dtype", choices=("uint16", "int32", "uint32", "int64"), default=None,
                   help="token dtype of a flat --data-path file (read from the .idx header when there is one)")
    g.add_argument("--eval-interval", type=int, default=0, help="validation loss every N iterations (0: never)")
    g.add_argument("--eval-iters", type=int, default=10, help="global batches per validation pass")
    g.add_argument("--eval-data-path", default=None,
                   help="held-out corpus (same forms as --data-path); default: synthetic ids from another seed, or "
                        "another window order of --data-path")
    g.add_argument("--log-interval", type=int, default=1)
    g.add_argument("--save", type=str, default=None)
    g.add_argument("--load", type=str, default=None)
    g.add_argument("--save-interval", type=int, default=0)
    g.add_argument("--device", type=str, default=None)
    g.add_argument("--dense-mode", type=str, default="fused", choices=("fused", "allreduce"))
    g.add_argument("--transport", type=str, default="auto", choices=("auto", "p2p", "nccl", "gloo", "local"))
    g.add_argument("--overlap-grad-reduce", type=C.sga_bool, default=True)
    g.add_argument("--comm-max-ctas", type=int, default=0)
    g.add_argument("--tensor-model-parallel-size", type=int, default=1)
    g.add_argument("--recompute-activations", action="store_true",
                   help="recompute the norm outputs and the SwiGLU output in the backward pass instead of keeping them")
    g.add_argument("--init-on-device", action="store_true",
                   help="draw the initial weights with the device generator (large models)")
    g.add_argument("--tp-comm", type=str, default="auto", choices=("auto", "fused", "library"),
                   help="tensor-parallel linears: collective fused into the GEMM kernel, or library collectives")
    g.add_argument("--nvls-dense", action="store_true",
                   help="dense gradient all-reduce through the NVSwitch's in-switch reduction (multimem): the "
                        "gradient arena is allocated as torch.distributed symmetric memory bound to a multicast "
                        "object; buffers without multicast support keep the peer-load kernels")
    g.add_argument("--vocab-parallel-embedding", action="store_true",
                   help="under tensor parallelism shard the embedding and the output layer by vocabulary rows "
                        "instead of replicating them (two library collectives per micro-batch)")
    g.add_argument("--pipeline-model-parallel-size", type=int, default=1)
    g.add_argument("--sequence-parallel", action="store_true")
    g.add_argument("--untie-embeddings-and-output-weights", action="store_true")
    g.add_argument("--use-distributed-optimizer", action="store_true")
    g.add_argument("--log-num-zeros-in-grad", action="store_true")
    g.add_argument("--sga-allow-config-override", action="store_true")
    g.add_argument("--save-sga-state", action="store_true",
                   help="checkpoints also hold every rank's residual, the active support and the engine's counters, "
                        "and a resume continues bit for bit instead of cold-starting the cycle")
    # Flags of the training stack the reference's yamls are written for. This trainer has one choice for each
    # (bf16 compute with fp32 master weights and gradients, bias-free linears, RMSNorm, rotary positions, SwiGLU,
    # its own attention kernels, no dropout, pre-tokenised data): the flags are accepted so that such a yaml
    # launches unchanged, and a value this trainer cannot honour is refused by check_compat_flags.
    c = p.add_argument_group("accepted for yaml compatibility")
    for flag in ("--disable-bias-linear", "--use-flash-attn", "--bf16", "--attention-softmax-in-fp32",
                 "--accumulate-allreduce-grads-in-fp32", "--log-throughput", "--log-params-norm",
                 "--group-query-attention", "--use-rotary-position-embeddings", "--swiglu"):
        c.add_argument(flag, action="store_true")
    c.add_argument("--rerun-mode", default=None)
    c.add_argument("--data-parallel-sharding-strategy", default=None)
    c.add_argument("--timing-log-level", type=int, default=None)
    c.add_argument("--transformer-impl", default=None)
    c.add_argument("--max-position-embeddings", type=int, default=None)
    c.add_argument("--normalization", default=None)
    c.add_argument("--position-embedding-type", default=None)
    c.add_argument("--attention-dropout", type=float, default=None)
    c.add_argument("--hidden-dropout", type=float, default=None)
    c.add_argument("--split", default=None)
    c.add_argument("--tokenizer-type", default=None)
    c.add_argument("--tokenizer-model", default=None)
    c.add_argument("--make-vocab-size-divisible-by", type=int, default=None)
    c.add_argument("--tensorboard-dir", default=None)
    c.add_argument("--wandb-save-dir", default=None)
    return p


def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser("sga_b200 trainer", allow_abbrev=False)
    add_trainer_args(p)
    C.add_sga_args(p)
    return p


def init_distributed(device_type: str):
    """One process per GPU; rendezvous from the torchrun environment."""
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world > 1 and not dist.is_initialized():
        backend = "nccl" if device_type == "cuda" else "gloo"
        kwargs = {}
        if device_type == "cuda":
            local = int(os.environ.get("LOCAL_RANK", "0"))
            torch.cuda.set_device(local)
            kwargs["device_id"] = torch.device("cuda", local)
        dist.init_process_group(backend=backend, **kwargs)
    rank = dist.get_rank() if dist.is_initialized() else 0
    return rank, (dist.get_world_size() if dist.is_initialized() else 1)


def check_compat_flags(args) -> None:
    """Refuses the values of the compatibility flags that would mean another model or another numerics."""
    bad = []
    if args.normalization not in (None, "RMSNorm"):
        bad.append(f"--normalization {args.normalization} (RMSNorm only)")
    if args.position_embedding_type not in (None, "rope"):
        bad.append(f"--position-embedding-type {args.position_embedding_type} (rope only)")
    for name in ("attention_dropout", "hidden_dropout"):
        if getattr(args, name) not in (None, 0.0):
            bad.append(f"--{name.replace('_', '-')} {getattr(args, name)} (no dropout)")
    if args.data_parallel_sharding_strategy not in (None, "no_shard"):
        bad.append(f"--data-parallel-sharding-strategy {args.data_parallel_sharding_strategy} (no_shard only)")
    if args.max_position_embeddings is not None and args.seq_length and args.max_position_embeddings < args.seq_length:
        bad.append(f"--max-position-embeddings {args.max_position_embeddings} < --seq-length {args.seq_length}")
    if bad:
        raise ValueError("not supported by this trainer: " + "; ".join(bad))


def scheduled_lr(args, done: int) -> float:
    """Learning rate of the step that follows ``done`` completed iterations: linear warm-up from
    ``--lr-warmup-init`` over ``--lr-warmup-iters``, then constant, linear or cosine decay to ``--min-lr`` at
    ``--lr-decay-iters`` (the schedule of the training stack the reference's yamls are written for:
    ``lr_decay_style`` / ``lr_warmup_iters`` / ``min_lr`` in ``examples/llama3/*.yaml`` there)."""
    import math

    max_lr, min_lr = float(args.lr), float(getattr(args, "min_lr", 0.0) or 0.0)
    decay = int(getattr(args, "lr_decay_iters", None) or args.train_iters)
    warm = int(getattr(args, "lr_warmup_iters", 0) or 0)
    frac = getattr(args, "lr_warmup_fraction", None)
    if frac is not None:
        if warm:
            raise ValueError("give --lr-warmup-iters or --lr-warmup-fraction, not both")
        warm = int(float(frac) * decay)
    if warm > 0 and done <= warm:
        init = float(getattr(args, "lr_warmup_init", 0.0) or 0.0)
        return init + (max_lr - init) * done / warm
    style = getattr(args, "lr_decay_style", "constant")
    if style == "constant":
        return max_lr
    if done > decay:
        return min_lr
    ratio = (done - warm) / max(decay - warm, 1)
    coeff = (1.0 - ratio) if style == "linear" else 0.5 * (math.cos(math.pi * ratio) + 1.0)
    return min_lr + coeff * (max_lr - min_lr)


class SyntheticTokens:
    """Uniform token ids over the vocabulary from a seed; each (step, rank,
    micro-batch) draws its own stream so that every rank sees different data
    and a given global batch is the same whatever the number of ranks."""

    def __init__(self, vocab: int, seq_len: int, seed: int, pin: bool = False):
        self.vocab, self.seq_len, self.seed = vocab, seq_len, seed
        self.pin = pin

    def batch(self, step: int, first_sample: int, n: int):
        """``n`` sequences starting at global sample index ``first_sample`` of ``step``."""
        out = torch.empty(n, self.seq_len + 1, dtype=torch.int64, pin_memory=self.pin)
        for i in range(n):
            g = torch.Generator().manual_seed((self.seed * 1000003 + step) * 1000003 + first_sample + i)
            out[i] = torch.randint(0, self.vocab, (self.seq_len + 1,), generator=g)
        return out


class _nvtx:
    """NVTX range around a phase of the step when ``SGA_NVTX=1`` (the launcher's profiler prefix captures
    ``nvtx,cuda,osrt``); a no-op otherwise."""

    on = os.environ.get("SGA_NVTX", "0") == "1"

    def __init__(self, name: str):
        self.name = name

    def __enter__(self):
        if self.on and torch.cuda.is_available():
            torch.cuda.nvtx.range_push(self.name)
        return self

    def __exit__(self, *exc):
        if self.on and torch.cuda.is_available():
            torch.cuda.nvtx.range_pop()
        return False


class Trainer:
    def __init__(self, args, quiet: bool = False):
        self.args = args
        dev = args.device or ("cuda" if torch.cuda.is_available() else "cpu")
        dev_type = torch.device(dev).type
        self.rank, self.world = init_distributed(dev_type)
        if dev_type == "cuda":
            local = int(os.environ.get("LOCAL_RANK", "0")) if self.world > 1 else (torch.device(dev).index or 0)
            self.device = torch.device("cuda", local)
            torch.cuda.set_device(self.device)
        else:
            self.device = torch.device("cpu")
        cuda = self.device.type == "cuda"
        if hasattr(args, "normalization"):
            check_compat_flags(args)
        over = {}
        if args.seq_length:
            over["seq_len"] = args.seq_length
        if args.num_layers:
            over["num_layers"] = args.num_layers
        if args.untie_embeddings_and_output_weights:
            over["tied_embeddings"] = False
        for flag, field in (("hidden_size", "hidden"), ("ffn_hidden_size", "ffn"), ("num_attention_heads", "n_heads"),
                            ("num_query_groups", "n_kv_heads"), ("kv_channels", "head_dim"),
                            ("padded_vocab_size", "vocab"), ("rotary_base", "rope_theta"),
                            ("norm_epsilon", "norm_eps"), ("init_method_std", "init_std")):
            if getattr(args, flag, None) is not None:
                over[field] = getattr(args, flag)
        if getattr(args, "qk_layernorm", False):
            over["qk_norm"] = True
        if ("hidden" in over or "n_heads" in over) and "head_dim" not in over:
            base = get_config(args.model)
            over["head_dim"] = over.get("hidden", base.hidden) // over.get("n_heads", base.n_heads)
        self.cfg = get_config(args.model, **over)
        c = self.cfg
        if c.n_heads % c.n_kv_heads or c.head_dim % 8 or c.hidden % 8 or c.ffn % 8:
            raise ValueError(f"model geometry: {c.n_heads} heads must be a multiple of {c.n_kv_heads} key/value heads; "
                             "head dimension, hidden and FFN sizes must be multiples of 8")
        self.tp_size = max(1, int(args.tensor_model_parallel_size))
        self.pp_size = max(1, int(args.pipeline_model_parallel_size or 1))
        mp = self.tp_size * self.pp_size
        assert self.world % mp == 0, "world size must be a multiple of tensor-parallel x pipeline-parallel size"
        self.dp_world = self.world // mp
        # rank = (pp_rank * dp + dp_rank) * tp + tp_rank: adjacent ranks form a tensor-parallel group,
        # data-parallel groups stride over them inside a pipeline stage, stages are the outermost axis
        tp, dp, pp = self.tp_size, self.dp_world, self.pp_size
        self.tp_rank = self.rank % tp
        self.dp_rank = (self.rank // tp) % dp
        self.pp_rank = self.rank // (tp * dp)
        self.tp_group = self.dp_group = self.pp_group = None

        def rank_of(p, d, t):
            return (p * dp + d) * tp + t

        # every rank creates every group, in the same order (a requirement of new_group)
        if tp > 1:
            for p in range(pp):
                for d in range(dp):
                    grp = dist.new_group(ranks=[rank_of(p, d, t) for t in range(tp)])
                    if (p, d) == (self.pp_rank, self.dp_rank):
                        self.tp_group = grp
        if tp > 1 or pp > 1:
            for p in range(pp):
                for t in range(tp):
                    grp = dist.new_group(ranks=[rank_of(p, d, t) for d in range(dp)])
                    if (p, t) == (self.pp_rank, self.tp_rank):
                        self.dp_group = grp
        if pp > 1:
            for d in range(dp):
                for t in range(tp):
                    grp = dist.new_group(ranks=[rank_of(p, d, t) for p in range(pp)])
                    if (d, t) == (self.dp_rank, self.tp_rank):
                        self.pp_group = grp
        self._last_stage_peer = rank_of(pp - 1, self.dp_rank, self.tp_rank)
        assert args.global_batch_size % (args.micro_batch_size * self.dp_world) == 0, (
            "global batch must be a multiple of micro_batch * data-parallel size")
        self.num_micro = args.global_batch_size // (args.micro_batch_size * self.dp_world)
        transport = args.transport
        sga_t = getattr(args, "sga_backend_transport", "auto")
        if transport == "auto" and sga_t != "auto":
            transport = sga_t
        self.pool = None
        if cuda and transport == "auto" and self.dp_world > 1 and not self._dp_group_on_one_host():
            # peer-mapped memory (CUDA IPC) covers one NVSwitch domain: a data-parallel group that spans
            # hosts, or has more than 8 ranks, takes the library collectives
            transport = "nccl"
            if self.rank == 0 and not quiet:
                print("[train] the data-parallel group spans hosts (or more than 8 ranks): transport nccl, "
                      "dense steps by all-reduce", flush=True)
        if cuda and transport in ("auto", "p2p"):
            from ..parallel.symm import McastPool, SymmPool

            pool_cls = McastPool if getattr(args, "nvls_dense", False) else SymmPool
            self.pool = pool_cls(group=self.dp_group, device=self.device)
        self.tp = None
        if self.tp_size > 1:
            from ..parallel.tp import TPContext

            tp_comm = args.tp_comm
            if tp_comm == "auto":
                tp_comm = "fused" if (cuda and transport in ("auto", "p2p")) else "library"
            self.tp = TPContext(group=self.tp_group, device=self.device, transport=tp_comm)
        self.sga = bool(getattr(args, "sga_enabled", False))  # the one gate: nothing else of sga_* is read when it is off
        if self.sga and self.tp_size > 1 and getattr(args, "sga_selection_locality", "shared") != "rank_local":
            raise NotImplementedError(
                "SGA under tensor parallelism needs --sga-selection-locality rank_local: a shared support's "
                "threshold is global over the model, so it would differ between tensor-parallel ranks and "
                "select different coordinates of the parameters they replicate")
        need_comm = (self.sga and getattr(args, "sga_selection_locality", "shared") == "rank_local"
                     and getattr(args, "sga_backend", None) != "torch_pipelined_mask")
        self.model = GPT(self.cfg, device=self.device, pool=self.pool,
                         bucket_elems=getattr(args, "sga_bucket_elems", 16 << 20), seed=args.seed,
                         need_comm_staging=need_comm, tp=self.tp,
                         init_on_device=bool(getattr(args, "init_on_device", False)),
                         pp_size=self.pp_size, pp_rank=self.pp_rank,
                         recompute=bool(getattr(args, "recompute_activations", False)),
                         vocab_parallel=bool(getattr(args, "vocab_parallel_embedding", False)))
        self.pipeline = None
        if self.pp_size > 1:
            from ..parallel.pp import Pipeline

            self.pipeline = Pipeline(self.model, pp_rank=self.pp_rank, pp_size=self.pp_size,
                                     prev_rank=self.rank - self.dp_world * self.tp_size if self.pp_rank > 0 else None,
                                     next_rank=(self.rank + self.dp_world * self.tp_size
                                                if self.pp_rank < self.pp_size - 1 else None))
        ddp_cfg = DDPConfig(average_in_collective=True, overlap_grad_reduce=bool(args.overlap_grad_reduce),
                            comm_max_ctas=args.comm_max_ctas)
        ddp_cfg.nvls_dense = bool(getattr(args, "nvls_dense", False))
        if getattr(args, "sga_backend_timer", None):
            ddp_cfg.overlap_grad_reduce = False
        if self.tp is not None:
            # Both kinds of kernel wait on other GPUs. Run concurrently, two ranks could start them in
            # opposite orders and each hold the SMs the other's peer is waiting for, so under tensor
            # parallelism the data-parallel synchronisation follows the backward pass on one stream order.
            ddp_cfg.overlap_grad_reduce = False
        self.ddp = DataParallel(self.model, group=self.dp_group, transport=transport, ddp_config=ddp_cfg,
                                pool=self.pool)
        if self.ddp.transport == "gloo":
            ddp_cfg.average_in_collective = False
        self.optimizer = FlatOptimizer(self.model.arena, OptimizerConfig(
            lr=args.lr, weight_decay=args.weight_decay, adam_beta1=args.adam_beta1, adam_beta2=args.adam_beta2,
            adam_eps=args.adam_eps, clip_grad=args.clip_grad, log_num_zeros_in_grad=args.log_num_zeros_in_grad))
        self.engine = None
        if getattr(args, "sga_backend_timer", None):
            from ..utils import backend_timer

            if not backend_timer.enabled():
                backend_timer.enable(args.sga_backend_timer, self.rank)
            backend_timer.time_full_syncs()
        if self.sga:
            self.engine = build_engine(trainer_args=args, quiet=quiet)
            self.engine.log_interval = args.log_interval
            if self.tp is not None or self.pp_size > 1:
                self.engine.model_parallel_norm = self._tp_norm
            self.engine.attach(self.ddp)
            self.engine.bind_optimizer(self.optimizer)
        if getattr(args, "data_path", None):
            from .data import TokenFile

            self.data = TokenFile(args.data_path, self.cfg.vocab, self.cfg.seq_len, args.data_seed,
                                  args.global_batch_size, dtype=getattr(args, "data_dtype", None), pin=cuda)
        else:
            self.data = SyntheticTokens(self.cfg.vocab, self.cfg.seq_len, args.data_seed, pin=cuda)
        self.iteration = 0
        self._dense = None
        if cuda:
            self._dev_sumsq = torch.zeros(1, device=self.device)
            self._dev_coeff = torch.ones(1, device=self.device)
            self._dev_norm = torch.zeros(1, device=self.device)
        self.last_grad_norm = None
        self._dup_ranges = []
        self._dev_dup = None
        if self.tp is not None:
            # merged element ranges of the parameters every tensor-parallel rank holds
            for sl in self.model.arena.slots:
                if sl.spec.tp_duplicate:
                    if self._dup_ranges and self._dup_ranges[-1][1] == sl.start:
                        self._dup_ranges[-1][1] = sl.end
                    else:
                        self._dup_ranges.append([sl.start, sl.end])
            self._dev_dup = torch.zeros(1, device=self.device) if cuda else None

    def _tp_norm(self, sumsq: torch.Tensor, source: torch.Tensor, mask=None) -> None:
        """``sumsq`` (this rank's sum of squares over ``source``) -> the whole model's: the sharded part
        summed over the tensor-parallel ranks with the replicated part counted once, then the stages of
        the pipeline added up."""
        if self.tp is not None:
            if self.device.type == "cuda":
                from .. import kernels as K

                first = True
                for lo, hi in self._dup_ranges:
                    K.sumsq(source[lo:hi], self._dev_dup, mask=None if mask is None else mask[lo:hi],
                            accumulate=not first)
                    first = False
                dup = self._dev_dup
            else:
                tot = 0.0
                for lo, hi in self._dup_ranges:
                    v = source[lo:hi].double()
                    if mask is not None:
                        v = torch.where(mask[lo:hi] > 0, v, torch.zeros_like(v))
                    tot += float((v ** 2).sum())
                dup = torch.tensor([tot], dtype=sumsq.dtype)
            sumsq.sub_(dup.to(sumsq.dtype))
            dist.all_reduce(sumsq, group=self.tp_group)
            sumsq.add_(dup.to(sumsq.dtype))
        if self.pp_group is not None:
            dist.all_reduce(sumsq, group=self.pp_group)

    # ----------------------------------------------------------------- data
    @torch.no_grad()
    def evaluate(self, iters: int) -> float:
        """Mean token loss over ``iters`` global batches of the validation stream, forward passes only,
        averaged over the data-parallel ranks. Touches neither gradients nor optimizer state."""
        if getattr(self, "_eval_data", None) is None:
            a, cuda = self.args, self.device.type == "cuda"
            path = getattr(a, "eval_data_path", None) or getattr(a, "data_path", None)
            if path:
                from .data import TokenFile

                self._eval_data = TokenFile(path, self.cfg.vocab, self.cfg.seq_len, a.data_seed + 7919,
                                            a.global_batch_size, dtype=getattr(a, "data_dtype", None), pin=cuda)
            else:
                self._eval_data = SyntheticTokens(self.cfg.vocab, self.cfg.seq_len, a.data_seed + 7919, pin=cuda)
        mb, per_rank = self.args.micro_batch_size, self.num_micro * self.args.micro_batch_size
        total = torch.zeros((), dtype=torch.float32, device=self.device)
        for step in range(iters):
            batch = self._eval_data.batch(step, self.dp_rank * per_rank, per_rank).to(self.device, non_blocking=True)
            if self.pipeline is not None:
                mbs = [(batch[i * mb:(i + 1) * mb][:, :-1], batch[i * mb:(i + 1) * mb][:, 1:])
                       for i in range(self.num_micro)]
                for loss in self.pipeline.run_forward(mbs):   # the last stage holds the losses
                    total += loss
                continue
            for i in range(self.num_micro):
                chunk = batch[i * mb:(i + 1) * mb]
                total += self.model.forward_backward(chunk[:, :-1], chunk[:, 1:], backward=False,
                                                     reduce_replicated=False)
        total /= max(iters * self.num_micro, 1)
        if self.pipeline is not None:
            # hand the last stage's mean to every stage of the replica
            t = total.reshape(1).clone()
            dist.broadcast(t, src=self._last_stage_peer, group=self.pp_group)
            total = t[0]
        if self.dp_world > 1:
            dist.all_reduce(total, group=self.dp_group)
            total /= self.dp_world
        return float(total.item())

    def _dp_group_on_one_host(self) -> bool:
        import socket

        if self.dp_world > 8:
            return False
        names = [None] * self.dp_world
        dist.all_gather_object(names, socket.gethostname(), group=self.dp_group)
        return len(set(names)) == 1

    # ------------------------------------------------- sharded optimizer state
    @property
    def sharded_state(self) -> bool:
        """True when each data-parallel rank keeps the fp32 weights and moments only for the slice
        of every bucket it owns (the fused dense step, and the sharded SGA step)."""
        if self.engine is not None:
            return bool(getattr(self.engine, "sharded", False))
        return self._fused_dense() and self.dp_world > 1

    def gather_optimizer_state(self) -> None:
        """All-gather the owner slices of the fp32 weights and both moments over the data-parallel
        group, so that every rank holds the whole replicated state again (what a checkpoint, a trace
        dump or a parameter norm reads). The cut is the update kernel's: a bucket of n elements is
        split at 16-byte granularity into ``dp`` equal slices, slice r owned by rank r."""
        if not self.sharded_state or self.dp_world == 1:
            return
        arena = self.model.arena
        W, r = self.dp_world, self.dp_rank
        for b in arena.buckets:
            n4 = (b.numel + 3) // 4
            per = (n4 + W - 1) // W * 4
            lo, hi = min(b.numel, per * r), min(b.numel, per * (r + 1))
            for t in (arena.main_param, arena.exp_avg, arena.exp_avg_sq):
                view = t[b.start:b.end]
                stage = torch.zeros(per, dtype=t.dtype, device=t.device)
                stage[:hi - lo].copy_(view[lo:hi])
                full = torch.empty(per * W, dtype=t.dtype, device=t.device)
                dist.all_gather_into_tensor(full, stage, group=self.dp_group)
                view.copy_(full[:b.numel])

    def host_batch(self, step: int) -> torch.Tensor:
        """This rank's ``[num_micro * micro_batch, seq + 1]`` token block for ``step`` (pinned host memory)."""
        per_rank = self.num_micro * self.args.micro_batch_size
        return self.data.batch(step, self.dp_rank * per_rank, per_rank)

    # ----------------------------------------------------------------- step
    def train_step(self, batch: torch.Tensor) -> torch.Tensor:
        """``batch``: ``[num_micro * micro_batch, seq + 1]`` int64 token ids, on the
        host (pinned) or already on the device. Returns the mean loss (device scalar)."""
        # the engine is called with the number of completed iterations, 0 on the first step of a fresh run and K
        # after a resume at K: the numbering of its step calendar, of the log line and of the trace files
        # ("dump at step t is the state with exactly t commits applied", sga/trace.py:37-41)
        it = self.iteration
        self.iteration += 1
        self.optimizer.set_lr(scheduled_lr(self.args, it))
        mb = self.args.micro_batch_size
        if batch.device != self.device:
            batch = batch.to(self.device, non_blocking=True)
        losses = []
        self.ddp.begin_step()

        def arm_last():
            if self.engine is not None:
                self.engine.begin_step(self.ddp, it)
            else:
                self._arm_dense()

        if self.pipeline is not None:
            mbs = []
            for i in range(self.num_micro):
                chunk = batch[i * mb:(i + 1) * mb]
                mbs.append((chunk[:, :-1], chunk[:, 1:]))
            losses = self.pipeline.run(mbs, loss_scale=1.0 / self.num_micro,
                                       on_param_done_last=self.ddp.on_param_done, before_last_backward=arm_last)
        else:
            for i in range(self.num_micro):
                chunk = batch[i * mb:(i + 1) * mb]
                tokens, targets = chunk[:, :-1], chunk[:, 1:]
                last = i == self.num_micro - 1
                if last:
                    arm_last()
                with _nvtx(f"micro_batch_{i}"):
                    loss = self.model.forward_backward(tokens, targets, loss_scale=1.0 / self.num_micro,
                                                       on_param_done=self.ddp.on_param_done if last else None,
                                                       reduce_replicated=last)
                losses.append(loss)
        if self.engine is not None:
            with _nvtx("grad_sync"):
                if not self.engine.grad_sync(self.ddp, False):
                    self.ddp.finish_grad_sync()
            with _nvtx("optimizer_step"):
                ok, gn, _nz = self.engine.optimizer_step(self.optimizer, [self.ddp], it)
            self.last_grad_norm = gn
        else:
            with _nvtx("dense_step"):
                self._dense_step()
        if self.pipeline is not None:
            # the loss lives on the last stage: hand it to every stage of the replica
            t = torch.stack(losses).mean() if losses else torch.zeros((), dtype=torch.float32, device=self.device)
            t = t.reshape(1).clone()
            dist.broadcast(t, src=self._last_stage_peer, group=self.pp_group)
            return t[0]
        return torch.stack(losses).mean()

    # ----------------------------------------------------------- dense path
    def _fused_dense(self) -> bool:
        # the sharded-update kernel sees one rank's slice of the gradient; the tensor-parallel norm needs
        # the whole replicated parameters, so that combination takes the all-reduce path
        return self.args.dense_mode == "fused" and self.ddp.transport == "p2p" and self.tp is None

    def _arm_dense(self) -> None:
        if self._fused_dense():
            self._dev_sumsq.zero_()
            self.ddp.arm(self._rs_bucket_sync)
        else:
            self.ddp.arm(None)

    def _rs_bucket_sync(self, bucket) -> None:
        from ..parallel import p2p

        ch, buf = self.ddp.channel_for(bucket), self.model.arena.symm_grad
        kw = dict(scale=self.ddp.gradient_scaling_factor, rs_only=True, sumsq_out=self._dev_sumsq, accumulate=True,
                  max_ctas=self.ddp.ddp_config.comm_max_ctas)
        if not (self.ddp.ddp_config.nvls_dense and p2p.nvls_allreduce_(ch, buf, 4 * bucket.start, bucket.numel, **kw)):
            p2p.allreduce_(ch, buf, 4 * bucket.start, bucket.numel, **kw)

    def _dense_step(self) -> None:
        arena = self.model.arena
        opt = self.optimizer
        clip = float(opt.config.clip_grad or 0.0)
        g0 = opt.param_groups[0]
        beta1, beta2 = g0["betas"]
        if self._fused_dense():
            from .. import kernels as K
            from ..parallel import p2p

            self.ddp.finish_pending()
            if self.pp_group is not None:
                dist.all_reduce(self._dev_sumsq, group=self.pp_group)  # the other stages' share of the norm
            K.clip_coeff(self._dev_sumsq, 1.0, clip, self._dev_coeff, self._dev_norm)
            if self._dense is None:
                bs = torch.tensor([b.start for b in arena.buckets], dtype=torch.int64, device=self.device)
                bl = torch.tensor([b.numel for b in arena.buckets], dtype=torch.int64, device=self.device)
                self._dense = (bs, bl)
            p2p.dense_adamw_ag_(self.ddp.channels[0], arena.main_param, arena.main_grad, arena.exp_avg,
                                arena.exp_avg_sq, arena.symm_model, self._dense[0], self._dense[1],
                                arena.segment_table(), opt.group_lr(), opt.group_wd(), beta1=beta1, beta2=beta2,
                                eps=g0["eps"], step=opt.peek_step(), coeff=self._dev_coeff if clip > 0 else None)
            opt.advance_step()
            arena.main_grad.zero_()
            self.last_grad_norm = self._dev_norm
            return
        self.ddp.finish_grad_sync()
        if self.device.type == "cuda":
            from .. import kernels as K

            K.sumsq(arena.main_grad, self._dev_sumsq)
            if self.tp is not None or self.pp_group is not None:
                self._tp_norm(self._dev_sumsq, arena.main_grad)
            K.clip_coeff(self._dev_sumsq, 1.0, clip, self._dev_coeff, self._dev_norm)
            K.adam_step(arena.main_param, arena.main_grad, arena.exp_avg, arena.exp_avg_sq, arena.segment_table(),
                        opt.group_lr(), opt.group_wd(), beta1=beta1, beta2=beta2, eps=g0["eps"],
                        step=opt.peek_step(), model=arena.model_param, coeff=self._dev_coeff if clip > 0 else None)
            opt.advance_step()
            self.last_grad_norm = self._dev_norm
        else:
            from ..plugins.optimizer.reference import grad_correct_torch

            sq = torch.tensor([float((arena.main_grad.double() ** 2).sum())], dtype=torch.float64)
            if self.tp is not None or self.pp_group is not None:
                self._tp_norm(sq, arena.main_grad)
            norm = float(sq.sqrt())
            coeff = 1.0
            if clip > 0 and clip / (norm + 1e-6) < 1.0:
                coeff = float(torch.tensor(clip / (norm + 1e-6), dtype=torch.float32))
            step = opt.peek_step()
            for s in arena.slots:
                sl = slice(s.start, s.end)
                grp = opt.param_groups[s.spec.group]
                grad_correct_torch(arena.main_param[sl], arena.main_grad[sl], arena.exp_avg[sl], arena.exp_avg_sq[sl],
                                   grp["lr"], beta1, beta2, g0["eps"], grp["weight_decay"], 1 - beta1 ** step,
                                   1 - beta2 ** step, None, None, coeff=coeff, model_param=arena.model_param[sl])
            opt.advance_step()
            self.last_grad_norm = norm
        arena.main_grad.zero_()

    # ------------------------------------------------------------ utilities
    def tokens_per_step(self) -> int:
        return self.args.global_batch_size * self.cfg.seq_len

    def check(self) -> None:
        self.ddp.check()
        if self.tp is not None:
            self.tp.check()

    def close(self) -> None:
        if self.engine is not None and self.engine._trace is not None:
            self.engine._trace.close()
        if self.tp is not None:
            self.tp.close()
            self.tp = None
        if self.pool is not None:
            self.pool.close()
            self.pool = None


def default_args(**overrides):
    args = build_parser().parse_args([])
    for k, v in overrides.items():
        if not hasattr(args, k):
            raise AttributeError(f"unknown trainer arg '{k}'")
        setattr(args, k, v)
    return args
