"""The SGA engine: three call points around a data-parallel model chunk.

  attach(ddp)                         once, after the model is built
  grad_sync(ddp, force_all_reduce)    after the backward pass of a step
  optimizer_step(optimizer, chunks, iteration)

plus ``begin_step`` which, called before the last micro-batch, lets every
bucket's synchronisation start while the backward pass is still running.

Step numbers are the caller's: the trainer passes the number of completed iterations (0 on the first
step of a fresh run, K after a resume at K), which is also the number in the log line and in the
trace file names (``sga/trace.py:37-41``: the dump at step t holds the state with t commits applied).
Calendar (``CycleManager``): a step is FULL when forced, when
``step <= start_iter``, at a cycle boundary ``(step - start) % period == 0``,
on the decoupled extra grid, or while no support exists. Reselection happens
only at non-forced boundaries. A full step runs the dense average of every
bucket and lets the optimizer template write the configured score into the
grad buffers; a sparse step communicates the support only, and what is not
communicated stays in the fp32 grad buffer: that buffer is the residual.

``optimizer_step`` runs a frozen order that tests pin:
prepare_grads -> masked clip -> count_zeros -> trace dump slot -> optimizer
full/sparse step -> model-parameter copy -> (boundary) selection -> optimizer
reset -> support activation -> count guard -> force-next probe -> host-state
reset -> log.

Two selection localities. ``shared`` reproduces the reference: one support for
all ranks, chosen at boundaries from dense-averaged scores, values-only
payloads in between. ``rank_local`` is this framework's addition: every sparse
step each rank takes the exact top-k of ``|grad + residual|`` per bucket and
exchanges (index, value) pairs (index backend) or the union of the ranks'
masks is reduced in place (mask backend); boundaries are dense flushes.

Reference: ``sga/engine.py`` (CycleManager ``:109-174``, attach ``:318-412``,
grad_sync ``:416-481``, optimizer_step ``:485-618``, shadow ``:622-743``,
selection tail ``:822-928``, clip ``:1052-1218``, checks ``:1299-1389``,
logging ``:1451-1472``).
"""
from __future__ import annotations

import json
import os
from typing import Optional

import torch
import torch.distributed as dist

from ..config import get_args
from ..plugins.optimizer import OptContext, ParamRecord
from ..plugins.scores import compute_score, get_score_spec
from ..support import BucketSupport, IndexPool, Support
from ..utils import backend_timer


class SGAEngineError(RuntimeError):
    """Cross-rank inconsistency or a violated engine contract."""


class BucketState:
    def __init__(self, grad_data, dp_group, gradient_scaling_factor, bucket_id, arena_start=0):
        self.grad_data = grad_data
        self.dp_group = dp_group
        self.gradient_scaling_factor = gradient_scaling_factor
        self.bucket_id = bucket_id
        self.arena_start = arena_start
        self.support_index = None
        self.param_spans = []     # [(slot, start, end)] relative to the bucket
        self.param_names = []
        self.active_mask_u8 = None


class ShardedStep:
    """Sharded form of the optimizer step over the peer-memory transport: one launch updates, on every
    rank, the slice of each bucket that the rank owns (the cut of ``csrc/dense_sync.cu``) and stores
    the bf16 parameters into every rank's model arena. The fp32 weights and moments outside a rank's
    slices go stale; ``Trainer.gather_optimizer_state`` rebuilds the replicated layout on demand."""

    def __init__(self, ddp):
        arena = ddp.arena
        self.ddp = ddp
        self.bucket_start = torch.tensor([b.start for b in arena.buckets], dtype=torch.int64, device=arena.device)
        self.bucket_len = torch.tensor([b.numel for b in arena.buckets], dtype=torch.int64, device=arena.device)

    def step(self, arena, grad, opt, *, beta1, beta2, eps, step, coeff, adams) -> None:
        from ..parallel import p2p

        p2p.dense_adamw_ag_(self.ddp.channels[0], arena.main_param, grad, arena.exp_avg, arena.exp_avg_sq,
                            arena.symm_model, self.bucket_start, self.bucket_len, arena.segment_table(),
                            opt.group_lr(), opt.group_wd(), beta1=beta1, beta2=beta2, eps=eps, step=step,
                            coeff=coeff, adams=adams, max_ctas=self.ddp.ddp_config.comm_max_ctas)


class SelectionContext:
    """What a selector sees: the eligible score views, the comm group and the
    warm-up target its own hook implied."""

    def __init__(self, grad_views, comm_group, warmup_target=None):
        self.grad_views = grad_views
        self.comm_group = comm_group
        self.warmup_target = warmup_target


class CycleManager:
    def __init__(self, start_iter: int, period: int, decouple: bool, full_sync_interval, allow_zero: bool = False):
        assert period >= 1 or (allow_zero and period == 0)
        if decouple:
            assert (full_sync_interval is not None and 0 < full_sync_interval < period
                    and period % full_sync_interval == 0), (
                f"decoupled full_sync_interval ({full_sync_interval}) must satisfy 0 < full_sync_interval < "
                f"period ({period}) and period % full_sync_interval == 0")
        else:
            assert full_sync_interval is None, (
                "full_sync_interval is only settable with decouple_full_sync_interval_and_period=true")
        self.start_iter = start_iter
        self.period = period
        self.decouple = decouple
        self.full_sync_interval = full_sync_interval
        self.force_next = False

    @property
    def fold_window(self) -> int:
        return self.full_sync_interval if self.decouple else max(self.period, 1)

    def reselect_boundary(self, step: int) -> bool:
        if self.period == 0:
            return False
        return step > self.start_iter and (step - self.start_iter) % self.period == 0

    def extra_full(self, step: int) -> bool:
        return (self.decouple and step > self.start_iter
                and (step - self.start_iter) % self.full_sync_interval == 0)

    def is_full(self, step: int, force: bool = False) -> bool:
        if force or step <= self.start_iter:
            return True
        return self.reselect_boundary(step) or self.extra_full(step)


class SGAEngine:
    def __init__(self, score_name: str, selection, opt, backend):
        cfg = get_args()
        self.score_name = score_name
        self.selection = selection
        self.opt = opt
        self.backend = backend
        assert self.opt.emit_score == self.score_name, (
            f"engine score '{score_name}' != optimizer emit_score '{self.opt.emit_score}'")
        self.rank_local = getattr(cfg, "sga_selection_locality", "shared") == "rank_local"
        self._cycle = CycleManager(cfg.sga_cycle_start_iter, cfg.sga_cycle_period,
                                   cfg.sga_cycle_decouple_full_sync_interval_and_period,
                                   cfg.sga_cycle_full_sync_interval, allow_zero=self.rank_local)
        layout = getattr(backend, "layout", "auto")
        if layout == "auto":
            layout = "er" if getattr(selection, "block_size", 1) == 1 else "bb"
        self._backend_layout = layout
        self._selection_block_size = getattr(selection, "block_size", 1)
        self._ratio = float(cfg.sga_selection_ratio_percent) / 100.0 if cfg.sga_selection_ratio_percent else 0.0
        self._chunks = {}
        self._bucket_states = []
        self._selection_meta = None
        self._active_support: Optional[Support] = None
        self._compact_values = {}
        self._compact_values_step = None
        self._mask_arenas = None
        self._mask_turn = 0
        self._idx_pools = None
        self._records = None
        self._iter = 0
        self._first_step = True
        self._step_full = None
        self._step_forced = False
        self._decided_step = None
        self._count_guard = cfg.sga_checks_count_guard
        self._support_consistency = cfg.sga_checks_support_consistency
        self._norm_spread = cfg.sga_checks_norm_spread
        self._rng_bracket = cfg.sga_checks_rng_bracket
        self._rank = dist.get_rank() if (dist.is_available() and dist.is_initialized()) else 0
        # set by a trainer that shards the model: fn(sumsq, source, mask) folds the other shards into the norm
        self.model_parallel_norm = None
        if not (self._count_guard and self._support_consistency and self._norm_spread and self._rng_bracket):
            if self._rank == 0:
                msg = (f"[SGA] WARN sga_checks escape hatch active (L1_count={int(self._count_guard)} "
                       f"L2_support={int(self._support_consistency)} L3_norm_spread={int(self._norm_spread)} "
                       f"rng_bracket={int(self._rng_bracket)}): benchmark measurement posture, not a production "
                       "setting")
                if not (self._count_guard and self._support_consistency and self._norm_spread):
                    msg += " -- cross-rank divergence detection is OFF"
                if not self._rng_bracket:
                    msg += " -- shadow RNG bracket skipped"
                print(msg, flush=True)
        layers = cfg.sga_always_sync_layers
        self._always_sync_layers = list(layers) if layers is not None else None
        self._forced_slots = set()
        self._trace = None
        if cfg.sga_trace_dir is not None:
            from ..trace import TraceCollector

            self._trace = TraceCollector(
                dir=cfg.sga_trace_dir, branch_points=cfg.sga_trace_branch_points, window=cfg.sga_trace_window,
                dump_dtype=cfg.sga_trace_dump_dtype, async_enabled=cfg.sga_trace_async,
                async_backend=cfg.sga_trace_async_backend, async_queue_depth=cfg.sga_trace_async_queue_depth,
                async_worker_count=cfg.sga_trace_async_worker_count,
                async_max_workset_gib=cfg.sga_trace_async_max_workset_gib)
        self._shadow = cfg.sga_shadow
        self._shadow_score = cfg.sga_shadow_score
        self._metrics_file = os.environ.get("SGA_METRICS_FILE")
        self.log_interval = 1
        self._ddp = None
        self._dev = {}
        self.last_ratio = None

    # ------------------------------------------------------------------ attach
    def attach(self, ddp) -> None:
        for attr in ("arena", "buckets", "module", "ddp_config", "finish_grad_sync"):
            if not hasattr(ddp, attr):
                raise TypeError(f"the engine attaches to DataParallel chunks (missing .{attr}); got "
                                f"{type(ddp).__name__}")
        if id(ddp) in self._chunks:
            return
        if self._chunks:
            raise SGAEngineError("one model chunk per rank (virtual pipeline stages are not supported)")
        self._chunks[id(ddp)] = ddp
        self._ddp = ddp
        arena = ddp.arena
        for b in arena.buckets:
            bs = BucketState(arena.main_grad[b.start:b.end], ddp.group, ddp.gradient_scaling_factor, b.index,
                             arena_start=b.start)
            bs.support_index = len(self._bucket_states)
            for slot in b.slots:
                bs.param_spans.append((slot, slot.start - b.start, slot.end - b.start))
                bs.param_names.append(slot.name)
            self._bucket_states.append(bs)
        self._selection_meta = None
        self._always_sync_attach_check()
        self.opt.ensure_state(self._bucket_states)
        if self._backend_layout == "bb" and getattr(self.backend, "block_form", "block_idx") == "block_desc":
            self._bb_alignment_check()
        bind = getattr(self.backend, "bind", None)
        if callable(bind):
            bind(ddp)
        prepare = getattr(self.backend, "prepare", None)
        if callable(prepare) and ddp.group is not None:
            prepare(ddp.group, device=arena.device)
        if self.rank_local:
            max_b = max(b.numel for b in arena.buckets)
            max_k = max(self._k_for_bucket(b.numel) for b in arena.buckets)
            self.backend.configure_rank_local(max_b, max_k)
            if self.backend.consumes == "idx" and arena.comm is None:
                arena.comm = torch.zeros(arena.numel, dtype=torch.float32, device=arena.device)
        # Sharded optimizer step: possible when every rank ends the sync with the same gradient and
        # nothing reads another rank's share of the weights or moments: rank-local index mode with the
        # |grad + residual| score, peer-memory transport, no model parallelism, no trace dumps.
        want = os.environ.get("SGA_SHARDED_STEP", "auto")
        self.sharded = None
        if (want != "0" and self.rank_local and self.backend.consumes == "idx" and self.score_name == "abs_g"
                and getattr(ddp, "transport", None) == "p2p" and ddp.world > 1 and arena.symm_model is not None
                and self._trace is None and self.model_parallel_norm is None and not self._shadow):
            self.sharded = ShardedStep(ddp)
        if arena.device.type == "cuda":
            z = lambda dt: torch.zeros(1, dtype=dt, device=arena.device)  # noqa: E731
            self._dev = {"sumsq": z(torch.float32), "coeff": torch.ones(1, dtype=torch.float32, device=arena.device),
                         "norm": z(torch.float32), "one": torch.ones(1, dtype=torch.float32, device=arena.device)}

    def _k_for_bucket(self, n: int) -> int:
        return max(1, min(n, int(round(n * self._ratio))))

    def _bb_alignment_check(self) -> None:
        x = self._selection_block_size
        for bs in self._bucket_states:
            for (slot, start, end), name in zip(bs.param_spans, bs.param_names):
                if start % x:
                    raise SGAEngineError(
                        f"sga_backend_layout bb (descriptor packing) needs every param span start {x}-aligned; "
                        f"bucket {bs.bucket_id} param '{name}' spans [{start}, {end}). Use layout eb instead")

    def _always_sync_attach_check(self) -> None:
        if self._always_sync_layers is None:
            return
        names = [(slot, name) for bs in self._bucket_states for (slot, _s, _e), name in
                 zip(bs.param_spans, bs.param_names)]
        forced = set()
        hit = {p: 0 for p in self._always_sync_layers}
        for slot, name in names:
            for pat in self._always_sync_layers:
                if pat in name:
                    forced.add(id(slot))
                    hit[pat] += 1
        if not forced:
            raise SGAEngineError(f"sga_always_sync_layers {self._always_sync_layers} matched no parameter name")
        if len(forced) == len(names):
            raise SGAEngineError("sga_always_sync_layers matched every parameter: the top-k pool would be empty")
        for pat, n in hit.items():
            if n == 0 and self._rank == 0:
                print(f"[SGA] WARN sga_always_sync_layers pattern '{pat}' matched no parameter", flush=True)
        self._forced_slots = forced
        if self._rank == 0:
            tot = sum(e - s for bs in self._bucket_states for (_sl, s, e) in bs.param_spans)
            fc = sum(e - s for bs in self._bucket_states for (sl, s, e) in bs.param_spans if id(sl) in forced)
            print(f"[SGA] always-sync layers: {len(forced)} params, {fc} of {tot} elements "
                  f"({100.0 * fc / max(tot, 1):.2f}%) forced into every support", flush=True)

    # -------------------------------------------------------------- grad sync
    def _dp_group(self):
        return self._ddp.group if self._ddp is not None else None

    def _world(self) -> int:
        return self._ddp.world if self._ddp is not None else 1

    def _decide(self, force_all_reduce: bool) -> bool:
        step = self._iter + 1
        if self._decided_step == step:
            return self._step_full
        backend_timer.at_step(step)
        forced = bool(force_all_reduce) or self._cycle.force_next
        if self._cycle.force_next:
            self._cycle.force_next = False
        if self.rank_local:
            full = forced or self._cycle.is_full(step)
        else:
            full = forced or self._cycle.is_full(step) or self._active_support is None
        self._step_full = full
        self._step_forced = forced
        self._decided_step = step
        if self._compact_values_step != step:
            self._compact_values = {}
            self._compact_values_step = step
        for key in ("sumsq",):
            if key in self._dev:
                self._dev[key].zero_()
        if getattr(self.backend, "sumsq", None) is not None:
            self.backend.sumsq.zero_()
        if getattr(self.backend, "union_count", None) is not None:
            self.backend.union_count.zero_()
        return full

    def begin_step(self, ddp, iteration: Optional[int] = None, force_all_reduce: bool = False) -> None:
        """Call before the last micro-batch: arms per-bucket sync for its backward pass."""
        if id(ddp) not in self._chunks or self._shadow:
            ddp.arm(None)
            return
        if self._first_step and iteration is not None:
            self._iter = iteration - 1
        full = self._decide(force_all_reduce)
        if backend_timer.enabled():
            ddp.disarm()
            return
        ddp.arm(None if full else self._sparse_bucket_sync)

    def _sparse_bucket_sync(self, bucket) -> None:
        bs = self._bucket_states[bucket.index]
        ddp = self._ddp
        arena = ddp.arena
        if self.rank_local:
            k = self._k_for_bucket(bucket.numel)
            if self.backend.consumes == "idx":
                # peer-memory transport, a bucket per channel: push now, add the ranks' pairs once every
                # bucket is out (no rank then waits for a slower peer in the middle of its backward pass)
                defer = (getattr(ddp, "transport", None) == "p2p" and len(getattr(ddp, "channels", ())) >= len(arena.buckets)
                         and callable(getattr(self.backend, "flush_rank_local", None)))
                self.backend.sync_rank_local(bs, k, arena.comm[bucket.start:bucket.end], ddp.group, ddp.world,
                                             score=self._rank_local_score(bs, bucket), defer_reduce=defer)
                if defer:
                    ddp.after_last_bucket = self.backend.flush_rank_local
            else:
                self.backend.sync_rank_local(bs, k, self._active_mask_arena()[bucket.start:bucket.end], ddp.group,
                                             ddp.world)
            return
        support = self._active_support.buckets[bs.support_index]
        avg = ddp.ddp_config.average_in_collective and ddp.transport != "gloo"
        op = dist.ReduceOp.AVG if avg else dist.ReduceOp.SUM
        factor = 1.0 if avg else bs.gradient_scaling_factor
        out = self.backend.allreduce_sparse(bs.grad_data, support, bs.dp_group, factor, op, key=bucket.index,
                                            bucket_state=bs)
        if self.backend.emission == "compact":
            if not isinstance(out, torch.Tensor):
                raise SGAEngineError(f"compact-emission backend returned {type(out).__name__} instead of a values "
                                     "Tensor")
            self._compact_values[id(bs)] = out

    def bind_optimizer(self, optimizer) -> None:
        """The rank-local scores other than ``abs_g`` read the optimizer's hyper-parameters and step
        counter while the buckets are synchronised, i.e. before ``optimizer_step`` hands it over."""
        self._optimizer = optimizer

    def _rank_local_score(self, bs, bucket):
        """Inputs of the fused kernel's score for one bucket (``None`` = ``|grad + residual|``)."""
        if self.score_name == "abs_g":
            return None
        opt = getattr(self, "_optimizer", None)
        if opt is None:
            raise SGAEngineError(f"rank-local score '{self.score_name}' reads the optimizer state: call "
                                 "engine.bind_optimizer(optimizer) after attach")
        from ..parallel.p2p import ScoreInputs

        arena = self._ddp.arena
        sl = slice(bucket.start, bucket.end)
        g0 = opt.param_groups[0]
        wds = tuple(float(opt.param_groups[slot.spec.group]["weight_decay"]) for (slot, _s, _e) in bs.param_spans)
        cached = getattr(bs, "_span_cache", None)
        if cached is None or cached[0] != wds:
            starts = [s for (_slot, s, _e) in bs.param_spans] + [bucket.numel]
            cached = (wds, torch.tensor(starts, dtype=torch.int32, device=arena.device),
                      torch.tensor(wds, dtype=torch.float32, device=arena.device))
            bs._span_cache = cached
        return ScoreInputs(self.score_name, w=arena.main_param[sl], m=arena.exp_avg[sl], v=arena.exp_avg_sq[sl],
                           beta1=g0["betas"][0], beta2=g0["betas"][1], eps=g0["eps"], step=opt.peek_step(),
                           adams=self.opt.optimizer_name == "adams", span_start=cached[1], span_wd=cached[2])

    def grad_sync(self, ddp, force_all_reduce: bool = False) -> bool:
        """True = the engine synchronised every bucket of this chunk."""
        if id(ddp) not in self._chunks:
            return False
        if self._shadow:
            return False
        full = self._decide(force_all_reduce)
        if full:
            ddp.finish_grad_sync(force_all_reduce=force_all_reduce)
            return True
        if ddp.bucket_sync_fn is not self._sparse_bucket_sync:
            ddp.bucket_sync_fn = self._sparse_bucket_sync
        ddp.finish_pending()
        return True

    # --------------------------------------------------------- optimizer step
    def optimizer_step(self, optimizer, model_chunks, iteration: int):
        if self._first_step:
            self._first_step = False
            self._iter = iteration - 1
        was_full = True if self._step_full is None else self._step_full
        step = self._iter + 1
        assert iteration == step, (f"SGA engine step {step} != trainer iteration {iteration}; eval/rerun "
                                   "interleaving broke the step accounting")
        if self._shadow:
            return self._shadow_step(optimizer, model_chunks, iteration, step)
        found_inf = optimizer.prepare_grads()
        if found_inf:
            self._full_clear()
            self._finish(iteration)
            return (False, None, None)
        # 2. masked clip
        grad_norm, coeff = self._masked_clip_grad_norm(optimizer, was_full, step)
        # 3. zeros count before the optimizer overwrites the grads
        num_zeros = self._count_zeros() if optimizer.config.log_num_zeros_in_grad else None
        # 3b. trace dump slot
        if self._trace is not None:
            self._trace.maybe_dump(self, optimizer, step, grad_norm)
        # 4. optimizer template
        arena = self._ddp.arena
        next_full = self._cycle.is_full(step + 1)
        reselect = (not self.rank_local) and self._cycle.reselect_boundary(step) and not self._step_forced
        ctx = OptContext(
            records=self._records or [], phase="full" if was_full else "sparse", support=self._active_support,
            bucket_states=self._bucket_states, fold_window=self._cycle.fold_window, next_step_is_full=next_full,
            apply_coeff=coeff, compact_values=(self._compact_values if (not was_full and self._compact_values)
                                               else None),
            arena=arena, optimizer=optimizer,
            mask_arena=(self._active_mask_arena() if self._mask_in_use(was_full) else None),
            grad_source=("comm" if (self.rank_local and not was_full and self.backend.consumes == "idx")
                         else "grad"),
            emit=not self.rank_local, sharded=self.sharded if self.model_parallel_norm is None else None)
        if was_full:
            self.opt.full_step(ctx)
        else:
            self.opt.sparse_step(ctx)
        # 5. model-parameter copy: fused into the optimizer kernel (and its CPU reference)
        # 6. reselection
        new_support = None
        if reselect:
            meta = self._selection_context()
            views = [arena.main_grad[bs.arena_start + s:bs.arena_start + e] for (bs, s, e, _slot) in meta]
            if self._norm_spread:
                self._check_norm_spread(views)
            new_support = self._run_selection(views, meta)
        # 7. selective reset with the old support, then the switch
        self.opt.reset(ctx, was_full=was_full)
        if new_support is not None:
            self._activate_support(new_support)
            if self._count_guard:
                self._check_counts()
        if hasattr(self.selection, "wants_force_full") and self.selection.wants_force_full(grad_norm):
            self._cycle.force_next = True
        # 8. host state, log
        self._ddp.begin_step()
        self._log_step(step, was_full, reselect, grad_norm)
        self._finish(iteration)
        return (True, grad_norm, num_zeros)

    def _finish(self, iteration) -> None:
        self._step_full = None
        self._step_forced = False
        self._decided_step = None
        self._iter = iteration

    def _mask_in_use(self, was_full: bool) -> bool:
        if self.rank_local:
            return (not was_full) and self.backend.consumes == "mask"
        return self._active_support is not None

    # ------------------------------------------------------------- shadow mode
    def _shadow_step(self, optimizer, model_chunks, iteration, step):
        """The stock dense step, replicated; state is only read at boundaries."""
        found_inf = optimizer.prepare_grads()
        if found_inf:
            self._full_clear()
            self._finish(iteration)
            return (False, None, None)
        self._step_full = True
        reselect = self._cycle.reselect_boundary(step)
        reselected = reselect and self._shadow_score
        # the boundary score reads the post-clip gradient (the stock step has clipped in place by then,
        # sga/shadow.py:34-36): on a scoring step the coefficient is applied now instead of inside the commit
        grad_norm, coeff = self._masked_clip_grad_norm(optimizer, True, step, shadow=True, scale_now=reselected)
        num_zeros = self._count_zeros() if optimizer.config.log_num_zeros_in_grad else 0
        if self._trace is not None:
            self._trace.maybe_dump(self, optimizer, step, grad_norm)
        if reselected:
            self._shadow_reselect(self._refresh_records(optimizer))
        arena = self._ddp.arena
        ctx = OptContext(records=[], phase="full", arena=arena, optimizer=optimizer, apply_coeff=coeff, emit=False,
                         bucket_states=self._bucket_states)
        self.opt.full_step(ctx)
        self._full_clear()
        self._ddp.begin_step()
        self._log_step(step, True, reselected, grad_norm)
        self._finish(iteration)
        return (True, grad_norm, num_zeros)

    def _shadow_reselect(self, records):
        rng_before = torch.get_rng_state() if self._rng_bracket else None
        cuda_before = (torch.cuda.get_rng_state_all() if (torch.cuda.is_available() and self._rng_bracket) else None)
        from .shadow import readonly_score

        rec_of = {id(r.model_param): r for r in records}
        meta = self._selection_context()
        views = []
        for (_bs, _s, _e, slot) in meta:
            rec = rec_of.get(id(slot.model))
            if rec is None:
                raise TypeError("shadow reselection: parameter without a record")
            views.append(readonly_score(rec, self.score_name, optimizer_name=self.opt.optimizer_name).view(-1))
        if self._norm_spread:
            self._check_norm_spread(views)
        self._activate_support(self._run_selection(views, meta))
        if self._count_guard:
            self._check_counts()
        if self._rng_bracket:
            if not torch.equal(torch.get_rng_state(), rng_before):
                raise RuntimeError("shadow: boundary scoring consumed CPU RNG; selections must be deterministic")
            if cuda_before is not None:
                after = torch.cuda.get_rng_state_all()
                if len(after) != len(cuda_before) or any(not torch.equal(a, b) for a, b in zip(cuda_before, after)):
                    raise RuntimeError("shadow: boundary scoring consumed CUDA RNG; selections must be deterministic")

    # --------------------------------------------------------------- selection
    def _selection_context(self):
        if self._selection_meta is None:
            self._selection_meta = [(bs, s, e, slot) for bs in self._bucket_states for (slot, s, e) in bs.param_spans]
        return self._selection_meta

    def _mask_arena_pair(self):
        if self._mask_arenas is None:
            arena = self._ddp.arena
            self._mask_arenas = [torch.zeros(arena.numel, dtype=torch.uint8, device=arena.device) for _ in range(2)]
        return self._mask_arenas

    def _active_mask_arena(self):
        return self._mask_arena_pair()[self._mask_turn]

    def _run_selection(self, views, meta) -> Support:
        forced = [id(m[3]) in self._forced_slots for m in meta] if self._always_sync_layers is not None else None
        has_forced = any(forced) if forced else False
        sel_views = [v for v, f in zip(views, forced) if not f] if has_forced else views
        hook = getattr(self.selection, "warmup_sync_target", None)
        ctx = SelectionContext(sel_views, self._dp_group(),
                               hook(self._cycle.start_iter, self._cycle.period) if callable(hook) else None)
        sel_masks = self.selection.select(ctx)
        if has_forced:
            if len(sel_masks) != len(sel_views):
                raise SGAEngineError(f"selection plugin '{type(self.selection).__name__}' returned {len(sel_masks)} "
                                     f"masks for {len(sel_views)} eligible views")
            it = iter(sel_masks)
            masks = [torch.ones(e - s, dtype=torch.uint8, device=v.device) if f else next(it)
                     for f, (_bs, s, e, _p), v in zip(forced, meta, views)]
        else:
            masks = sel_masks
        bucket_masks = self._assemble_bucket_masks(masks, meta)
        if self._support_consistency:
            self._verify_support_consistency(bucket_masks)
        return self._support_from_bucket_masks(bucket_masks)

    def _support_from_bucket_masks(self, bucket_masks) -> Support:
        x = getattr(self.selection, "block_size", 1)
        if self._idx_pools is None:
            self._idx_pools = [IndexPool(self._ddp.arena.device) for _ in self._bucket_states]
        return Support([
            BucketSupport(m, idx_pool=self._idx_pools[i], block_size=x,
                          block_spans=(sorted((s, e) for (_p, s, e) in self._bucket_states[i].param_spans)
                                       if x > 1 else None))
            for i, m in enumerate(bucket_masks)])

    # ------------------------------------------------------ continuation state
    def state_dict(self) -> dict:
        """What a checkpoint of the optimizer does not hold and a bit-continuous resume needs: this rank's
        residual (the gradient arena), the active support, the step counter, the calendar's pending forced
        step and the selection plugin's running state. The reference keeps none of it (its resumed engine
        cold-starts with dense steps until the next boundary, ``sga/engine.py:488-494``); saving it is opt-in."""
        arena = self._ddp.arena
        hook = getattr(self.selection, "state_dict", None)
        sel = hook() if callable(hook) else {}
        return {"iter": self._iter, "residual": arena.main_grad.detach().cpu().clone(),
                "mask": (self._active_mask_arena().detach().cpu().clone() if self._active_support is not None else None),
                "force_next": bool(getattr(self._cycle, "force_next", False)), "selection": sel,
                "last_ratio": self.last_ratio}

    def load_state_dict(self, state: dict) -> None:
        arena = self._ddp.arena
        if state["residual"].numel() != arena.main_grad.numel():
            raise ValueError("saved SGA state belongs to another parameter layout")
        arena.main_grad.copy_(state["residual"].to(arena.device))
        self._iter, self._first_step = state["iter"], False
        self._cycle.force_next = bool(state.get("force_next", False))
        hook = getattr(self.selection, "load_state_dict", None)
        if callable(hook) and state.get("selection"):
            hook(state["selection"])
        if state.get("mask") is not None:
            inactive = self._mask_arena_pair()[1 - self._mask_turn]
            inactive.copy_(state["mask"].to(arena.device))
            masks = [inactive[bs.arena_start:bs.arena_start + bs.grad_data.numel()] for bs in self._bucket_states]
            self._activate_support(self._support_from_bucket_masks(masks))
        self.last_ratio = state.get("last_ratio", self.last_ratio)

    def _assemble_bucket_masks(self, masks, meta):
        """Write the per-parameter masks into the inactive arena-wide mask buffer
        (ping-pong: the outgoing support's mask stays intact until the switch)."""
        inactive = self._mask_arena_pair()[1 - self._mask_turn]
        inactive.zero_()
        for m, (bs, s, e, _p) in zip(masks, meta):
            inactive[bs.arena_start + s:bs.arena_start + e] = m
        return [inactive[bs.arena_start:bs.arena_start + bs.grad_data.numel()] for bs in self._bucket_states]

    def _activate_support(self, support: Support) -> None:
        self._mask_turn = 1 - self._mask_turn
        self._active_support = support
        for bs, sup in zip(self._bucket_states, support.buckets):
            bs.active_mask_u8 = sup.mask_u8
            sup.num_selected()
            if self.backend.consumes == "idx":
                if self._backend_layout == "bb":
                    _ = sup.block_desc if getattr(self.backend, "block_form", "") == "block_desc" else sup.block_idx
                else:
                    _ = sup.idx
        hook = getattr(self.backend, "on_support_activated", None)
        if callable(hook):
            hook(support, self._bucket_states)
        self.last_ratio = support.total_selected / max(support.total_elements, 1)

    # ------------------------------------------------------------------- clip
    def _masked_clip_grad_norm(self, optimizer, was_full, step, shadow=False, scale_now=False):
        """Norm over what was communicated this step; returns ``(norm, coeff)``.
        On CUDA both stay on the device (``coeff`` is a device scalar the
        optimizer kernel reads); the norm is fetched once, for the log."""
        clip = float(getattr(optimizer.config, "clip_grad", 0.0) or 0.0)
        arena = self._ddp.arena
        ddp = self._ddp
        world = ddp.world
        cuda = arena.device.type == "cuda"
        mask = None if was_full else (self._active_mask_arena() if self._mask_in_use(False) else None)
        fused = (not was_full) and getattr(self.backend, "sumsq", None) is not None and ddp.transport == "p2p"
        if cuda:
            from .. import kernels as K

            sumsq = self._dev["sumsq"]
            if fused:
                sumsq.copy_(self.backend.sumsq)
            elif (not was_full) and self.rank_local and self.backend.consumes == "idx":
                K.sumsq(arena.comm, sumsq)
            elif (not was_full) and self._compact_values and not self.rank_local:
                first = True
                for bs in self._bucket_states:
                    vals = self._compact_values.get(id(bs))
                    if vals is not None and vals.numel():
                        K.sumsq(vals, sumsq, accumulate=not first)
                        first = False
                if first:
                    sumsq.zero_()
            else:
                K.sumsq(arena.main_grad, sumsq, mask=mask)
            reduced_over_dp = not (world > 1 and ddp.transport != "p2p")
            if self.model_parallel_norm is not None:
                # shards of other tensor-parallel ranks join the norm; replicated parameters count once
                if (not was_full) and self._compact_values and not self.rank_local:
                    raise NotImplementedError("tensor parallelism with compact shared supports: use "
                                              "--sga-selection-locality rank_local or a mask backend")
                src = arena.comm if ((not was_full) and self.rank_local and self.backend.consumes == "idx") \
                    else arena.main_grad
                self.model_parallel_norm(sumsq, src, mask if src is arena.main_grad else None)
            if not reduced_over_dp:
                dist.all_reduce(sumsq, op=dist.ReduceOp.SUM, group=ddp.group)  # DP-bitwise fix
                K.clip_coeff(sumsq, 1.0 / world, clip, self._dev["coeff"], self._dev["norm"])
            else:
                K.clip_coeff(sumsq, 1.0, clip, self._dev["coeff"], self._dev["norm"])
            wants_dump = scale_now or (self._trace is not None and any(self._trace.wants(step)))
            if wants_dump and clip > 0.0:
                # the dump slot reads post-clip gradients: scale explicitly, hand the kernel 1.0
                self._scale_communicated(was_full, mask)
                return _LazyNorm(self._dev["norm"]), 1.0
            return _LazyNorm(self._dev["norm"]), (self._dev["coeff"] if clip > 0.0 else 1.0)
        # CPU path
        if (not was_full) and self.rank_local and self.backend.consumes == "idx":
            total = float((arena.comm.double() ** 2).sum())
        elif mask is not None:
            total = float((torch.where(mask > 0, arena.main_grad, torch.zeros_like(arena.main_grad)).double() ** 2).sum())
        else:
            total = float((arena.main_grad.double() ** 2).sum())
        t = torch.tensor([total], dtype=torch.float64)
        if self.model_parallel_norm is not None:
            src = arena.comm if ((not was_full) and self.rank_local and self.backend.consumes == "idx") \
                else arena.main_grad
            self.model_parallel_norm(t, src, mask if src is arena.main_grad else None)
        if world > 1 and dist.is_initialized():
            dist.all_reduce(t, op=dist.ReduceOp.SUM, group=ddp.group)
            t /= world
        norm = float(t.sqrt().item())
        coeff = 1.0
        if clip > 0.0:
            c = clip / (norm + 1.0e-6)
            if c < 1.0:
                coeff = float(torch.tensor(c, dtype=torch.float32).item())
        wants_dump = scale_now or (self._trace is not None and any(self._trace.wants(step)))
        if wants_dump and coeff != 1.0:
            self._scale_communicated(was_full, mask, coeff)
            return norm, 1.0
        return norm, coeff

    def _scale_communicated(self, was_full, mask, coeff=None) -> None:
        arena = self._ddp.arena
        target = arena.comm if (self.rank_local and not was_full and self.backend.consumes == "idx") else arena.main_grad
        if arena.device.type == "cuda":
            c = self._dev["coeff"]
            if mask is None:
                from .. import kernels as K

                K.scale_(target, c)
            else:
                target.mul_(torch.where(mask > 0, c, self._dev["one"]))
        else:
            if mask is None:
                target.mul_(coeff)
            else:
                target[mask > 0] *= coeff

    def _count_zeros(self):
        g = self._ddp.arena.main_grad
        pad = self._ddp.arena.numel - sum(s.end - s.start for s in self._ddp.arena.slots)
        return float(g.numel() - int(torch.count_nonzero(g).item()) - pad)

    # ----------------------------------------------------------------- checks
    def _check_counts(self) -> None:
        group = self._dp_group()
        if group is None or self._active_support is None or not dist.is_initialized():
            return
        ks = [b.num_selected() for b in self._active_support.buckets]
        dev = self._ddp.arena.device
        t = torch.tensor(ks, dtype=torch.int64, device=dev)
        packed = torch.stack([t, -t], dim=1).flatten()
        dist.all_reduce(packed, op=dist.ReduceOp.MAX, group=group)
        maxs = packed[0::2].tolist()
        mins = [-v for v in packed[1::2].tolist()]
        if maxs != mins:
            raise SGAEngineError(f"SGA support count mismatch across ranks: local ks={ks}, cluster min={mins}, "
                                 f"max={maxs}. Refusing the mismatched collective (it would deadlock or corrupt).")

    def _verify_support_consistency(self, masks) -> None:
        group = self._dp_group()
        if group is None or not dist.is_initialized():
            return
        dev = masks[0].device
        sums = torch.zeros(2 * len(masks), dtype=torch.int64, device=dev)
        for i, m in enumerate(masks):
            if m.is_cuda:
                from .. import kernels as K

                st = K.mask_stats(m)
            else:
                from .. import kernels_torch as KT

                st = KT.mask_stats(m)
            sums[2 * i] = st[1]
            sums[2 * i + 1] = st[2]
        lo, hi = sums.clone(), sums.clone()
        dist.all_reduce(lo, op=dist.ReduceOp.MIN, group=group)
        dist.all_reduce(hi, op=dist.ReduceOp.MAX, group=group)
        if not torch.equal(lo, hi):
            raise SGAEngineError(f"SGA support checksum mismatch across ranks (dual-value MIN {lo.tolist()} != MAX "
                                 f"{hi.tolist()}); masks diverged.")

    def _check_norm_spread(self, tensors) -> None:
        group = self._dp_group()
        if group is None or not tensors or not dist.is_initialized():
            return
        norms = torch.stack([t.float().pow(2).sum() for t in tensors])
        lo, hi = norms.clone(), norms.clone()
        dist.all_reduce(lo, op=dist.ReduceOp.MIN, group=group)
        dist.all_reduce(hi, op=dist.ReduceOp.MAX, group=group)
        spread = ((hi - lo) / hi.clamp(min=torch.finfo(torch.float32).tiny)).max().item()
        if spread > 1.0e-6:
            raise SGAEngineError(f"SGA scoring-input norm spread across ranks {spread:.3e} > 1e-6; the upstream "
                                 "full sync is inconsistent -- refusing to score.")

    # ------------------------------------------------------------------ state
    def _full_clear(self) -> None:
        arena = self._ddp.arena
        arena.main_grad.zero_()
        if arena.comm is not None:
            arena.comm.zero_()
        self._compact_values = {}

    def _refresh_records(self, optimizer):
        """Per-parameter records over the arena (trace collector, shadow scorer)."""
        arena = self._ddp.arena
        step = optimizer.peek_step()
        recs = []
        for bs in self._bucket_states:
            for (slot, s, e) in bs.param_spans:
                grp = optimizer.param_groups[slot.spec.group]
                sl = slice(slot.start, slot.end)
                recs.append(ParamRecord(
                    model_param=slot.model, main_param=slot.main, bucket_state=bs, start=s, end=e, lr=grp["lr"],
                    beta1=grp["betas"][0], beta2=grp["betas"][1], eps=grp["eps"], weight_decay=grp["weight_decay"],
                    step=step, name=slot.name, grad=slot.grad, m=arena.exp_avg[sl].view(slot.spec.shape),
                    v=arena.exp_avg_sq[sl].view(slot.spec.shape), group=slot.spec.group))
        self._records = recs
        return recs

    # ---------------------------------------------------------------- logging
    def _log_step(self, step, was_full, reselected, grad_norm) -> None:
        if self.log_interval <= 0 or step % self.log_interval:
            return
        # line and record of sga/engine.py:1451-1472: the ratio is the active support's selected fraction
        # (-1 while there is none, bootstrap and dense steps included), the threshold is the last selection's
        if self.rank_local:
            ratio = 1.0 if was_full else self._ratio
        elif self._active_support is not None and self._active_support.total_elements:
            ratio = self._active_support.total_selected / self._active_support.total_elements
        else:
            ratio = -1.0
        gn = float(grad_norm) if grad_norm is not None else float("nan")
        if self._rank != 0:
            return
        thr = getattr(self.selection, "last_threshold", None)
        extra = f" sel_thresh={thr:.3e}" if thr else ""
        print(f"[SGA] step={step} phase={'full' if was_full else 'sparse'} ratio={ratio:.4f}{extra} "
              f"grad_norm={gn:.3f}", flush=True)
        if self._metrics_file:
            with open(self._metrics_file, "a") as fh:
                fh.write(json.dumps({"step": step, "phase": "full" if was_full else "sparse", "ratio": ratio,
                                     "grad_norm": gn, "reselected": bool(reselected)}) + "\n")


class _LazyNorm:
    """A device scalar that turns into a float on first use (one host sync, at log time)."""

    def __init__(self, t):
        self._t = t
        self._v = None

    def __float__(self):
        if self._v is None:
            self._v = float(self._t.item())
        return self._v

    def item(self):
        return float(self)

    def __format__(self, spec):
        return format(float(self), spec)

    def __repr__(self):
        return repr(float(self))
