"""Cross-argument rules for the ``sga_*`` namespace.

``validate_sga_args(args)`` raises ``ValueError`` naming the offending key, or
returns ``None`` after writing derived values back onto ``args`` (percent ->
absolute start step, comma tokens -> sorted lists, a false ``sga_checks``
forcing every ``sga_checks_*`` off, layout ``auto`` -> er/eb/bb). Nothing is
checked while ``sga_enabled`` is false. Defaults are never restated: they are
read from the parser that ``arguments.add_sga_args`` builds.

Rule set follows the reference (``sga/config/validation.py:130-514``); the
rank-local locality rules at the end are additions of this framework.
"""
from __future__ import annotations

import argparse
import math
import os

from .arguments import add_sga_args

_PARSER = None


def _parser() -> argparse.ArgumentParser:
    global _PARSER
    if _PARSER is None:
        _PARSER = argparse.ArgumentParser(add_help=False)
        add_sga_args(_PARSER)
    return _PARSER


def sga_actions() -> dict:
    """dest -> argparse action for every SGA flag."""
    return {a.dest: a for a in _parser()._actions if a.dest.startswith("sga_")}


def sga_defaults() -> dict:
    """dest -> declared default."""
    return {d: a.default for d, a in sga_actions().items()}


def parse_branch_points(raw):
    """Comma token, int, or list of ints -> sorted de-duplicated list (empty when unset)."""
    if raw is None:
        return []
    if isinstance(raw, bool):
        raise TypeError(f"branch points must be ints (got {raw!r})")
    if isinstance(raw, int):
        items = [raw]
    elif isinstance(raw, str):
        if not raw.strip():
            return []
        if raw.strip().lower() == "null":
            raise ValueError("'null' is not accepted here; leave the flag unset for no state dumps")
        items = [tok.strip() for tok in raw.split(",")]
    elif isinstance(raw, (list, tuple)):
        items = list(raw)
    else:
        raise TypeError(f"branch points must be a comma token or an int list (got {raw!r})")
    out = set()
    for it in items:
        if isinstance(it, bool):
            raise TypeError(f"branch points must be ints (got {it!r})")
        if isinstance(it, str):
            if not it or not it.lstrip("+-").isdigit():
                raise ValueError(f"not an integer step: {it!r}")
            it = int(it)
        if not isinstance(it, int):
            raise TypeError(f"branch points must be ints (got {it!r})")
        if it < 0:
            raise ValueError(f"branch points must be >= 0 (got {it})")
        out.add(it)
    return sorted(out)


def parse_layer_patterns(raw):
    """Always-sync patterns -> sorted de-duplicated list of non-empty strings, or None."""
    if raw is None:
        return None
    if isinstance(raw, str):
        if not raw.strip():
            return None
        items = raw.split(",")
    elif isinstance(raw, (list, tuple)):
        items = list(raw)
    else:
        raise ValueError(f"must be a comma-joined string or a list of strings (got {raw!r})")
    out = set()
    for it in items:
        if not isinstance(it, str) or not it.strip():
            raise ValueError(f"patterns must be non-empty strings (got {it!r})")
        pat = it.strip()
        if pat == "null":
            raise ValueError("'null' would match a parameter name literally; leave the flag unset instead")
        out.add(pat)
    return sorted(out) or None


def _is_int(x) -> bool:
    return isinstance(x, int) and not isinstance(x, bool)


def _validate_trace(args, dflt) -> None:
    keys = ("sga_trace_branch_points", "sga_trace_window", "sga_trace_dump_dtype", "sga_trace_async",
            "sga_trace_async_backend", "sga_trace_async_queue_depth", "sga_trace_async_worker_count",
            "sga_trace_async_max_workset_gib")
    present = args.sga_trace_dir is not None or any(getattr(args, k) != dflt[k] for k in keys)
    if not present:
        return
    if not isinstance(args.sga_trace_dir, str) or not args.sga_trace_dir:
        raise ValueError("sga_trace_dir is required (a non-empty path) once any trace key is set")
    if args.sga_trace_dump_dtype not in ("fp32", "bf16"):
        raise ValueError(f"sga_trace_dump_dtype must be 'fp32' or 'bf16' (got {args.sga_trace_dump_dtype!r})")
    if args.sga_trace_async_backend not in ("cpu_snapshot", "pinned_cuda"):
        raise ValueError("sga_trace_async_backend must be 'cpu_snapshot' or 'pinned_cuda' "
                         f"(got {args.sga_trace_async_backend!r})")
    if args.sga_trace_async_backend != "cpu_snapshot" and not args.sga_trace_async:
        raise ValueError("sga_trace_async_backend='pinned_cuda' requires sga_trace_async=true")
    try:
        args.sga_trace_branch_points = parse_branch_points(args.sga_trace_branch_points)
    except (TypeError, ValueError) as e:
        raise ValueError(f"sga_trace_branch_points: {e}") from None
    if not _is_int(args.sga_trace_window) or args.sga_trace_window < 1:
        raise ValueError(f"sga_trace_window must be an int >= 1 (got {args.sga_trace_window!r})")
    depth, workers = args.sga_trace_async_queue_depth, args.sga_trace_async_worker_count
    if not _is_int(depth) or depth < 1:
        raise ValueError(f"sga_trace_async_queue_depth must be an int >= 1 (got {depth!r})")
    if not _is_int(workers) or workers < 1:
        raise ValueError(f"sga_trace_async_worker_count must be an int >= 1 (got {workers!r})")
    if workers > depth:
        raise ValueError(f"sga_trace_async_worker_count must be <= sga_trace_async_queue_depth ({workers} > {depth})")
    gib = args.sga_trace_async_max_workset_gib
    if isinstance(gib, bool) or not isinstance(gib, (int, float)) or not math.isfinite(gib) or gib <= 0:
        raise ValueError(f"sga_trace_async_max_workset_gib must be a finite float > 0 (got {gib!r})")


def validate_sga_args(args=None) -> None:
    if args is None:
        from . import get_args

        args = get_args()
    if not args.sga_enabled:
        return
    from ..plugins import plugin_class, register_default_plugins, resolve_layout

    register_default_plugins()
    dflt = sga_defaults()
    # additions of this framework may be absent on hand-built namespaces
    for k in ("sga_selection_locality", "sga_backend_transport", "sga_bucket_elems"):
        if not hasattr(args, k):
            setattr(args, k, dflt[k])

    if not args.sga_checks:
        for d in dflt:
            if d.startswith("sga_checks_"):
                setattr(args, d, False)

    if args.sga_score is None:
        raise ValueError("sga_score is required when sga_enabled is true")
    if args.sga_backend == "dense":
        raise ValueError("sga_enabled is true but sga_backend is still 'dense'; name a sparse backend")
    plugin_class("selection", args.sga_selection)
    plugin_class("optimizer", args.sga_optimizer)
    plugin_class("backend", args.sga_backend)

    rank_local = args.sga_selection_locality == "rank_local"

    # ---- cycle
    if args.sga_cycle_start_iter_percent is not None:
        if args.sga_cycle_start_iter != dflt["sga_cycle_start_iter"]:
            raise ValueError("set either sga_cycle_start_iter or sga_cycle_start_iter_percent, not both")
        iters = getattr(args, "train_iters", None)
        if not iters or int(iters) <= 0:
            raise ValueError("sga_cycle_start_iter_percent requires train_iters > 0")
        pct = float(args.sga_cycle_start_iter_percent)
        if not 0.0 <= pct <= 100.0:
            raise ValueError(f"sga_cycle_start_iter_percent must be in [0, 100] (got {pct})")
        args.sga_cycle_start_iter = max(0, int(round(pct / 100.0 * int(iters))))
        args.sga_cycle_start_iter_percent = None
    period = int(args.sga_cycle_period)
    if period < 1 and not (rank_local and period == 0):
        raise ValueError("sga_cycle_period must be >= 1 (0 = never flush is accepted only with "
                         "sga_selection_locality rank_local)")
    decouple = bool(args.sga_cycle_decouple_full_sync_interval_and_period)
    interval = args.sga_cycle_full_sync_interval
    if not decouple:
        if interval is not None:
            raise ValueError(f"sga_cycle_full_sync_interval is set ({interval}) but the decouple switch is false")
    elif interval is None:
        raise ValueError("sga_cycle_decouple_full_sync_interval_and_period is true but "
                         f"sga_cycle_full_sync_interval is unset (period={period})")
    elif not (0 < int(interval) < period and period % int(interval) == 0):
        raise ValueError(f"sga_cycle_full_sync_interval ({interval}) must satisfy 0 < interval < period "
                         f"({period}) and period % interval == 0")

    _validate_trace(args, dflt)

    # ---- shadow
    shadow = bool(args.sga_shadow)
    if args.sga_shadow_score is not True and not shadow:
        raise ValueError("sga_shadow_score is set but sga_shadow is not true")
    if shadow and args.sga_optimizer == "adams":
        raise ValueError("sga_optimizer 'adams' is refused with sga_shadow true: shadow replicates the "
                         "stock AdamW step, so the run would not be AdamS")

    # ---- always-sync layers
    try:
        args.sga_always_sync_layers = parse_layer_patterns(args.sga_always_sync_layers)
    except ValueError as e:
        raise ValueError(f"sga_always_sync_layers: {e}") from None
    if args.sga_always_sync_layers is not None and int(getattr(args, "pipeline_model_parallel_size", 1) or 1) > 1:
        raise ValueError("sga_always_sync_layers requires pipeline_model_parallel_size == 1 "
                         "(matching is per rank over the attached stage's parameters)")

    # ---- dual lr
    scale = args.sga_optimizer_full_sync_inactive_lr_scale
    if scale != 1.0:
        if not math.isfinite(scale) or scale < 0.0:
            raise ValueError(f"sga_optimizer_full_sync_inactive_lr_scale must be a finite float >= 0 (got {scale!r})")
        if shadow:
            raise ValueError(f"sga_optimizer_full_sync_inactive_lr_scale ({scale!r}) is refused with sga_shadow true")
        if period == 1:
            raise ValueError(f"sga_optimizer_full_sync_inactive_lr_scale ({scale!r}) is refused with "
                             "sga_cycle_period 1: every step is a full sync")

    emission = args.sga_backend_emission
    if emission == "compact" and args.sga_backend != "torch_pipelined_index":
        raise ValueError(f"sga_backend_emission 'compact' is only supported by torch_pipelined_index "
                         f"(got backend '{args.sga_backend}')")

    # ---- selection
    if args.sga_selection == "topk":
        if args.sga_selection_method is None:
            raise ValueError("sga_selection_method is required by topk (adaptive | exact | histogram)")
        if args.sga_selection_ratio_percent is None:
            raise ValueError("sga_selection_ratio_percent is required by topk")
        ratio = args.sga_selection_ratio_percent
        if not isinstance(ratio, float) or not math.isfinite(ratio) or not 0.0 < ratio < 100.0:
            raise ValueError(f"sga_selection_ratio_percent must be a finite float in (0, 100) (got {ratio!r})")
        frozen_ok = args.sga_selection_method == "histogram" and args.sga_selection_histogram_mode == "balanced"
        if not frozen_ok and not rank_local:
            if os.environ.get("SGA_ALLOW_FROZEN_SELECTION") == "1":
                print("[sga] WARNING: selection freeze lifted by SGA_ALLOW_FROZEN_SELECTION=1 "
                      f"(method '{args.sga_selection_method}', mode '{args.sga_selection_histogram_mode}')",
                      flush=True)
            else:
                raise ValueError("selection is frozen to histogram balanced: got method "
                                 f"'{args.sga_selection_method}', mode '{args.sga_selection_histogram_mode}' "
                                 "(SGA_ALLOW_FROZEN_SELECTION=1 lifts the gate)")
        bs = args.sga_selection_block_size
        if not _is_int(bs) or bs < 1 or bs > 1024 or bs & (bs - 1):
            raise ValueError(f"sga_selection_block_size must be a power of two in [1, 1024] (got {bs!r})")
        if args.sga_selection_method != "histogram" and bs != dflt["sga_selection_block_size"]:
            raise ValueError("sga_selection_block_size only applies to the histogram method "
                             f"(got method '{args.sga_selection_method}')")
        explicit = args.sga_backend_layout != "auto"
        if not explicit:
            args.sga_backend_layout = resolve_layout(args.sga_backend_layout, bs)
        layout = args.sga_backend_layout
        if bs > 1:
            if args.sga_selection_histogram_mode == "fast":
                raise ValueError("sga_selection_block_size > 1 with sga_selection_histogram_mode 'fast': the "
                                 "lower-edge threshold over-selects and blocks amplify it (0.253 measured vs 0.20)")
            if layout == "er":
                raise ValueError(f"sga_backend_layout 'er' refuses sga_selection_block_size > 1 (got {bs})")
        elif explicit and layout in ("eb", "bb"):
            raise ValueError(f"sga_backend_layout '{layout}' refuses sga_selection_block_size == 1")
        if explicit and args.sga_backend == "torch_pipelined_mask":
            raise ValueError(f"sga_backend_layout '{layout}' is refused with backend torch_pipelined_mask "
                             "(no index form is ever built there)")
        if layout == "bb" and args.sga_backend == "torch_pipelined_index" and emission != "writeback":
            raise ValueError("sga_backend_layout 'bb' with backend torch_pipelined_index needs "
                             f"sga_backend_emission 'writeback' (got '{emission}')")
        if layout == "bb" and args.sga_backend == "nccl_pipelined_index" and not 4 <= bs <= 64:
            raise ValueError("sga_backend_layout 'bb' with backend nccl_pipelined_index bounds "
                             f"sga_selection_block_size to a power of two in [4, 64] (got {bs})")

    # ---- rank-local additions
    if rank_local:
        if shadow:
            raise ValueError("sga_selection_locality rank_local is refused with sga_shadow true")
        if args.sga_selection_block_size != 1:
            raise ValueError("sga_selection_locality rank_local is element-granular (block_size must be 1)")
        if args.sga_score != "abs_g" and args.sga_backend != "torch_pipelined_index":
            raise ValueError("sga_selection_locality rank_local with the mask backend scores |grad + residual| "
                             "(spelled sga_score abs_g); update / abs_m / coi need backend torch_pipelined_index")
        if decouple:
            raise ValueError("sga_selection_locality rank_local has no decoupled full-sync grid")
    if not _is_int(args.sga_bucket_elems) or args.sga_bucket_elems < 1024:
        raise ValueError(f"sga_bucket_elems must be an int >= 1024 (got {args.sga_bucket_elems!r})")
