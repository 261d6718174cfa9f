"""Declarations of every ``--sga-*`` flag.

One flat vocabulary is the whole configuration surface: a yaml ``sga:`` key,
the command-line flag (``-`` for ``_``), the attribute on the parsed namespace
and the attribute stored in a checkpoint are the same name. This file only
declares; rules that need more than one argument live in ``validation.py``,
which learns the vocabulary by introspecting the parser built here.

The first 44 flags reproduce the reference surface
(``sga/config/arguments.py:91-477``) name for name, type for type and default
for default. The flags in the last group are additions of this framework:
they select the rank-local per-bucket top-k exchange and the in-kernel
peer-memory transport, which the reference does not have.
"""
from __future__ import annotations

import argparse

SCORE_CHOICES = ("abs_g", "abs_m", "coi", "update")


def sga_bool(text):
    """``"true"`` / ``"false"`` in any case -> ``bool``; real bools pass through."""
    if isinstance(text, bool):
        return text
    low = str(text).strip().lower()
    if low in ("true", "false"):
        return low == "true"
    raise argparse.ArgumentTypeError(f"expected 'true' or 'false', got {text!r}")


def sga_int_or_null(text):
    """An int, or the spelling ``null`` (-> ``None``)."""
    if text is None:
        return None
    if isinstance(text, str) and text.strip().lower() == "null":
        return None
    return int(text)


def _core(p):
    g = p.add_argument_group("SGA core")
    g.add_argument("--sga-enabled", type=sga_bool, default=False,
                   help="Master switch. false (or no --sga-* flag at all) is plain dense training "
                        "and no other SGA flag is looked at.")
    g.add_argument("--sga-shadow", type=sga_bool, default=False,
                   help="Shadow mode: run the stock dense step unchanged and only read optimizer "
                        "state at cycle boundaries (for offline analysis and trace capture).")
    g.add_argument("--sga-shadow-score", type=sga_bool, default=True,
                   help="false also drops the read-only boundary scoring of a shadow run. Only "
                        "meaningful with --sga-shadow true.")
    g.add_argument("--sga-always-sync-layers", type=str, default=None,
                   help="Comma-joined substrings of parameter names that are communicated in "
                        "full every step: they leave the top-k pool and its denominator and are "
                        "forced into every support. Refused with pipeline parallelism > 1.")


def _cycle(p):
    g = p.add_argument_group("SGA cycle")
    g.add_argument("--sga-cycle-start-iter", type=int, default=0,
                   help="Step at which the reselection calendar is anchored; steps up to it are "
                        "dense warm-up and the first reselection is at start + period.")
    g.add_argument("--sga-cycle-start-iter-percent", type=float, default=None,
                   help="The same anchor as a percentage of train-iters ([0, 100]); resolved "
                        "into --sga-cycle-start-iter during validation. Not with an explicit "
                        "--sga-cycle-start-iter.")
    g.add_argument("--sga-cycle-period", type=int, default=1,
                   help="Reselection period T >= 1: a new support every T steps at a full-sync "
                        "boundary; the support is frozen in between. With rank-local selection "
                        "T is the dense flush interval and 0 means never flush.")
    g.add_argument("--sga-cycle-decouple-full-sync-interval-and-period", type=sga_bool, default=False,
                   help="Allow extra full syncs inside a period; needs "
                        "--sga-cycle-full-sync-interval.")
    g.add_argument("--sga-cycle-full-sync-interval", type=int, default=None,
                   help="Full sync every N steps, N a strict divisor of the period. Only with "
                        "the decouple switch.")


def _checks(p):
    g = p.add_argument_group("SGA checks")
    g.add_argument("--sga-checks", type=sga_bool, default=True,
                   help="Master over all consistency checks; false forces every check below off.")
    g.add_argument("--sga-checks-count-guard", type=sga_bool, default=True,
                   help="Layer 1: cross-rank agreement of the selected element counts at each "
                        "support activation.")
    g.add_argument("--sga-checks-support-consistency", type=sga_bool, default=True,
                   help="Layer 2: two position checksums of the selected support compared "
                        "across ranks at every reselection.")
    g.add_argument("--sga-checks-norm-spread", type=sga_bool, default=True,
                   help="Layer 3: cross-rank spread of the norms of the scoring inputs before a "
                        "reselection.")
    g.add_argument("--sga-checks-rng-bracket", type=sga_bool, default=True,
                   help="Shadow runs: assert that boundary scoring consumed no CPU or CUDA RNG.")


def _trace(p):
    g = p.add_argument_group("SGA trace")
    g.add_argument("--sga-trace-dir", type=str, default=None,
                   help="Trace output directory; setting it turns the collector on.")
    g.add_argument("--sga-trace-branch-points", type=str, default=None,
                   help="Comma-joined steps at which the full optimizer state is dumped.")
    g.add_argument("--sga-trace-window", type=int, default=100,
                   help="Number of steps after each branch point whose gradients are dumped.")
    g.add_argument("--sga-trace-dump-dtype", type=str, default="fp32", choices=("fp32", "bf16"),
                   help="Storage dtype of the gradient payloads; state files stay fp32.")
    g.add_argument("--sga-trace-async", type=sga_bool, default=False,
                   help="Write gradient files from a background writer.")
    g.add_argument("--sga-trace-async-backend", type=str, default="cpu_snapshot",
                   choices=("cpu_snapshot", "pinned_cuda"),
                   help="How the async writer snapshots a step: a blocking CPU copy, or a "
                        "non-blocking device-to-host copy into reusable pinned slots.")
    g.add_argument("--sga-trace-async-queue-depth", type=int, default=2,
                   help="Most gradient items in flight before the dump slot blocks.")
    g.add_argument("--sga-trace-async-worker-count", type=int, default=1,
                   help="Writer threads; at most the queue depth.")
    g.add_argument("--sga-trace-async-max-workset-gib", type=float, default=16.0,
                   help="Cap on the host memory the async path may hold, in GiB.")


def _score(p):
    g = p.add_argument_group("SGA score")
    g.add_argument("--sga-score", type=str, default=None, choices=SCORE_CHOICES,
                   help="Boundary score (required when enabled).")


def _selection(p):
    g = p.add_argument_group("SGA selection")
    g.add_argument("--sga-selection", type=str, default="topk", help="Selection plugin name.")
    g.add_argument("--sga-selection-method", type=str, default=None,
                   choices=("adaptive", "exact", "histogram"),
                   help="adaptive = persistent threshold controller; exact = k-th value plus "
                        "OR-merge; histogram = bit-pattern histogram select.")
    g.add_argument("--sga-selection-ratio-percent", type=float, default=None,
                   help="Selected fraction in percent, strictly inside (0, 100).")
    g.add_argument("--sga-selection-histogram-mode", type=str, default="exact",
                   choices=("balanced", "exact", "fast"), help="Histogram geometry tier.")
    g.add_argument("--sga-selection-topk-histogram-add-global-allreduce", type=sga_bool, default=False,
                   help="SUM-all-reduce the per-rank histograms before the threshold select.")
    g.add_argument("--sga-selection-adaptive-warmup-syncs", type=sga_int_or_null, default=5,
                   help="Gated warm-up selects before the persistent threshold takes over; "
                        "'null' disables the gate.")
    g.add_argument("--sga-selection-adaptive-warmup-mode", type=str, default="fast",
                   choices=("balanced", "exact", "fast"),
                   help="Histogram tier used to bootstrap the adaptive threshold.")
    g.add_argument("--sga-selection-block-size", type=int, default=1,
                   help="Select contiguous blocks of this many elements (power of two in "
                        "[1, 1024]); 1 is element-granular. Histogram method only.")
    g.add_argument("--sga-selection-block-reduce", type=str, default="mean", choices=("mean", "max"),
                   help="Per-block score: mean or max of |score| over the block's real length.")


def _optimizer(p):
    g = p.add_argument_group("SGA optimizer")
    g.add_argument("--sga-optimizer", type=str, default="adamw",
                   help="adamw, or adams (second moment rebuilt from the pre-commit first "
                        "moment, no bias correction).")
    g.add_argument("--sga-optimizer-residual-mean", type=sga_bool, default=False,
                   help="Divide the accumulated residual by the fold window on the step before "
                        "a full sync.")
    g.add_argument("--sga-optimizer-full-sync-inactive-lr-scale", type=float, default=1.0,
                   help="On full steps, apply lr * scale at coordinates outside the outgoing "
                        "support. Refused in shadow mode and with period 1 when != 1.")
    g.add_argument("--sga-optimizer-compact-search", type=str, default="table",
                   choices=("table", "bisection"),
                   help="How the compact sparse step aligns bucket-sorted indices with a "
                        "parameter span.")


def _backend(p):
    g = p.add_argument_group("SGA backend")
    g.add_argument("--sga-backend", type=str, default="dense",
                   help="dense | torch_pipelined_index | torch_pipelined_mask | "
                        "nccl_pipelined_index.")
    g.add_argument("--sga-backend-emission", type=str, default="auto",
                   choices=("auto", "compact", "writeback"),
                   help="Hand-off of the reduced values: kept compact, or scattered back into "
                        "the dense gradient buffer.")
    g.add_argument("--sga-backend-layout", type=str, default="auto", choices=("auto", "er", "eb", "bb"),
                   help="Index form on the wire: element selection + element index, block "
                        "selection + element index, or block selection + block index.")
    g.add_argument("--sga-backend-high-priority-group", type=sga_bool, default=False,
                   help="torch_pipelined_index: run the sparse collectives on a twin "
                        "high-priority communicator / stream.")
    g.add_argument("--sga-backend-index-slices", type=int, default=2,
                   help="torch_pipelined_index: pipeline slices per bucket (>= 1).")
    g.add_argument("--sga-backend-mask-slices", type=int, default=2,
                   help="torch_pipelined_mask: pipeline slices per bucket (>= 1).")
    g.add_argument("--sga-backend-timer", type=str, default=None,
                   help="Directory for isolated, synchronised timings of the comm regions "
                        "(per-rank JSONL). A breakdown instrument, never a throughput number.")


def _b200(p):
    g = p.add_argument_group("SGA B200 extensions (not in the reference)")
    g.add_argument("--sga-selection-locality", type=str, default="shared", choices=("shared", "rank_local"),
                   help="shared: one support for all ranks, chosen at cycle boundaries from "
                        "dense-averaged scores (the reference semantics). rank_local: every "
                        "sparse step each rank takes the exact per-bucket top-k of "
                        "|grad + residual| and exchanges (index, value) pairs.")
    g.add_argument("--sga-backend-transport", type=str, default="auto", choices=("auto", "p2p", "nccl"),
                   help="p2p: fused CUDA kernels that read and write peer memory over NVLink. "
                        "nccl: library collectives (the baseline arm). auto picks p2p on CUDA "
                        "with more than one rank on a node, nccl/gloo otherwise.")
    g.add_argument("--sga-bucket-elems", type=int, default=16 * 1024 * 1024,
                   help="Target gradient bucket size in elements (fp32); 16 Mi keeps a bucket "
                        "inside the L2 between the select passes.")


def add_sga_args(parser: argparse.ArgumentParser) -> argparse.ArgumentParser:
    for fn in (_core, _cycle, _checks, _trace, _score, _selection, _optimizer, _backend, _b200):
        fn(parser)
    return parser
