"""Engine builder: seeds the SGA args singleton from the trainer's arguments,
validates, refuses what the engine cannot drive, builds the three plugins and
returns the engine.

Refusal list (``sga/runtime.py:23-142``), adapted to this framework's trainer:
the distributed optimizer, fp16 / loss scaling, per-token loss, virtual
pipeline stages, expert parallelism and CUDA-graph capture of the whole step
are refused; pipeline parallelism is accepted only with untied embeddings and
no always-sync layers. Tensor parallelism is accepted here (the reference
refuses it): parameters replicated across tensor-parallel ranks are reduced
over that group before residual accounting, so no tensor-parallel collective
touches residual coordinates afterwards.
"""
from __future__ import annotations

import json

from .. import config as C
from ..plugins import build_backend_plugin, build_optimizer, build_selection, register_default_plugins
from .engine import SGAEngine

SGA_API_VERSION = 2


def _assert_args_compatible(args) -> None:
    def g(name, default=None):
        return getattr(args, name, default)

    if g("use_distributed_optimizer", False):
        raise ValueError("SGA requires use_distributed_optimizer=false (replicated optimizer state)")
    if g("fp16", False) or g("loss_scale", None):
        raise ValueError("SGA supports bf16 without loss scaling only")
    if g("calculate_per_token_loss", False):
        raise ValueError("SGA refuses calculate_per_token_loss")
    if (g("virtual_pipeline_model_parallel_size", None) or 1) > 1:
        raise ValueError("SGA refuses virtual pipeline stages")
    if (g("expert_model_parallel_size", 1) or 1) > 1 or g("num_experts", None):
        raise ValueError("SGA refuses expert parallelism / MoE")
    if g("enable_cuda_graph", False):
        raise ValueError("SGA refuses whole-step CUDA-graph capture (the step type changes per iteration)")
    pp = g("pipeline_model_parallel_size", 1) or 1
    if pp > 1:
        if not g("untie_embeddings_and_output_weights", False):
            raise ValueError("SGA with pipeline parallelism needs untied embeddings")
        if g("sga_always_sync_layers", None):
            raise ValueError("sga_always_sync_layers requires pipeline_model_parallel_size == 1")
    if g("rerun_mode", "disabled") not in (None, "disabled"):
        raise ValueError("SGA requires the rerun state machine to be disabled")


def build_engine(api_version: int = SGA_API_VERSION, trainer_args=None, quiet: bool = False) -> SGAEngine:
    if api_version != SGA_API_VERSION:
        raise ValueError(f"SGA api version mismatch: caller {api_version}, engine {SGA_API_VERSION}")
    if trainer_args is not None:
        C.set_args(C.copy_from_trainer_args(trainer_args))
    args = C.get_args()
    C.validate_sga_args(args)
    if not args.sga_enabled:
        raise ValueError("build_engine called with sga_enabled false")
    if trainer_args is not None:
        _assert_args_compatible(trainer_args)
    register_default_plugins()
    selection = build_selection(args.sga_selection)
    opt = build_optimizer(args.sga_optimizer)
    backend = build_backend_plugin(args.sga_backend)
    probe = getattr(backend, "validate_runtime", None)
    if callable(probe):
        probe(trainer_args if trainer_args is not None else args)
    engine = SGAEngine(args.sga_score, selection, opt, backend)
    if engine._rank == 0 and not quiet:
        print("[SGA] engine built: " + json.dumps(C.sga_config_attrs(args), sort_keys=True, default=str), flush=True)
    return engine
