"""The SGA args singleton (bottom of the import graph: argparse only).

``set_args`` / ``get_args`` hold the one validated namespace that the engine
builder seeds from the trainer's arguments; plugins read their knobs from it in
zero-argument constructors. Mirrors ``sga/config/__init__.py:32-69``.
"""
from __future__ import annotations

import argparse

from .arguments import add_sga_args, sga_bool, sga_int_or_null  # noqa: F401
from .validation import (parse_branch_points, parse_layer_patterns, sga_actions, sga_defaults,  # noqa: F401
                         validate_sga_args)

_ARGS = None

# sga_* attributes that are run plumbing rather than configuration identity
# (excluded from the resume guard's comparison).
NON_CONFIG_SGA_KEYS = frozenset({"sga_allow_config_override", "sga_backend_timer"})


def set_args(ns) -> None:
    global _ARGS
    _ARGS = ns


def get_args():
    if _ARGS is None:
        raise RuntimeError("sga args are not set (call sga_b200.config.set_args or build_engine first)")
    return _ARGS


def sga_config_attrs(ns) -> dict:
    """The ``sga_*`` attributes of ``ns`` that make up the run's SGA identity."""
    out = {}
    for key in sorted(vars(ns)):
        if key.startswith("sga_") and key not in NON_CONFIG_SGA_KEYS:
            out[key] = getattr(ns, key)
    return out


def copy_from_trainer_args(src) -> argparse.Namespace:
    """A fresh namespace with every ``sga_*`` default, overlaid by ``src``'s
    ``sga_*`` attributes plus the few trainer fields validation consults."""
    ns = argparse.Namespace(**sga_defaults())
    for key, val in vars(src).items():
        if key.startswith("sga_"):
            setattr(ns, key, val)
    for key in ("train_iters", "pipeline_model_parallel_size", "tensor_model_parallel_size"):
        setattr(ns, key, getattr(src, key, None))
    return ns


def make_args(**overrides) -> argparse.Namespace:
    """Namespace of declared defaults with ``overrides`` applied (tests, tools)."""
    ns = argparse.Namespace(**sga_defaults())
    ns.train_iters = overrides.pop("train_iters", None)
    ns.pipeline_model_parallel_size = overrides.pop("pipeline_model_parallel_size", 1)
    ns.tensor_model_parallel_size = overrides.pop("tensor_model_parallel_size", 1)
    for k, v in overrides.items():
        if not hasattr(ns, k):
            raise AttributeError(f"unknown sga arg '{k}'")
        setattr(ns, k, v)
    return ns
