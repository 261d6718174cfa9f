"""Plugin registries for the three class-valued axes (selection, optimizer,
backend) and the shared ``auto`` resolutions of emission and layout.

The score axis is data, not classes (``plugins/scores.py``). Mirrors
``sga/plugins/__init__.py:57-153``.
"""
from __future__ import annotations

_SELECTIONS: dict = {}
_OPTIMIZERS: dict = {}
_BACKENDS: dict = {}
_REGISTRIES = {"selection": _SELECTIONS, "optimizer": _OPTIMIZERS, "backend": _BACKENDS}


def resolve_emission(value, inherent):
    """``None`` / ``auto`` -> the backend's inherent form; explicit values win."""
    return inherent if value in (None, "auto") else value


def resolve_layout(layout, block_size):
    """``auto`` -> ``er`` for element-granular selection, ``bb`` for blocks."""
    if layout not in (None, "auto"):
        return layout
    return "er" if block_size == 1 else "bb"


def _register(reg, axis, name, cls):
    if name in reg:
        raise ValueError(f"Duplicate {axis} registration for '{name}'")
    reg[name] = cls


def register_selection(name, cls):
    _register(_SELECTIONS, "selection", name, cls)


def register_optimizer(name, cls):
    _register(_OPTIMIZERS, "optimizer", name, cls)


def register_backend_plugin(name, cls):
    _register(_BACKENDS, "backend", name, cls)


def register_default_plugins() -> None:
    """Idempotent; a name a test registered first is never overwritten."""
    from ..backends.nccl_pipelined_index import NcclPipelinedIndexBackend
    from ..backends.torch_pipelined_index import TorchPipelinedIndexBackend
    from ..backends.torch_pipelined_mask import TorchPipelinedMaskBackend
    from .optimizer.adam import SgaAdamS, SgaAdamW
    from .selection.topk import TopkSelection

    _SELECTIONS.setdefault("topk", TopkSelection)
    _OPTIMIZERS.setdefault("adamw", SgaAdamW)
    _OPTIMIZERS.setdefault("adams", SgaAdamS)
    _BACKENDS.setdefault("torch_pipelined_index", TorchPipelinedIndexBackend)
    _BACKENDS.setdefault("torch_pipelined_mask", TorchPipelinedMaskBackend)
    _BACKENDS.setdefault("nccl_pipelined_index", NcclPipelinedIndexBackend)


def plugin_class(axis: str, name: str):
    registry = _REGISTRIES[axis]
    register_default_plugins()
    try:
        return registry[name]
    except KeyError:
        raise ValueError(f"Unknown SGA {axis} plugin '{name}'. Registered: {sorted(registry)}") from None


def build_selection(name):
    return plugin_class("selection", name)()


def build_optimizer(name):
    return plugin_class("optimizer", name)()


def build_backend_plugin(name):
    return plugin_class("backend", name)()
