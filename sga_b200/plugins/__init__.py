"""Name -> class tables of the three class-valued plugin axes (selection,
optimizer, backend) and the two ``auto`` resolutions shared by validation and
the backends. The score axis is data, not classes (``plugins/scores.py``).

A table is filled lazily with the built-in plugins the first time it is asked
for a name; a name registered earlier (by a test or an extension) is kept.
Public surface as in ``sga/plugins/__init__.py:57-153``: ``register_*``,
``build_*``, ``plugin_class``, ``resolve_emission``, ``resolve_layout``.
"""
from __future__ import annotations

import importlib

# axis -> {name: class}
_TABLES: dict = {"selection": {}, "optimizer": {}, "backend": {}}

# axis -> {name: (module relative to this package's parent, attribute)}: the built-ins
_BUILTIN = {
    "selection": {"topk": ("plugins.selection.topk", "TopkSelection")},
    "optimizer": {"adamw": ("plugins.optimizer.adam", "SgaAdamW"), "adams": ("plugins.optimizer.adam", "SgaAdamS")},
    "backend": {"torch_pipelined_index": ("backends.torch_pipelined_index", "TorchPipelinedIndexBackend"),
                "torch_pipelined_mask": ("backends.torch_pipelined_mask", "TorchPipelinedMaskBackend"),
                "nccl_pipelined_index": ("backends.nccl_pipelined_index", "NcclPipelinedIndexBackend")},
}


def resolve_emission(value, inherent):
    """An explicit emission wins; ``None`` / ``auto`` means the backend's own form."""
    return value if value not in (None, "auto") else inherent


def resolve_layout(layout, block_size):
    """An explicit layout wins; ``auto`` is ``er`` for single elements and ``bb`` for blocks."""
    if layout not in (None, "auto"):
        return layout
    return "bb" if block_size != 1 else "er"


def _add(axis: str, name: str, cls) -> None:
    table = _TABLES[axis]
    if name in table:
        raise ValueError(f"Duplicate {axis} registration for '{name}'")
    table[name] = cls


def register_selection(name, cls):
    _add("selection", name, cls)


def register_optimizer(name, cls):
    _add("optimizer", name, cls)


def register_backend_plugin(name, cls):
    _add("backend", name, cls)


def register_default_plugins() -> None:
    """Import the built-in plugins into the tables (idempotent; existing names are kept)."""
    root = __name__.rsplit(".", 1)[0]
    for axis, names in _BUILTIN.items():
        for name, (module, attr) in names.items():
            if name not in _TABLES[axis]:
                _TABLES[axis][name] = getattr(importlib.import_module(f"{root}.{module}"), attr)


def plugin_class(axis: str, name: str):
    register_default_plugins()
    table = _TABLES[axis]
    if name not in table:
        raise ValueError(f"Unknown SGA {axis} plugin '{name}'. Registered: {sorted(table)}")
    return table[name]


def build_selection(name):
    return plugin_class("selection", name)()


def build_optimizer(name):
    return plugin_class("optimizer", name)()


def build_backend_plugin(name):
    return plugin_class("backend", name)()
