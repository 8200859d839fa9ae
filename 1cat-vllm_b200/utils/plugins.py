"""Out-of-tree extension points loaded through Python entry points (reference: vllm/plugins/__init__.py ``load_general_plugins``,
``load_plugins_by_group``; env ``VLLM_PLUGINS`` selects a subset).

Group ``onecat_vllm.general_plugins``: each entry point names a callable that is run once per process before the engine is
built; it typically calls ``onecat_vllm.models.register_model`` or registers a tool / reasoning parser. ``ONECAT_PLUGINS`` (comma
separated names) restricts which ones load."""
from __future__ import annotations

import os
from typing import Callable

from onecat_vllm.logger import init_logger

log = init_logger(__name__)
GENERAL_GROUP = "onecat_vllm.general_plugins"
_loaded = False


def load_plugins_by_group(group: str) -> dict[str, Callable]:
    from importlib.metadata import entry_points
    allowed = os.environ.get("ONECAT_PLUGINS")
    allowed_set = {x.strip() for x in allowed.split(",")} if allowed is not None else None
    out: dict[str, Callable] = {}
    for ep in entry_points(group=group):
        if allowed_set is not None and ep.name not in allowed_set:
            continue
        try:
            out[ep.name] = ep.load()
        except Exception as e:  # a broken plugin must not take the engine down
            log.error(f"plugin {ep.name} failed to load: {e!r}")
    return out


def load_general_plugins() -> list[str]:
    """Run every general plugin once per process; returns the names that ran."""
    global _loaded
    if _loaded:
        return []
    _loaded = True
    ran = []
    for name, fn in load_plugins_by_group(GENERAL_GROUP).items():
        try:
            fn()
            ran.append(name)
        except Exception as e:
            log.error(f"plugin {name} raised: {e!r}")
    return ran


# ---- out-of-tree layer classes (reference: model_executor/custom_op.py:32,103 ``CustomOp.register`` / ``PluggableLayer``)
_LAYER_OVERRIDES: dict[str, type] = {}


def register_layer(name: str, cls: type) -> None:
    """Replace one of the decoder's building blocks (``Attention``, ``MLAAttention``, ``GatedDeltaNet``, ``MLP``, ``SparseMoeBlock``,
    ``RMSNorm``) by ``cls``, which must take the same constructor arguments and keep the parameter names (checkpoints load by name).
    A plugin calls this before the engine is built."""
    _LAYER_OVERRIDES[name] = cls


def unregister_layer(name: str) -> None:
    _LAYER_OVERRIDES.pop(name, None)


def layer_class(name: str, default: type) -> type:
    return _LAYER_OVERRIDES.get(name, default)
