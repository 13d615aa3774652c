"""The architecture registry and what every architecture's configuration shares.

A configuration is read from the architecture's own ``config.json`` keys; no
size and no constant that ``config.json`` gives is written down in code.  The
registry maps an architecture name (``architectures[0]`` or ``model_type``) to
two callables: one that parses the json into a typed configuration and one that
turns a configuration into a :class:`~vapi_b200.models.plan.ModelPlan`.  The
typed configuration of an architecture lives with its plan (``models/<name>.py``);
this module holds none.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Any, Callable, Dict, List, Tuple


class ConfigError(ValueError):
    """A config.json that cannot be turned into a model."""


def require_int(v: Dict[str, Any], key: str) -> int:
    """A non-negative integer key that config.json must have."""
    x = v.get(key)
    if isinstance(x, bool) or not isinstance(x, int) or x < 0:
        raise ConfigError(f"config.json: missing integer `{key}`")
    return int(x)


# --------------------------------------------------------------------------
# registry


@dataclass(frozen=True)
class Architecture:
    """One registered architecture.

    ``parse`` turns the config.json dictionary into a typed configuration;
    ``plan`` turns that configuration into a ``ModelPlan`` (the parts of every
    layer, their tensor names and the order in which layers run).
    """

    name: str
    model_types: Tuple[str, ...]
    parse: Callable[[Dict[str, Any]], Any]
    plan: Callable[[Any], Any]


_REGISTRY: Dict[str, Architecture] = {}


def register_architecture(arch: Architecture, *, replace: bool = False) -> None:
    """Add an architecture.  Its ``name`` is matched against
    ``architectures[0]`` and each of ``model_types`` against ``model_type``."""
    keys = (arch.name,) + tuple(arch.model_types)
    for k in keys:
        if k in _REGISTRY and not replace and _REGISTRY[k] is not arch:
            raise ValueError(f"architecture key `{k}` is already registered")
    for k in keys:
        _REGISTRY[k] = arch


def unregister_architecture(name: str) -> None:
    arch = _REGISTRY.get(name)
    if arch is None:
        return
    for k in [k for k, a in _REGISTRY.items() if a is arch]:
        del _REGISTRY[k]


def registered_architectures() -> List[str]:
    _ensure_builtin()
    return sorted({a.name for a in _REGISTRY.values()})


def resolve_architecture(v: Dict[str, Any]) -> Architecture:
    """Pick the architecture for a config.json dictionary.

    ``architectures[0]`` wins; ``model_type`` is the fallback, which is the key
    the reference dispatches on (crates/vapi-backend-candle/src/backend.rs:237-248).
    """
    _ensure_builtin()
    archs = v.get("architectures")
    tried = []
    if isinstance(archs, list) and archs and isinstance(archs[0], str):
        tried.append(archs[0])
        if archs[0] in _REGISTRY:
            return _REGISTRY[archs[0]]
    mt = v.get("model_type")
    if isinstance(mt, str):
        tried.append(mt)
        if mt in _REGISTRY:
            return _REGISTRY[mt]
    raise ConfigError(
        f"architecture {tried or '(none named)'} is not supported; registered: "
        f"{registered_architectures()}")


def load_config_json(model_dir: str) -> Dict[str, Any]:
    path = os.path.join(model_dir, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"{model_dir}: no config.json")
    with open(path, "r", encoding="utf-8") as f:
        v = json.load(f)
    if not isinstance(v, dict):
        raise ConfigError(f"{path}: not a json object")
    return v


def eos_token_ids(model_dir: str, cfg_json: Dict[str, Any]) -> Tuple[int, ...]:
    """EOS ids: ``generation_config.json`` wins over ``config.json``; sorted,
    without duplicates (crates/vapi-backend-candle/src/backend.rs:324-330)."""

    def ids_of(v: Any) -> List[int]:
        e = v.get("eos_token_id") if isinstance(v, dict) else None
        if isinstance(e, int) and not isinstance(e, bool):
            return [int(e)]
        if isinstance(e, list):
            return [int(x) for x in e if isinstance(x, int) and not isinstance(x, bool)]
        return []

    gen = os.path.join(model_dir, "generation_config.json")
    out: List[int] = []
    if os.path.isfile(gen):
        try:
            with open(gen, "r", encoding="utf-8") as f:
                out = ids_of(json.load(f))
        except (OSError, ValueError):
            out = []
    if not out:
        out = ids_of(cfg_json)
    return tuple(sorted(set(out)))


_BUILTIN_DONE = False


def _ensure_builtin() -> None:
    """Register the architectures that ship with the package (lazily, so that
    importing the configuration module does not import the model code)."""
    global _BUILTIN_DONE
    if _BUILTIN_DONE:
        return
    _BUILTIN_DONE = True
    import importlib
    for module in BUILTIN_ARCHITECTURE_MODULES:
        importlib.import_module(module)       # registers itself


#: modules that ship with the package and register an architecture when imported
BUILTIN_ARCHITECTURE_MODULES = ["vapi_b200.models.lfm2"]
