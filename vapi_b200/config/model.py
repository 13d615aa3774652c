"""Typed model configuration and the architecture registry.

A configuration is read from the architecture's own ``config.json`` keys; no
size and no constant that ``config.json`` gives is written down in code.  The
registry maps an architecture name (``architectures[0]`` or ``model_type``) to
two callables: one that parses the json into a typed configuration and one that
turns a configuration into a :class:`~vapi_b200.models.plan.ModelPlan`.

The LFM2 rules follow the reference's ``Lfm2Config::from_json``
(crates/vapi-backend-candle/src/models/lfm2.rs:60-138).
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Any, Callable, Dict, List, Tuple


class ConfigError(ValueError):
    """A config.json that cannot be turned into a model."""


def _req_int(v: Dict[str, Any], key: str) -> int:
    x = v.get(key)
    if isinstance(x, bool) or not isinstance(x, int) or x < 0:
        raise ConfigError(f"config.json: missing integer `{key}`")
    return int(x)


@dataclass(frozen=True)
class Lfm2Config:
    """LFM2: gated short-convolution blocks mixed with GQA attention blocks.

    Field meanings and defaults are those of the reference
    (crates/vapi-backend-candle/src/models/lfm2.rs:33-51, 60-138).
    ``intermediate_size`` is the *effective* feed-forward width after the
    ``block_auto_adjust_ff_dim`` rule has been applied.
    """

    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    norm_eps: float
    max_position_embeddings: int
    rope_theta: float
    conv_L_cache: int
    conv_bias: bool
    tie_word_embeddings: bool
    layer_types: Tuple[str, ...]
    eos_token_ids: Tuple[int, ...] = ()
    architecture: str = "Lfm2ForCausalLM"

    LAYER_KINDS = ("conv", "full_attention")

    @staticmethod
    def effective_ff_dim(v: Dict[str, Any]) -> int:
        """The feed-forward width rule (lfm2.rs:70-87): start from
        ``intermediate_size``; if ``block_auto_adjust_ff_dim``, take two thirds
        (integer division), scale by ``block_ffn_dim_multiplier`` when present
        (truncating), and round up to ``block_multiple_of`` (default 256)."""
        ff = _req_int(v, "intermediate_size")
        if bool(v.get("block_auto_adjust_ff_dim", False)):
            i = (2 * ff) // 3
            m = v.get("block_ffn_dim_multiplier")
            if isinstance(m, (int, float)) and not isinstance(m, bool):
                i = int(float(m) * i)
            mult = v.get("block_multiple_of", 256)
            if isinstance(mult, bool) or not isinstance(mult, int) or mult <= 0:
                raise ConfigError("config.json: `block_multiple_of` must be a positive integer")
            ff = mult * ((i + mult - 1) // mult)
        return ff

    @classmethod
    def from_json(cls, v: Dict[str, Any]) -> "Lfm2Config":
        hidden = _req_int(v, "hidden_size")
        heads = _req_int(v, "num_attention_heads")
        layers = _req_int(v, "num_hidden_layers")
        if heads == 0:
            raise ConfigError("config.json: `num_attention_heads` must be positive")
        head_dim = v.get("head_dim")
        if isinstance(head_dim, bool) or not isinstance(head_dim, int):
            head_dim = hidden // heads
        lt = v.get("layer_types")
        if isinstance(lt, list):
            layer_types = tuple(str(x) for x in lt if isinstance(x, str))
        else:
            layer_types = tuple("conv" for _ in range(layers))
        if len(layer_types) != layers:
            raise ConfigError("layer_types does not cover every layer")
        for t in layer_types:
            if t not in cls.LAYER_KINDS:
                raise ConfigError(
                    f"config.json: layer type `{t}` is not one of {list(cls.LAYER_KINDS)}")
        rp = v.get("rope_parameters")
        theta = None
        if isinstance(rp, dict):
            theta = rp.get("rope_theta")
        if theta is None:
            theta = v.get("rope_theta")
        if isinstance(theta, bool) or not isinstance(theta, (int, float)):
            theta = 1_000_000.0
        eos = v.get("eos_token_id")
        if isinstance(eos, int) and not isinstance(eos, bool):
            eos_ids: Tuple[int, ...] = (int(eos),)
        elif isinstance(eos, list):
            eos_ids = tuple(int(x) for x in eos if isinstance(x, int) and not isinstance(x, bool))
        else:
            eos_ids = ()
        kv = _req_int(v, "num_key_value_heads")
        if kv == 0 or heads % kv != 0:
            raise ConfigError(
                f"config.json: num_attention_heads ({heads}) must be a multiple of "
                f"num_key_value_heads ({kv})")
        arch = "Lfm2ForCausalLM"
        archs = v.get("architectures")
        if isinstance(archs, list) and archs and isinstance(archs[0], str):
            arch = archs[0]
        return cls(
            vocab_size=_req_int(v, "vocab_size"),
            hidden_size=hidden,
            intermediate_size=cls.effective_ff_dim(v),
            num_hidden_layers=layers,
            num_attention_heads=heads,
            num_key_value_heads=kv,
            head_dim=int(head_dim),
            norm_eps=float(v.get("norm_eps", 1e-5)),
            max_position_embeddings=_req_int(v, "max_position_embeddings"),
            rope_theta=float(theta),
            conv_L_cache=int(v.get("conv_L_cache", 3)),
            conv_bias=bool(v.get("conv_bias", False)),
            tie_word_embeddings=bool(v.get("tie_word_embeddings", True)),
            layer_types=layer_types,
            eos_token_ids=tuple(sorted(set(eos_ids))),
            architecture=arch,
        )

    def to_json(self) -> Dict[str, Any]:
        """A config.json that parses back to this configuration.  The effective
        feed-forward width is written as-is with the auto-adjust rule off."""
        return {
            "architectures": [self.architecture],
            "model_type": "lfm2",
            "vocab_size": self.vocab_size,
            "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size,
            "block_auto_adjust_ff_dim": False,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "norm_eps": self.norm_eps,
            "max_position_embeddings": self.max_position_embeddings,
            "rope_theta": self.rope_theta,
            "conv_L_cache": self.conv_L_cache,
            "conv_bias": self.conv_bias,
            "tie_word_embeddings": self.tie_word_embeddings,
            "layer_types": list(self.layer_types),
            "eos_token_id": list(self.eos_token_ids),
        }

    def is_attention(self, layer: int) -> bool:
        return self.layer_types[layer] == "full_attention"


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
    from ..models import lfm2 as _lfm2  # noqa: F401  (registers itself)
