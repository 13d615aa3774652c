"""LFM2 (`Lfm2ForCausalLM`, model_type `lfm2`) as a plan of parts.

Layer l is a pre-norm residual block whose mixer is the gated short convolution or GQA
attention according to ``layer_types[l]``, followed by a SwiGLU feed-forward; the model ends
with ``embedding_norm`` and a (usually tied) output head.  Tensor names are the checkpoint's
own (crates/vapi-backend-candle/src/models/lfm2.rs:315-323, 438-464, 579-587, 616-629,
675-684).  Everything here is data handed to parameterised parts; the parts do not know
they are in LFM2.  The typed configuration follows the reference's ``Lfm2Config::from_json``
(crates/vapi-backend-candle/src/models/lfm2.rs:60-138).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Tuple

from ..config.model import Architecture, ConfigError, register_architecture, require_int as _req_int
from ..parts import (GQAttention, OutputHead, PreNormBlock, RMSNorm, RotaryEncoding, ShortConv, SwiGLU,
                     TokenEmbedding)
from .plan import LayerCall, ModelPlan


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


def lfm2_plan(cfg: Lfm2Config) -> ModelPlan:
    H = cfg.hidden_size
    emb = TokenEmbedding(cfg.vocab_size, H, "model.embed_tokens.weight")
    layers, prefixes = [], []
    for l in range(cfg.num_hidden_layers):
        if cfg.is_attention(l):
            mixer = GQAttention(H, cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim,
                                qk_norm_eps=cfg.norm_eps, pos="rope", rot_dim=cfg.head_dim)
            mixer_sub = "self_attn."
        else:
            mixer = ShortConv(H, cfg.conv_L_cache, cfg.conv_bias)
            mixer_sub = "conv."
        layers.append(PreNormBlock(
            RMSNorm(H, cfg.norm_eps), mixer, RMSNorm(H, cfg.norm_eps),
            SwiGLU(H, cfg.intermediate_size, {"gate": "w1", "up": "w3", "down": "w2"}),
            {"mixer_norm": "operator_norm.", "mixer": mixer_sub, "ffn_norm": "ffn_norm.",
             "ffn": "feed_forward."}))
        prefixes.append(f"model.layers.{l}.")
    return ModelPlan(
        architecture=cfg.architecture,
        vocab_size=cfg.vocab_size,
        hidden_size=H,
        max_positions=cfg.max_position_embeddings,
        embedding=emb,
        layers=layers,
        layer_prefixes=prefixes,
        order=[LayerCall(l) for l in range(cfg.num_hidden_layers)],
        final_norm=RMSNorm(H, cfg.norm_eps),
        final_norm_prefix="model.embedding_norm.",
        head=OutputHead(cfg.vocab_size, H, cfg.tie_word_embeddings, emb, "lm_head.weight"),
        position_encodings=[RotaryEncoding(cfg.head_dim, cfg.rope_theta, cfg.max_position_embeddings, "rope")],
        eos_token_ids=cfg.eos_token_ids,
        config=cfg,
    )


register_architecture(Architecture(
    name="Lfm2ForCausalLM", model_types=("lfm2",), parse=Lfm2Config.from_json, plan=lfm2_plan))
