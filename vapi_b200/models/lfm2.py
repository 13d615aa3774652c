"""LFM2 (`Lfm2ForCausalLM`, model_type `lfm2`) as a plan of parts.

Layer l is a pre-norm residual block whose mixer is the gated short convolution or GQA
attention according to ``layer_types[l]``, followed by a SwiGLU feed-forward; the model ends
with ``embedding_norm`` and a (usually tied) output head.  Tensor names are the checkpoint's
own (crates/vapi-backend-candle/src/models/lfm2.rs:315-323, 438-464, 579-587, 616-629,
675-684).  Everything here is data handed to parameterised parts; the parts do not know
they are in LFM2.
"""
from __future__ import annotations

from ..config.model import Architecture, Lfm2Config, register_architecture
from ..parts import (GQAttention, OutputHead, PreNormBlock, RMSNorm, RotaryEncoding, ShortConv, SwiGLU,
                     TokenEmbedding)
from .plan import LayerCall, ModelPlan


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
