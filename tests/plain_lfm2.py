"""A plain, slow LFM2: whole sequences, no cache, float32 (or float64) on the CPU.

This file rests on the formulas of the reference's source, not on running it: the
reference is a Rust workspace and no Rust toolchain exists where these tests run, and its
golden file (tests/goldens/lfm2-tiny.json) comes without the weights it was made from.  Each
function cites the lines of the reference (paths relative to the reference's root) that it
restates.  Nothing here imports the package under test: it reads config.json and
model.safetensors by itself, one function per part of the model.
"""
from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Sequence

import torch
from safetensors import safe_open


# --------------------------------------------------------------------------------------
# configuration (crates/vapi-backend-candle/src/models/lfm2.rs:60-138)
def read_config(model_dir: str) -> dict:
    with open(os.path.join(model_dir, "config.json")) as f:
        v = json.load(f)
    c = {}
    c["vocab"] = v["vocab_size"]
    c["hidden"] = v["hidden_size"]
    c["layers"] = v["num_hidden_layers"]
    c["heads"] = v["num_attention_heads"]
    c["kv_heads"] = v["num_key_value_heads"]
    c["head_dim"] = v.get("head_dim", c["hidden"] // c["heads"])                      # :64-68
    ff = v["intermediate_size"]
    if v.get("block_auto_adjust_ff_dim", False):                                       # :72-87
        i = (2 * ff) // 3
        if "block_ffn_dim_multiplier" in v and v["block_ffn_dim_multiplier"] is not None:
            i = int(float(v["block_ffn_dim_multiplier"]) * i)
        mult = v.get("block_multiple_of", 256)
        ff = mult * ((i + mult - 1) // mult)
    c["ff"] = ff
    c["eps"] = v.get("norm_eps", 1e-5)                                                 # :122
    c["max_pos"] = v["max_position_embeddings"]
    rp = v.get("rope_parameters") or {}
    c["theta"] = float(rp.get("rope_theta", v.get("rope_theta", 1_000_000.0)))        # :98-103
    c["L"] = v.get("conv_L_cache", 3)                                                  # :125
    c["conv_bias"] = v.get("conv_bias", False)                                         # :126-129
    c["tied"] = v.get("tie_word_embeddings", True)                                     # :130-133
    c["layer_types"] = v.get("layer_types", ["conv"] * c["layers"])                    # :88-97
    assert len(c["layer_types"]) == c["layers"]
    return c


def read_weights(model_dir: str, dtype=torch.float32) -> Dict[str, torch.Tensor]:
    out = {}
    with safe_open(os.path.join(model_dir, "model.safetensors"), framework="pt", device="cpu") as f:
        for k in f.keys():
            out[k] = f.get_tensor(k).to(dtype)
    return out


# --------------------------------------------------------------------------------------
# parts
def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """x * rsqrt(mean(x^2) + eps) * w over the last dim; the weight multiplies as it is
    (lfm2.rs:322-323, 626-628, 681: candle RmsNorm with norm_eps everywhere)."""
    return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * w


def rope_tables(positions: torch.Tensor, d: int, theta: float, dtype):
    """inv_freq_i = 1/theta^(2i/d) and angle = p * inv_freq_i, both float32 as in
    lfm2.rs:163-183; cos/sin are then used in the working dtype."""
    th = torch.tensor(theta, dtype=torch.float32)
    inv = 1.0 / torch.pow(th, torch.arange(0, d, 2, dtype=torch.float32) / float(d))
    ang = positions.to(torch.float32)[:, None] * inv[None, :]
    return torch.cos(ang).to(dtype), torch.sin(ang).to(dtype)


def rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """Rotate-half pairing (i, i + d/2) on x [T, heads, d] (rope_thd as used at
    lfm2.rs:336-341): out[i] = x[i] cos_i - x[i+d/2] sin_i; out[i+d/2] = x[i+d/2] cos_i + x[i] sin_i."""
    h = x.shape[-1] // 2
    x1, x2 = x[..., :h], x[..., h:]
    c, s = cos[:, None, :], sin[:, None, :]
    return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], -1)


def attention_heads(a: torch.Tensor, w: Dict[str, torch.Tensor], pre: str, c: dict, pos0: int = 0):
    """q, k, v of a whole sequence as [T, heads, d], q and k normed per head and rotated
    (lfm2.rs:343-376)."""
    T = a.shape[0]
    nh, nkv, d = c["heads"], c["kv_heads"], c["head_dim"]
    q = (a @ w[pre + "q_proj.weight"].T).view(T, nh, d)
    k = (a @ w[pre + "k_proj.weight"].T).view(T, nkv, d)
    v = (a @ w[pre + "v_proj.weight"].T).view(T, nkv, d)
    q = rmsnorm(q, w[pre + "q_layernorm.weight"], c["eps"])                             # :364
    k = rmsnorm(k, w[pre + "k_layernorm.weight"], c["eps"])                             # :365
    cos, sin = rope_tables(torch.arange(pos0, pos0 + T), d, c["theta"], a.dtype)
    return rope(q, cos, sin), rope(k, cos, sin), v


def attend(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, window: int = 0) -> torch.Tensor:
    """Causal softmax attention of q [T, nh, d] over k, v [T, nkv, d]; query head h reads kv head
    h // (nh / nkv); with a window only the last ``window`` keys up to the query's own position are
    seen (attention.rs:87-163)."""
    T, nh, d = q.shape
    rep = nh // k.shape[1]
    k = k.repeat_interleave(rep, dim=1)                                                 # head h -> kv head h // rep
    v = v.repeat_interleave(rep, dim=1)
    scale = 1.0 / math.sqrt(d)                                                          # lfm2.rs:377
    s = torch.einsum("thd,shd->hts", q, k) * scale
    mask = torch.ones(T, T, dtype=torch.bool).tril()                                    # key i <= query position
    if window > 0:
        mask &= ~torch.ones(T, T, dtype=torch.bool).tril(-window)                      # and i > position - window
    s = s.masked_fill(~mask[None], float("-inf"))
    p = torch.softmax(s, dim=-1)
    return torch.einsum("hts,shd->thd", p, v).reshape(T, nh * d)


def attention(a: torch.Tensor, w: Dict[str, torch.Tensor], pre: str, c: dict, pos0: int = 0) -> torch.Tensor:
    """Whole-sequence causal GQA with per-head q/k RMSNorm and RoPE
    (lfm2.rs:343-406; masking and softmax as attention.rs:90-163)."""
    q, k, v = attention_heads(a, w, pre, c, pos0)
    return attend(q, k, v) @ w[pre + "out_proj.weight"].T


def shortconv(a: torch.Tensor, w: Dict[str, torch.Tensor], pre: str, c: dict) -> torch.Tensor:
    """in_proj -> B, C, x (checkpoint order); g = B * x; causal depthwise conv, tap L-1 on the
    current token, zeros before the sequence; y = C * conv; out_proj.  conv_bias switches all
    three biases (lfm2.rs:7-13, 438-485, 536-564; taps fused.rs:27-59)."""
    T, H, L = a.shape[0], c["hidden"], c["L"]
    h3 = a @ w[pre + "in_proj.weight"].T
    if c["conv_bias"]:
        h3 = h3 + w[pre + "in_proj.bias"]
    B, C, x = h3[:, :H], h3[:, H:2 * H], h3[:, 2 * H:]
    g = B * x
    taps = w[pre + "conv.weight"][:, 0, :]                                              # (H, L)
    conv = torch.zeros_like(g)
    for t in range(T):
        for k in range(L):
            src = t - (L - 1 - k)
            if src >= 0:
                conv[t] += taps[:, k] * g[src]
    if c["conv_bias"]:
        conv = conv + w[pre + "conv.bias"]
    y = C * conv
    o = y @ w[pre + "out_proj.weight"].T
    if c["conv_bias"]:
        o = o + w[pre + "out_proj.bias"]
    return o


def feed_forward(f: torch.Tensor, w: Dict[str, torch.Tensor], pre: str) -> torch.Tensor:
    """w2( silu(w1 f) * (w3 f) ), silu(g) = g / (1 + exp(-g)) (lfm2.rs:568-595, fused.rs:16-25)."""
    g = f @ w[pre + "w1.weight"].T
    u = f @ w[pre + "w3.weight"].T
    return ((g / (1.0 + torch.exp(-g))) * u) @ w[pre + "w2.weight"].T


def block(x: torch.Tensor, w: Dict[str, torch.Tensor], l: int, c: dict) -> torch.Tensor:
    """x + op(norm(x)); then x + ffn(norm(x)) (lfm2.rs:633-648)."""
    pre = f"model.layers.{l}."
    a = rmsnorm(x, w[pre + "operator_norm.weight"], c["eps"])
    if c["layer_types"][l] == "full_attention":
        x = x + attention(a, w, pre + "self_attn.", c)
    else:
        x = x + shortconv(a, w, pre + "conv.", c)
    f = rmsnorm(x, w[pre + "ffn_norm.weight"], c["eps"])
    return x + feed_forward(f, w, pre + "feed_forward.")


def logits(tokens: Sequence[int], w: Dict[str, torch.Tensor], c: dict) -> torch.Tensor:
    """Logits at every position of one whole sequence, [T, vocab] (lfm2.rs:803-818; the head
    is the embedding when tied or when the file has no lm_head.weight, :676-680)."""
    x = w["model.embed_tokens.weight"][torch.tensor(list(tokens), dtype=torch.long)]
    for l in range(c["layers"]):
        x = block(x, w, l, c)
    x = rmsnorm(x, w["model.embedding_norm.weight"], c["eps"])
    head = w["model.embed_tokens.weight"] if (c["tied"] or "lm_head.weight" not in w) else w["lm_head.weight"]
    return x @ head.T


class PlainLfm2:
    def __init__(self, model_dir: str, dtype=torch.float32):
        self.c = read_config(model_dir)
        self.w = read_weights(model_dir, dtype)
        self.dtype = dtype

    def logits(self, tokens: Sequence[int]) -> torch.Tensor:
        with torch.no_grad():
            return logits(tokens, self.w, self.c).to(torch.float32)

    def greedy(self, prompt: Sequence[int], steps: int) -> List[int]:
        toks = list(prompt)
        out = []
        for _ in range(steps):
            nxt = int(torch.argmax(self.logits(toks)[-1]).item())   # first index wins ties (sampler.rs:285-295)
            out.append(nxt)
            toks.append(nxt)
        return out

    def sample(self, prompt: Sequence[int], steps: int, temperature: float, seed: int) -> List[int]:
        """Temperature sampling by the Gumbel-max rule with the reference's noise: the k-th generated
        token is argmax(logits / T + g(seed, k)) (crates/vapi-backend-candle/src/fused.rs:236-293)."""
        from plain_ops import gumbel_noise
        toks, out = list(prompt), []
        for k in range(steps):
            row = self.logits(toks)[-1]
            g = gumbel_noise(seed & ((1 << 64) - 1), k, row.numel())
            nxt = int(torch.argmax(row.double() * float(torch.tensor(1.0 / temperature, dtype=torch.float32)) + g))
            out.append(nxt)
            toks.append(nxt)
        return out
