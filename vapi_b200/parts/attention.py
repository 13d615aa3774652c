"""Grouped-query attention over the paged cache."""
from __future__ import annotations

import math
from typing import Any, Dict, List, Optional

import torch

from .. import ops
from .base import CacheView, Mixer, PagedSpec, StreamState, TensorSpec, register_mixer


class GQAttention(Mixer):
    """q/k/v projection, optional per-head RMSNorm of q and k, optional rotary encoding,
    cache write, causal attention over the block table (optionally windowed), out
    projection (crates/vapi-backend-candle/src/models/lfm2.rs:343-406; attention semantics
    crates/vapi-backend-candle/src/attention.rs:90-163).

    The three projections are fused into one matrix at bind time.  ``names`` maps the roles
    ``q k v o q_norm k_norm`` to checkpoint sub-names, so another architecture's naming is a
    parameter, not a subclass.  ``pos`` names the position encoding whose ``(cos, sin)`` to
    apply (None: no rotation).
    """

    def __init__(self, hidden: int, n_heads: int, n_kv_heads: int, head_dim: int, *,
                 qk_norm_eps: Optional[float] = None, pos: Optional[str] = "rope",
                 rot_dim: Optional[int] = None, window: int = 0, bias: bool = False,
                 scale: Optional[float] = None, names: Optional[Dict[str, str]] = None):
        if n_heads <= 0 or n_kv_heads <= 0 or n_heads % n_kv_heads:
            raise ValueError(f"{n_heads} heads are not a multiple of {n_kv_heads} kv heads")
        if head_dim % 16 or not 16 <= head_dim <= 256:
            raise ValueError(f"head_dim {head_dim} must be a multiple of 16 in 16..256")
        self.hidden, self.nh, self.nkv, self.d = int(hidden), int(n_heads), int(n_kv_heads), int(head_dim)
        self.qk_norm_eps = qk_norm_eps
        self.pos = pos
        self.rot_dim = int(rot_dim) if rot_dim is not None else self.d
        self.window = int(window)
        self.bias = bool(bias)
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(self.d)
        self.names = {"q": "q_proj", "k": "k_proj", "v": "v_proj", "o": "out_proj",
                      "q_norm": "q_layernorm", "k_norm": "k_layernorm"}
        if names:
            self.names.update(names)
        self.w_qkv = self.b_qkv = self.w_o = self.b_o = self.q_w = self.k_w = None

    def cache_spec(self):
        return PagedSpec.kv(self.nkv, self.d, self.window)

    def tensor_specs(self, prefix: str) -> List[TensorSpec]:
        n, (h, nh, nkv, d) = self.names, (self.hidden, self.nh, self.nkv, self.d)
        specs = [TensorSpec(f"{prefix}{n['q']}.weight", (nh * d, h)),
                 TensorSpec(f"{prefix}{n['k']}.weight", (nkv * d, h)),
                 TensorSpec(f"{prefix}{n['v']}.weight", (nkv * d, h)),
                 TensorSpec(f"{prefix}{n['o']}.weight", (h, nh * d))]
        if self.bias:
            specs += [TensorSpec(f"{prefix}{n['q']}.bias", (nh * d,), role="vector"),
                      TensorSpec(f"{prefix}{n['k']}.bias", (nkv * d,), role="vector"),
                      TensorSpec(f"{prefix}{n['v']}.bias", (nkv * d,), role="vector"),
                      TensorSpec(f"{prefix}{n['o']}.bias", (h,), role="vector")]
        if self.qk_norm_eps is not None:
            specs += [TensorSpec(f"{prefix}{n['q_norm']}.weight", (d,), role="vector", init="ones"),
                      TensorSpec(f"{prefix}{n['k_norm']}.weight", (d,), role="vector", init="ones")]
        return specs

    def bind(self, tensors, prefix, dtype):
        n = self.names
        parts = [tensors[f"{prefix}{n[r]}.weight"] for r in ("q", "k", "v")]
        wd = parts[0].dtype if all(p.dtype == parts[0].dtype for p in parts) else torch.float32
        self.w_qkv = torch.cat([p.to(wd) for p in parts], 0).contiguous()
        self.w_o = tensors[f"{prefix}{n['o']}.weight"].contiguous()
        if self.bias:
            self.b_qkv = torch.cat([tensors[f"{prefix}{n[r]}.bias"] for r in ("q", "k", "v")], 0).contiguous()
            self.b_o = tensors[f"{prefix}{n['o']}.bias"].contiguous()
        if self.qk_norm_eps is not None:
            self.q_w = tensors[f"{prefix}{n['q_norm']}.weight"].contiguous()
            self.k_w = tensors[f"{prefix}{n['k_norm']}.weight"].contiguous()

    def decode_splits(self, batch: int, max_context: int, page_size: int, dtype: torch.dtype) -> int:
        keys = min(max_context, self.window) if self.window > 0 else max_context
        dec = ops.decode_attention_applies(dtype, self.d, page_size, self.nh // self.nkv)
        return ops.attention_splits(batch, 1, keys, self.nh, self.nkv, dec)

    def forward(self, a: torch.Tensor, ctx: Any, cache: CacheView) -> torch.Tensor:
        qkv = ops.linear(a, self.w_qkv, self.b_qkv)
        return ops.linear(self._attend(qkv, ctx, cache), self.w_o, self.b_o)

    def forward_stream(self, a, ctx, cache, x, next_weight):
        n = x.shape[0]
        if not (ops.few_rows_applies(n, self.w_qkv) and ops.few_rows_applies(n, self.w_o)):
            return NotImplemented
        qkv = ops.few_rows_linear(self.w_qkv, xw=a.xw, ss_in=a.ss, eps=a.eps, epilogue="bf16", bias=self.b_qkv)
        y = self._attend(qkv, ctx, cache)
        ss, xw = ops.few_rows_linear(self.w_o, act=y, epilogue="resid", resid=x, bias=self.b_o, next_weight=next_weight)
        return StreamState(xw, ss)

    def _attend(self, qkv: torch.Tensor, ctx: Any, cache: CacheView) -> torch.Tensor:
        nh, nkv, d = self.nh, self.nkv, self.d
        cos = sin = None
        if self.pos is not None:
            cos, sin = ctx.pos[self.pos]
        grp = cache.group
        n_rep = nh // nkv
        kv = cache.stacked() if cache.tensor is not None else None      # [pages, 2, n_kv, page_size, head_dim]
        splits = grp.splits if getattr(grp, "splits", None) is not None else ctx.attention_splits
        max_k = getattr(grp, "max_k", None) or ctx.max_k
        if self.window > 0:
            max_k = min(max_k, self.window + ctx.max_q - 1)      # a query reads at most `window` keys
        if (ops.FUSED_DECODE_ROPE and qkv.is_cuda and kv is not None
                and ops.decode_attention_fused_applies(qkv.dtype, d, kv.shape[3], ctx.max_q * n_rep,
                                                       self.rot_dim if cos is not None else None)
                and (cos is None or (cos.is_contiguous() and sin.is_contiguous()))):
            # a decode step: norm, rotation and the cache write ride in the attention kernel
            return ops.decode_attention_fused(qkv, nh, nkv, d, self.q_w, self.k_w,
                                              self.qk_norm_eps if self.qk_norm_eps is not None else 0.0, cos, sin,
                                              kv, cache.write, grp.block_table, ctx.cu_q, ctx.seqlens_k,
                                              ctx.n, ctx.num_seqs, ctx.max_q, max_k, self.scale, self.window,
                                              splits, ctx.status)
        ops.qk_norm_rope_write(qkv, nh, nkv, d, self.q_w, self.k_w,
                               self.qk_norm_eps if self.qk_norm_eps is not None else 0.0,
                               cos, sin, self.rot_dim,
                               kv if cache.write else None, grp.slot_mapping, ctx.status)
        y = ops.paged_attention(qkv, qkv.stride(0), kv, grp.block_table, ctx.cu_q,
                                ctx.seqlens_k, ctx.n, ctx.num_seqs, ctx.max_q, max_k, nh, nkv, d,
                                self.scale, self.window, splits, ctx.status)
        return y


register_mixer("gqa_attention", GQAttention)
