"""Plain float32 restatements of every kernel, one function per kernel, written as loops
over sequences and tokens from the reference's formulas.  They have the signatures of
``vapi_b200.ops`` so that (a) each CUDA kernel can be compared with its plain version alone
and (b) the host side of the engine (cache manager, packer, step function, scheduler) can be
exercised on a CPU by standing these in for the kernels.  They are test code: nothing in the
package imports them, and the package has no CPU path of its own.
"""
from __future__ import annotations

import math

import torch


def _f(t):
    return t.to(torch.float32)


def embed(table, tokens, status=None, next_weight=None):
    out = _f(table[tokens.long()])
    if next_weight is None:
        return out
    return out, (out ** 2).sum(1)[None, :], (out * next_weight).to(torch.bfloat16)


def resolve_tokens(tokens, src, prev, status=None):
    """tokens[i] = prev[src[i]] where src[i] >= 0 (tokens the step before sampled on the device)."""
    m = src >= 0
    tokens[m] = prev[src[m].long()]


def add_residual_ss(x, delta, next_weight):
    x += _f(delta)
    return (x ** 2).sum(1)[None, :], (x * next_weight).to(torch.bfloat16)


def skinny_applies(rows, weight):
    return False


def tc_applies(rows, weight):
    return False


def few_rows_applies(rows, weight):
    return False


def add_rmsnorm(x, delta, weight, eps, out_dtype, rows=None):
    """crates/vapi-backend-candle/src/models/lfm2.rs:633-648: residual add, then RMSNorm."""
    if rows is None:
        if delta is not None:
            x += _f(delta)
        src = x
    else:
        src = x[rows.long()]
        if delta is not None:
            src = src + _f(delta[rows.long()])
    y = src * torch.rsqrt(src.pow(2).mean(-1, keepdim=True) + eps) * weight
    return y.to(out_dtype)


def add_residual(x, delta):
    x += _f(delta)


def swiglu(g):
    """crates/vapi-backend-candle/src/fused.rs:157-165."""
    f = g.shape[1] // 2
    a, b = _f(g[:, :f]), _f(g[:, f:])
    return ((a / (1.0 + torch.exp(-a))) * b).to(g.dtype)


def linear(x, weight, bias=None, out_dtype=None):
    y = _f(x) @ _f(weight).t()
    if bias is not None:
        y = y + _f(bias)
    return y.to(out_dtype or x.dtype)


def strict_fp32():
    pass


def rope_cos_sin(positions, inv_freq):
    """crates/vapi-backend-candle/src/models/lfm2.rs:169-178: angle = p as f32 * inv_freq."""
    ang = positions.to(torch.float32)[:, None] * inv_freq[None, :]
    return torch.cos(ang), torch.sin(ang)


def qk_norm_rope_write(qkv, nh, nkv, d, q_weight, k_weight, eps, cos, sin, rot, cache_layer,
                       slot_mapping, status=None):
    """crates/vapi-backend-candle/src/models/lfm2.rs:364-375."""
    n = qkv.shape[0]
    heads = qkv.view(n, nh + 2 * nkv, d)
    page = cache_layer.shape[3] if cache_layer is not None else 0
    for t in range(n):
        for h in range(nh + 2 * nkv):
            v = _f(heads[t, h])
            is_q, is_k = h < nh, nh <= h < nh + nkv
            w = q_weight if is_q else (k_weight if is_k else None)
            if w is not None:
                v = v * torch.rsqrt(v.pow(2).mean() + eps) * w
            if (is_q or is_k) and cos is not None:
                half = rot // 2
                a, b = v[:half].clone(), v[half:rot].clone()
                v = v.clone()
                v[:half] = a * cos[t] - b * sin[t]
                v[half:rot] = b * cos[t] + a * sin[t]
            if is_q:
                heads[t, h] = v.to(qkv.dtype)
            elif cache_layer is not None:
                slot = int(slot_mapping[t])
                g = h - nh if is_k else h - nh - nkv
                cache_layer[slot // page, 0 if is_k else 1, g, slot % page] = v.to(cache_layer.dtype)


def attention_splits(num_seqs, max_q, max_k, nh, nkv):
    return 1


def paged_attention(q, q_row_stride, cache_layer, block_table, cu_q, seqlens_k, n, num_seqs, max_q,
                    max_k, nh, nkv, d, scale, window=0, splits=None, status=None):
    """crates/vapi-backend-candle/src/attention.rs:90-163: gather each sequence's keys
    through its block table; query j of len_q over len_k keys sits at len_k - len_q + j and
    sees keys i <= its position (and i > position - window)."""
    page = cache_layer.shape[3]
    rep = nh // nkv
    qh = q.reshape(n, -1)[:, :nh * d].reshape(n, nh, d)
    out = torch.zeros((n, nh * d), dtype=torch.float32)
    for s in range(num_seqs):
        q0, q1, klen = int(cu_q[s]), int(cu_q[s + 1]), int(seqlens_k[s])
        qlen = q1 - q0
        keys = torch.zeros((klen, nkv, d))
        vals = torch.zeros((klen, nkv, d))
        lo_needed = 0 if window <= 0 else max(0, klen - qlen - window + 1)
        for i in range(lo_needed, klen):
            pg = int(block_table[s, i // page])
            keys[i] = _f(cache_layer[pg, 0, :, i % page])
            vals[i] = _f(cache_layer[pg, 1, :, i % page])
        for j in range(qlen):
            p = klen - qlen + j
            lo = 0 if window <= 0 else max(0, p - window + 1)
            for h in range(nh):
                g = h // rep
                sc = (keys[lo:p + 1, g] @ _f(qh[q0 + j, h])) * scale
                pr = torch.softmax(sc, 0)
                out[q0 + j, h * d:(h + 1) * d] = pr @ vals[lo:p + 1, g]
    return out.to(q.dtype)


def shortconv(h3, in_bias, taps, conv_bias, state_layer, state_slots, tok_seq, cu_q, positions, status=None):
    """crates/vapi-backend-candle/src/models/lfm2.rs:509-565 with the state kept as the last
    L-1 rows of g per request instead of paged rows: per sequence, rebuild the history from
    the state, run the causal conv over the portion, store the new last L-1 rows."""
    n, H, L = h3.shape[0], h3.shape[1] // 3, taps.shape[0]
    dt = h3.dtype
    out = torch.zeros((n, H), dtype=torch.float32)
    S = cu_q.numel() - 1
    for s in range(S):
        r0, r1 = int(cu_q[s]), int(cu_q[s + 1])
        if r1 == r0:
            continue
        p0 = int(positions[r0])
        slot = int(state_slots[s])
        hist = []                                   # g at positions p0-(L-1) .. p0-1
        for j in range(L - 1):
            pos = p0 - (L - 1) + j
            hist.append(_f(state_layer[slot, j]) if pos >= 0 else torch.zeros(H))
        for r in range(r0, r1):
            B, C, x = _f(h3[r, :H]), _f(h3[r, H:2 * H]), _f(h3[r, 2 * H:])
            if in_bias is not None:
                B, C, x = B + in_bias[:H], C + in_bias[H:2 * H], x + in_bias[2 * H:]
            g = (B * x).to(dt).to(torch.float32)    # the stored row has the storage precision
            hist.append(g)
            acc = torch.zeros(H)
            for k in range(L):
                acc = acc + taps[k] * hist[len(hist) - L + k]
            if conv_bias is not None:
                acc = acc + conv_bias
            out[r] = C * acc
            hist = hist[-(L - 1):] if L > 1 else []
        for j in range(L - 1):
            state_layer[slot, j] = hist[j].to(dt)
    return out.to(dt)


def _mix64(x):
    m = (1 << 64) - 1
    x ^= x >> 33
    x = (x * 0xff51afd7ed558ccd) & m
    x ^= x >> 33
    x = (x * 0xc4ceb9fe1a85ec53) & m
    x ^= x >> 33
    return x


def gumbel_noise(seed, draw, vocab):
    """crates/vapi-backend-candle/src/fused.rs:252-293."""
    m = (1 << 64) - 1
    key = _mix64((seed ^ _mix64((draw + 0x9E3779B97F4A7C15) & m)) & m)
    out = torch.empty(vocab, dtype=torch.float64)
    for v in range(vocab):
        h = _mix64((key + v * 0xBF58476D1CE4E5B9) & m)
        u = ((h >> 40) + 0.5) / 16777216.0
        out[v] = -math.log(-math.log(u))
    return out


def sample_rows(logits, mode=None, inv_t=None, seeds=None, draws=None, out=None):
    rows, vocab = logits.shape
    res = torch.zeros(rows, dtype=torch.int32) if out is None else out
    for r in range(rows):
        md = 1 if mode is None else int(mode[r])
        if md == 0:
            continue
        if md == 1:
            res[r] = int(torch.argmax(logits[r]))
        else:
            g = gumbel_noise(int(seeds[r]) & ((1 << 64) - 1), int(draws[r]), vocab)
            res[r] = int(torch.argmax(logits[r].double() * float(inv_t[r]) + g))
    return res


def sample_truncated(logits, inv_t, top_k, top_p, min_p, seeds, draws, out=None, check=False):
    """Gumbel-max over the host sampler's survivors; rows with a negative top_k are left alone."""
    rows, vocab = logits.shape
    res = torch.zeros(rows, dtype=torch.int32) if out is None else out
    for r in range(rows):
        k = int(top_k[r]) if top_k is not None else 0
        if k < 0:
            continue
        ids, _, scaled = truncated_survivors(logits[r].float().numpy(), float(inv_t[r]), k or None,
                                             float(top_p[r]) if top_p is not None else 1.0,
                                             float(min_p[r]) if min_p is not None else 0.0)
        g = gumbel_noise(int(seeds[r]) & ((1 << 64) - 1), int(draws[r]), vocab)
        best = max(ids.tolist(), key=lambda t: (float(scaled[t]) + float(g[t]), -t))
        res[r] = best
    return res


def truncated_survivors(row, inv_t, top_k=None, top_p=1.0, min_p=0.0):
    """Token ids that survive the host sampler's cuts, in its order (probability descending, then
    id), and their probabilities over the 30-nat window
    (crates/vapi-engine/src/sampler.rs:302-376): window, top-k, min-p, top-p."""
    import numpy as np
    scaled = row.astype(np.float32) * np.float32(inv_t)
    mx = scaled.max()
    keep = np.nonzero(scaled >= mx - np.float32(30.0))[0]
    e = np.exp((scaled[keep] - mx).astype(np.float64))
    prob = e / e.sum()
    order = np.lexsort((keep, -prob))
    ids, prob = keep[order], prob[order]
    if top_k:
        ids, prob = ids[:top_k], prob[:top_k]
    if min_p > 0.0:
        n = max(int(np.sum(np.cumprod(prob >= min_p * prob[0]))), 1)
        ids, prob = ids[:n], prob[:n]
    if top_p < 1.0:
        cum = np.cumsum(prob)
        n = max(min(int(np.searchsorted(cum, top_p, side="left")) + 1, len(prob)), 1)
        ids, prob = ids[:n], prob[:n]
    return ids, prob, scaled


def apply_penalties(logits, rows, toks, counts, rep, freq, pres):
    """crates/vapi-engine/src/sampler.rs:262-283."""
    for i in range(rows.numel()):
        r, t = int(rows[i]), int(toks[i])
        v = float(logits[r, t])
        p = float(rep[r])
        if p != 1.0:
            v = v / p if v > 0 else v * p
        v -= float(freq[r]) * float(counts[i])
        if float(counts[i]) > 0:
            v -= float(pres[r])
        logits[r, t] = v


ALL = ["embed", "resolve_tokens", "sample_truncated", "add_rmsnorm", "add_residual", "add_residual_ss", "skinny_applies", "tc_applies", "few_rows_applies", "swiglu", "linear", "strict_fp32", "rope_cos_sin",
       "qk_norm_rope_write", "attention_splits", "paged_attention", "shortconv", "sample_rows",
       "apply_penalties"]
