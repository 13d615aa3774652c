"""Each CUDA kernel alone against its plain float32 restatement, at sizes other than the
engine tests' (sizes that are no power of two, head sizes from 16 to 256, odd group counts)."""
import itertools
import math

import pytest
import torch

import plain_ops

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]


def tol(dtype):
    return dict(atol=2e-5, rtol=2e-5) if dtype == torch.float32 else dict(atol=2e-2, rtol=2e-2)


def dev(t):
    return t.cuda() if t is not None else None


@pytest.fixture(scope="module")
def ops():
    from vapi_b200 import ops as o
    return o


def test_cpu_tensors_are_refused(ops):
    with pytest.raises(ops.KernelError):
        ops.swiglu(torch.zeros(2, 8))


@pytest.mark.parametrize("wdt", DTYPES)
def test_embed(ops, wdt):
    torch.manual_seed(0)
    table = torch.randn(301, 72).to(wdt)
    toks = torch.randint(0, 301, (19,), dtype=torch.int32)
    got = ops.embed(dev(table), dev(toks))
    assert got.dtype == torch.float32
    torch.testing.assert_close(got.cpu(), plain_ops.embed(table, toks), atol=0, rtol=0)


def test_resolve_tokens(ops):
    g = torch.Generator().manual_seed(5)
    toks = torch.randint(0, 1000, (300,), generator=g, dtype=torch.int32)
    src = torch.full((300,), -1, dtype=torch.int32)
    src[torch.randperm(300, generator=g)[:77]] = torch.randint(0, 64, (77,), generator=g, dtype=torch.int32)
    prev = torch.randint(0, 1000, (64,), generator=g, dtype=torch.int32)
    want = toks.clone()
    plain_ops.resolve_tokens(want, src, prev)
    got = dev(toks.clone())
    ops.resolve_tokens(got, dev(src), dev(prev))
    assert torch.equal(got.cpu(), want) and not torch.equal(want, toks)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hidden", [72, 2048, 1000, 70, 5000])
def test_add_rmsnorm(ops, dtype, hidden):
    torch.manual_seed(1)
    n = 13
    x = torch.randn(n, hidden) * 3
    delta = torch.randn(n, hidden).to(dtype)
    w = 1 + 0.1 * torch.randn(hidden)
    x_ref = x.clone()
    want = plain_ops.add_rmsnorm(x_ref, delta, w, 1e-6, dtype)
    xg = dev(x.clone())
    got = ops.add_rmsnorm(xg, dev(delta), dev(w), 1e-6, dtype)
    torch.testing.assert_close(xg.cpu(), x_ref, atol=1e-6, rtol=1e-6)       # the stream got the add
    torch.testing.assert_close(got.cpu().float(), want.float(), **tol(dtype))
    # rows form: x untouched, rows gathered (with a repeat)
    rows = torch.tensor([3, 0, 3, 12], dtype=torch.int32)
    x2 = dev(x.clone())
    got2 = ops.add_rmsnorm(x2, dev(delta), dev(w), 1e-6, dtype, dev(rows))
    want2 = plain_ops.add_rmsnorm(x.clone(), delta, w, 1e-6, dtype, rows)
    torch.testing.assert_close(x2.cpu(), x, atol=0, rtol=0)
    torch.testing.assert_close(got2.cpu().float(), want2.float(), **tol(dtype))
    # no delta
    got3 = ops.add_rmsnorm(dev(x.clone()), None, dev(w), 1e-5, dtype)
    want3 = plain_ops.add_rmsnorm(x.clone(), None, w, 1e-5, dtype)
    torch.testing.assert_close(got3.cpu().float(), want3.float(), **tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
def test_swiglu(ops, dtype):
    torch.manual_seed(2)
    for rows, ff in ((1, 8), (7, 24), (33, 1000), (5, 10), (3, 4099), (4, 2056)):
        g = (torch.randn(rows, 2 * ff) * 4).to(dtype)
        torch.testing.assert_close(ops.swiglu(dev(g)).cpu().float(), plain_ops.swiglu(g).float(), **tol(dtype))


def test_rope_cos_sin(ops):
    pos = torch.tensor([0, 1, 2, 63, 64, 1000, 4095, 100000], dtype=torch.int32)
    inv = 1.0 / torch.pow(torch.tensor(1e6), torch.arange(0, 48, 2, dtype=torch.float32) / 48.0)
    c, s = ops.rope_cos_sin(dev(pos), dev(inv))
    cr, sr = plain_ops.rope_cos_sin(pos, inv)
    torch.testing.assert_close(c.cpu(), cr, atol=2e-6, rtol=0)
    torch.testing.assert_close(s.cpu(), sr, atol=2e-6, rtol=0)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nh,nkv,d,rot", [(4, 2, 16, 16), (6, 1, 32, 32), (3, 3, 48, 32), (5, 5, 256, 256), (8, 2, 64, 64)])
def test_qk_norm_rope_write(ops, dtype, nh, nkv, d, rot):
    torch.manual_seed(3)
    n, page, pages = 11, 16, 7
    qkv = torch.randn(n, (nh + 2 * nkv) * d).to(dtype)
    qw, kw = 1 + 0.1 * torch.randn(d), 1 + 0.1 * torch.randn(d)
    pos = torch.randint(0, 500, (n,), dtype=torch.int32)
    inv = 1.0 / torch.pow(torch.tensor(1e4), torch.arange(0, rot, 2, dtype=torch.float32) / rot)
    cos, sin = plain_ops.rope_cos_sin(pos, inv)
    slots = torch.randperm(page * pages)[:n].to(torch.int32)
    cache = torch.full((pages, 2, nkv, page, d), 7.0).to(dtype)
    cache_ref, qkv_ref = cache.clone(), qkv.clone()
    plain_ops.qk_norm_rope_write(qkv_ref, nh, nkv, d, qw, kw, 1e-5, cos, sin, rot, cache_ref, slots)
    qg, cg = dev(qkv.clone()), dev(cache.clone())
    ops.qk_norm_rope_write(qg, nh, nkv, d, dev(qw), dev(kw), 1e-5, dev(cos), dev(sin), rot, cg, dev(slots))
    torch.testing.assert_close(qg.cpu().float()[:, :nh * d], qkv_ref.float()[:, :nh * d], **tol(dtype))
    torch.testing.assert_close(cg.cpu().float(), cache_ref.float(), **tol(dtype))   # untouched slots keep 7.0
    # no norm, no rope, no cache: q is left as it was
    q2 = dev(qkv.clone())
    ops.qk_norm_rope_write(q2, nh, nkv, d, None, None, 0.0, None, None, rot, None, None)
    torch.testing.assert_close(q2.cpu(), qkv, atol=0, rtol=0)


def _attention_case(ops, dtype, nh, nkv, d, page, lens, window=0, splits=None, planted=False, seed=4, impl="auto"):
    """lens: list of (len_q, len_k) per sequence; pages are handed out in a shuffled order."""
    torch.manual_seed(seed)
    S = len(lens)
    n = sum(q for q, _ in lens)
    need = [-(-k // page) for _, k in lens]
    num_pages = sum(need) + 3
    perm = torch.randperm(num_pages).tolist()
    width = max(need) + 1
    table = torch.zeros((S, width), dtype=torch.int32)
    it = iter(perm)
    for s in range(S):
        for j in range(need[s]):
            table[s, j] = next(it)
    cache = torch.randn(num_pages, 2, nkv, page, d).to(dtype)
    q = torch.randn(n, nh * d).to(dtype)
    if planted:
        # one far key per sequence gets a score that stands out; its value is marked so that
        # losing the key (a page edge, a split boundary) changes the output a lot
        r = 0
        for s, (ql, kl) in enumerate(lens):
            far = min(kl - ql, 3) if kl - ql > 0 else 0
            pg, off = int(table[s, far // page]), far % page
            cache[pg, 0, :, off] = 0
            cache[pg, 0, :, off, 0] = 6.0
            cache[pg, 1, :, off] = 50.0
            q[r:r + ql] = 0
            q.view(n, nh, d)[r:r + ql, :, 0] = 2.0 * math.sqrt(d)   # score 12 for the planted key
            r += ql
    cu_q = torch.tensor([0] + list(itertools.accumulate(a for a, _ in lens)), dtype=torch.int32)
    kl = torch.tensor([b for _, b in lens], dtype=torch.int32)
    max_q, max_k = max(a for a, _ in lens), max(b for _, b in lens)
    scale = 1.0 / math.sqrt(d)
    want = plain_ops.paged_attention(q, nh * d, cache, table, cu_q, kl, n, S, max_q, max_k, nh, nkv, d, scale, window)
    before = ops.launch_count
    got = ops.paged_attention(dev(q), nh * d, dev(cache), dev(table), dev(cu_q), dev(kl), n, S, max_q, max_k,
                              nh, nkv, d, scale, window, splits, None, impl)
    launches = ops.launch_count - before
    t = dict(atol=3e-5, rtol=3e-5) if dtype == torch.float32 else dict(atol=3e-2, rtol=3e-2)
    torch.testing.assert_close(got.cpu().float(), want.float(), **t)
    return launches


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nh,nkv,d", [(4, 2, 16), (6, 1, 32), (3, 1, 48), (8, 2, 64), (2, 2, 128), (40, 1, 16), (2, 1, 256)])
def test_paged_attention_mixed_batch(ops, dtype, nh, nkv, d):
    # a whole prompt, a portion over a cached prefix, decode tokens, a 2-token portion at a page edge
    _attention_case(ops, dtype, nh, nkv, d, 16, [(37, 37), (9, 50), (1, 81), (1, 1), (2, 33), (1, 16), (1, 17)])


@pytest.mark.parametrize("dtype", DTYPES)
def test_paged_attention_far_key_stands_out(ops, dtype):
    _attention_case(ops, dtype, 8, 2, 64, 64, [(1, 700), (5, 300), (1, 65)], planted=True)
    _attention_case(ops, dtype, 8, 2, 64, 64, [(1, 700), (1, 640), (1, 65)], planted=True, splits=4)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("splits", [2, 3, 7])
def test_paged_attention_split_keys(ops, dtype, splits):
    _attention_case(ops, dtype, 8, 2, 64, 32, [(1, 1000), (1, 31), (1, 32), (1, 33), (3, 200)], splits=splits)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("window", [1, 5, 16, 40])
def test_paged_attention_window(ops, dtype, window):
    _attention_case(ops, dtype, 4, 2, 32, 16, [(20, 20), (7, 90), (1, 64), (1, 3)], window=window)
    _attention_case(ops, dtype, 4, 2, 32, 16, [(1, 200), (1, 64)], window=window, splits=3)


# ---- the tensor-core kernel of the serving path (bfloat16, head_dim 64 / 128, pages of 64n) ----
TC = dict(dtype=torch.bfloat16, impl="tensor_core")


@pytest.mark.parametrize("nh,nkv,d,page", [(8, 2, 64, 64), (32, 8, 64, 64), (6, 1, 64, 128), (4, 4, 128, 64), (40, 1, 64, 64), (3, 1, 128, 128)])
def test_tensor_core_attention_mixed_batch(ops, nh, nkv, d, page):
    # whole prompts (one longer than a block's 16 tokens x 4 heads), a portion over a cached prefix,
    # decode tokens at and beside page and tile edges, a 2-token portion
    _attention_case(ops, nh=nh, nkv=nkv, d=d, page=page,
                    lens=[(150, 150), (9, 200), (1, 64), (1, 65), (1, 1), (2, 129), (1, 128), (70, 70), (1, 63)], **TC)


def test_tensor_core_attention_decode_only_and_splits(ops):
    for splits in (1, 2, 5, 16):
        _attention_case(ops, nh=32, nkv=8, d=64, page=64, lens=[(1, 1000), (1, 64), (1, 65), (1, 3), (1, 513)],
                        splits=splits, **TC)
    _attention_case(ops, nh=16, nkv=1, d=128, page=64, lens=[(1, 300), (1, 64)], splits=3, **TC)      # 16 rows exactly
    _attention_case(ops, nh=34, nkv=2, d=64, page=64, lens=[(1, 300), (1, 64)], splits=3, **TC)       # 17 rows: 4-warp blocks


def test_tensor_core_attention_far_key_stands_out(ops):
    _attention_case(ops, nh=8, nkv=2, d=64, page=64, lens=[(1, 700), (5, 300), (1, 65), (100, 400)], planted=True, **TC)
    _attention_case(ops, nh=8, nkv=2, d=64, page=64, lens=[(1, 700), (1, 640), (1, 65)], planted=True, splits=4, **TC)


@pytest.mark.parametrize("window", [1, 5, 64, 100])
def test_tensor_core_attention_window(ops, window):
    _attention_case(ops, nh=4, nkv=2, d=64, page=64, lens=[(90, 90), (7, 300), (1, 64), (1, 3), (1, 129)], window=window, **TC)
    _attention_case(ops, nh=4, nkv=2, d=64, page=64, lens=[(1, 500), (1, 64)], window=window, splits=3, **TC)


def test_tensor_core_attention_far_key_in_a_long_context(ops):
    """Forty thousand keys: the planted key near the start must still be found by a decode token
    (split keys, offsets beyond 2^15 tokens and a cache of tens of megabytes)."""
    _attention_case(ops, nh=8, nkv=2, d=64, page=64, lens=[(1, 40000), (1, 33000), (3, 20000)], planted=True, **TC)


def test_tensor_core_attention_ignores_garbage_beyond_the_sequence(ops):
    """Cache memory past a sequence's last key (and pages nobody wrote) may hold anything,
    NaN included; it must not reach the result."""
    torch.manual_seed(11)
    nh, nkv, d, page = 8, 2, 64, 64
    cache = torch.full((6, 2, nkv, page, d), float("nan")).to(torch.bfloat16)
    lens = [(1, 70), (3, 10)]
    table = torch.tensor([[4, 1, 0, 0], [2, 0, 0, 0]], dtype=torch.int32)
    cache[4] = torch.randn(2, nkv, page, d)
    cache[1, :, :, :6] = torch.randn(2, nkv, 6, d).to(torch.bfloat16)
    cache[2, :, :, :10] = torch.randn(2, nkv, 10, d).to(torch.bfloat16)
    q = torch.randn(4, nh * d).to(torch.bfloat16)
    cu, kl = torch.tensor([0, 1, 4], dtype=torch.int32), torch.tensor([70, 10], dtype=torch.int32)
    want = plain_ops.paged_attention(q, nh * d, cache, table, cu, kl, 4, 2, 3, 70, nh, nkv, d, 0.125)
    for impl in ("tensor_core", "general"):
        got = ops.paged_attention(dev(q), nh * d, dev(cache), dev(table), dev(cu), dev(kl), 4, 2, 3, 70, nh, nkv, d,
                                  0.125, 0, None, None, impl)
        assert torch.isfinite(got.float()).all(), impl
        torch.testing.assert_close(got.cpu().float(), want.float(), atol=3e-2, rtol=3e-2)


def test_tensor_core_attention_is_refused_where_it_does_not_apply(ops):
    with pytest.raises(ops.KernelError, match="tensor-core kernel needs"):
        _attention_case(ops, nh=4, nkv=2, d=32, page=64, lens=[(1, 10)], **TC)
    with pytest.raises(ops.KernelError, match="tensor-core kernel needs"):
        _attention_case(ops, nh=4, nkv=2, d=64, page=16, lens=[(1, 10)], **TC)


# ---- the tcgen05 kernel for prompt portions (bfloat16, head_dim 64, pages of 64n) ----
T5 = dict(dtype=torch.bfloat16, impl="tcgen05")


@pytest.mark.parametrize("nh,nkv,page", [(8, 2, 64), (32, 8, 64), (6, 1, 128), (4, 4, 64), (40, 8, 64), (3, 1, 64)])
def test_tcgen05_attention_mixed_batch(ops, nh, nkv, page):
    # whole prompts (shorter and longer than a block's 128 rows, ending inside and at the end of a
    # page), portions over a cached prefix, single tokens, a 2-token portion at a page edge
    _attention_case(ops, nh=nh, nkv=nkv, d=64, page=page,
                    lens=[(150, 150), (9, 200), (1, 64), (1, 65), (1, 1), (2, 129), (128, 128), (70, 390), (33, 63)], **T5)


def test_tcgen05_attention_long_prompt_and_far_key(ops):
    _attention_case(ops, nh=8, nkv=2, d=64, page=64, lens=[(1100, 1100)], **T5)
    _attention_case(ops, nh=8, nkv=2, d=64, page=64, lens=[(300, 700), (5, 300), (1, 65), (100, 400)], planted=True, **T5)


@pytest.mark.parametrize("window", [1, 5, 64, 100])
def test_tcgen05_attention_window(ops, window):
    _attention_case(ops, nh=4, nkv=2, d=64, page=64, lens=[(90, 90), (7, 300), (1, 64), (200, 500), (1, 129)], window=window, **T5)


def test_tcgen05_attention_ignores_garbage_beyond_the_sequence(ops):
    torch.manual_seed(12)
    nh, nkv, d, page = 8, 2, 64, 64
    cache = torch.full((6, 2, nkv, page, d), float("nan")).to(torch.bfloat16)
    table = torch.tensor([[4, 1, 0, 0], [2, 0, 0, 0]], dtype=torch.int32)
    cache[4] = torch.randn(2, nkv, page, d)
    cache[1, :, :, :6] = torch.randn(2, nkv, 6, d).to(torch.bfloat16)
    cache[2, :, :, :10] = torch.randn(2, nkv, 10, d).to(torch.bfloat16)
    q = torch.randn(43, nh * d).to(torch.bfloat16)
    cu, kl = torch.tensor([0, 40, 43], dtype=torch.int32), torch.tensor([70, 10], dtype=torch.int32)
    want = plain_ops.paged_attention(q, nh * d, cache, table, cu, kl, 43, 2, 40, 70, nh, nkv, d, 0.125)
    got = ops.paged_attention(dev(q), nh * d, dev(cache), dev(table), dev(cu), dev(kl), 43, 2, 40, 70, nh, nkv, d,
                              0.125, 0, None, None, "tcgen05")
    assert torch.isfinite(got.float()).all()
    torch.testing.assert_close(got.cpu().float(), want.float(), atol=3e-2, rtol=3e-2)


DEC = dict(dtype=torch.bfloat16, impl="decode")


@pytest.mark.parametrize("nh,nkv", [(8, 2), (6, 2), (16, 1), (5, 5), (32, 8)])
@pytest.mark.parametrize("page", [64, 128, 256])
@pytest.mark.parametrize("splits", [1, 3])
def test_decode_attention_mixed_lengths(ops, nh, nkv, page, splits):
    # single tokens over contexts that end at, before and after a tile's and a page's edge, the very
    # first token, and short portions (as many tokens as 16 rows allow)
    tokens = 16 // (nh // nkv)
    lens = [(1, 1), (1, 63), (1, 64), (1, 65), (1, 128), (1, 129), (1, 700), (1, 257), (1, 1000)]
    if tokens >= 2:
        lens += [(2, 129), (tokens, 400), (tokens, tokens), (2, 64)]
    _attention_case(ops, nh=nh, nkv=nkv, d=64, page=page, lens=lens, splits=splits, **DEC)


def _decode_launches(ops, num_seqs, nkv, splits):
    """One launch while the slices of a (sequence, kv head) combine among themselves as a
    thread-block cluster, two (the kernel, then the combine kernel) otherwise."""
    return 1 if splits == 1 or ops.decode_attention_combines(num_seqs, nkv, splits) else 2


@pytest.mark.parametrize("splits", [1, 2, 5, 9, 12, 16, 32])
def test_decode_attention_far_key_and_many_slices(ops, splits):
    # (1, 65) is two tiles of keys: with more slices than that, most of its slices are empty
    lens = [(1, 2500), (1, 640), (1, 65), (2, 3000)]
    launches = _attention_case(ops, nh=8, nkv=2, d=64, page=64, lens=lens, planted=True, splits=splits, **DEC)
    assert launches == _decode_launches(ops, len(lens), 2, splits)
    _, cluster = ops.decode_attention_limits()
    if 1 < splits <= cluster:
        assert launches == 1, "a resident grid of at most a cluster's worth of slices combines inside the kernel"
    if splits > cluster:
        assert launches == 2


@pytest.mark.parametrize("splits", [9, 12, 16])
@pytest.mark.parametrize("lens", [[(1, 4096)], [(1, 700), (1, 8000)], [(1, 200)]])
def test_decode_attention_large_clusters_few_sequences(ops, splits, lens):
    """One or two sequences over long and short contexts (decode at batch 1 or 2): slices above the
    portable cluster size, slices that get no tile at all, and the planted far key in the first."""
    launches = _attention_case(ops, nh=32, nkv=8, d=64, page=64, lens=lens, planted=True, splits=splits, **DEC)
    assert launches == _decode_launches(ops, len(lens), 8, splits)


@pytest.mark.parametrize("window", [1, 5, 64, 100, 1000])
def test_decode_attention_window(ops, window):
    _attention_case(ops, nh=8, nkv=2, d=64, page=64, lens=[(1, 90), (1, 300), (1, 64), (3, 500), (1, 129), (1, 1)],
                    window=window, **DEC)
    _attention_case(ops, nh=8, nkv=2, d=64, page=128, lens=[(1, 900), (2, 300)], window=window, splits=4, **DEC)
    for splits in (9, 12, 16):
        launches = _attention_case(ops, nh=8, nkv=2, d=64, page=64, lens=[(1, 2000), (2, 1300)], window=window,
                                   planted=True, splits=splits, **DEC)
        assert launches == _decode_launches(ops, 2, 2, splits)


def test_decode_attention_ignores_garbage_beyond_the_sequence(ops):
    torch.manual_seed(13)
    nh, nkv, d, page = 8, 2, 64, 128
    cache = torch.full((6, 2, nkv, page, d), float("nan")).to(torch.bfloat16)
    table = torch.tensor([[4, 1, 0, 0], [2, 0, 0, 0], [5, 0, 0, 0]], dtype=torch.int32)
    cache[4] = torch.randn(2, nkv, page, d)
    cache[1, :, :, :6] = torch.randn(2, nkv, 6, d).to(torch.bfloat16)
    cache[2, :, :, :10] = torch.randn(2, nkv, 10, d).to(torch.bfloat16)
    cache[5, :, :, :70] = torch.randn(2, nkv, 70, d).to(torch.bfloat16)
    q = torch.randn(4, nh * d).to(torch.bfloat16)
    cu, kl = torch.tensor([0, 1, 2, 4], dtype=torch.int32), torch.tensor([134, 10, 70], dtype=torch.int32)
    want = plain_ops.paged_attention(q, nh * d, cache, table, cu, kl, 4, 3, 2, 134, nh, nkv, d, 0.125)
    for splits in (1, 2):
        got = ops.paged_attention(dev(q), nh * d, dev(cache), dev(table), dev(cu), dev(kl), 4, 3, 2, 134, nh, nkv, d,
                                  0.125, 0, splits, None, "decode")
        assert torch.isfinite(got.float()).all()
        torch.testing.assert_close(got.cpu().float(), want.float(), atol=3e-2, rtol=3e-2)


@pytest.mark.parametrize("nh,nkv,page,splits", [(8, 2, 64, 1), (8, 2, 64, 3), (32, 8, 128, 5), (6, 2, 64, 2), (4, 4, 64, 1),
                                                (16, 1, 256, 4), (8, 2, 64, 12)])
@pytest.mark.parametrize("norm,rope,write", [(True, True, True), (False, True, True), (True, False, True), (True, True, False)])
def test_decode_attention_fused_with_norm_rope_and_cache_write(ops, nh, nkv, page, splits, norm, rope, write):
    """One kernel against the two it stands for, on the same inputs: the same output and the same cache, bit for
    bit, and both close to the plain functions.  Sequences end at and around tile and page edges, some bring
    several tokens (which may lie in two tiles, and so in two slices), the first token of a sequence included."""
    torch.manual_seed(5)
    d, n_rep = 64, nh // nkv
    tokens = 16 // n_rep
    lens = [(1, 1), (1, 64), (1, 65), (1, 128), (1, 129), (1, 700), (1, 1000), (1, 63)]
    if tokens >= 2:
        lens += [(2, 65), (tokens, 400), (tokens, tokens), (2, 129), (min(tokens, 3), 66)]
    S, n = len(lens), sum(a for a, _ in lens)
    need = [-(-k // page) for _, k in lens]
    num_pages = sum(need) + 2
    perm = torch.randperm(num_pages).tolist()
    table = torch.zeros((S, max(need) + 1), dtype=torch.int32)
    it = iter(perm)
    for s_ in range(S):
        for j in range(need[s_]):
            table[s_, j] = next(it)
    cache = torch.randn(num_pages, 2, nkv, page, d).to(torch.bfloat16)
    qkv = torch.randn(n, (nh + 2 * nkv) * d).to(torch.bfloat16)
    qw = (1 + 0.2 * torch.randn(d)) if norm else None
    kw = (1 + 0.2 * torch.randn(d)) if norm else None
    pos, slots = [], []
    for s_, (a, b) in enumerate(lens):
        for j in range(a):
            p_ = b - a + j
            pos.append(p_)
            slots.append(int(table[s_, p_ // page]) * page + p_ % page)
    cos = sin = None
    if rope:
        ang = torch.tensor(pos, dtype=torch.float32)[:, None] * (1e4 ** (-torch.arange(0, d, 2).float() / d))[None]
        cos, sin = ang.cos().contiguous(), ang.sin().contiguous()
    cu = torch.tensor([0] + list(itertools.accumulate(a for a, _ in lens)), dtype=torch.int32)
    kl = torch.tensor([b for _, b in lens], dtype=torch.int32)
    sm = torch.tensor(slots, dtype=torch.int32)
    max_q, max_k, scale = max(a for a, _ in lens), max(b for _, b in lens), 0.125
    # the plain functions
    p_qkv, p_cache = qkv.clone(), cache.clone()
    plain_ops.qk_norm_rope_write(p_qkv, nh, nkv, d, qw, kw, 1e-5, cos, sin, d, p_cache if write else None, sm)
    want = plain_ops.paged_attention(p_qkv, (nh + 2 * nkv) * d, p_cache, table, cu, kl, n, S, max_q, max_k, nh, nkv, d, scale)
    # two kernels
    g_qkv, g_cache = dev(qkv.clone()), dev(cache.clone())
    ops.qk_norm_rope_write(g_qkv, nh, nkv, d, dev(qw), dev(kw), 1e-5, dev(cos), dev(sin), d, g_cache if write else None, dev(sm))
    two = ops.paged_attention(g_qkv, (nh + 2 * nkv) * d, g_cache, dev(table), dev(cu), dev(kl), n, S, max_q, max_k,
                              nh, nkv, d, scale, 0, splits, None, "decode")
    # one kernel
    f_qkv, f_cache = dev(qkv.clone()), dev(cache.clone())
    before = ops.launch_count
    one = ops.decode_attention_fused(f_qkv, nh, nkv, d, dev(qw), dev(kw), 1e-5, dev(cos), dev(sin), f_cache, write,
                                     dev(table), dev(cu), dev(kl), n, S, max_q, max_k, scale, 0, splits)
    assert ops.launch_count - before == (1 if splits == 1 or ops.decode_attention_combines(S, nkv, splits) else 2)
    assert torch.equal(f_qkv.cpu(), qkv), "qkv is left as it was"
    assert torch.equal(f_cache.cpu().view(torch.int16), g_cache.cpu().view(torch.int16)), "the same cache, bit for bit"
    assert torch.equal(one.cpu().view(torch.int16), two.cpu().view(torch.int16)), "the same output, bit for bit"
    torch.testing.assert_close(one.cpu().float(), want.float(), atol=3e-2, rtol=3e-2)
    if write:
        torch.testing.assert_close(f_cache.cpu().float(), p_cache.float(), atol=2e-2, rtol=2e-2)
    else:
        assert torch.equal(f_cache.cpu().view(torch.int16), cache.view(torch.int16)), "a reader leaves the cache alone"


def test_decode_attention_fused_refuses_what_it_cannot_do(ops):
    qkv = torch.zeros(1, (4 + 4) * 128, dtype=torch.bfloat16, device="cuda")
    cache = torch.zeros(2, 2, 2, 64, 128, dtype=torch.bfloat16, device="cuda")
    z = torch.zeros(1, 1, dtype=torch.int32, device="cuda")
    cu = torch.tensor([0, 1], dtype=torch.int32, device="cuda")
    kl = torch.tensor([1], dtype=torch.int32, device="cuda")
    with pytest.raises(ops.KernelError, match="needs head_dim 64"):
        ops.decode_attention_fused(qkv, 4, 2, 128, None, None, 0.0, None, None, cache, True, z, cu, kl, 1, 1, 1, 1, 0.1)
    assert not ops.decode_attention_fused_applies(torch.bfloat16, 64, 64, 4, 32)      # a partial rotation
    assert not ops.decode_attention_fused_applies(torch.bfloat16, 64, 64, 17, 64)
    assert ops.decode_attention_fused_applies(torch.bfloat16, 64, 128, 16, None)


def test_decode_attention_is_what_a_decode_step_gets_and_refuses_what_it_cannot_do(ops):
    before = ops.launch_count
    _attention_case(ops, dtype=torch.bfloat16, nh=32, nkv=8, d=64, page=64, lens=[(1, 500), (1, 64), (4, 95)], splits=1)
    assert ops.launch_count - before == 1
    assert ops.decode_attention_applies(torch.bfloat16, 64, 64, 16)
    assert not ops.decode_attention_applies(torch.bfloat16, 128, 64, 4)
    assert not ops.decode_attention_applies(torch.float32, 64, 64, 4)
    with pytest.raises(ops.KernelError, match="decode kernel needs"):
        _attention_case(ops, nh=4, nkv=2, d=128, page=64, lens=[(1, 70)], **DEC)
    with pytest.raises(ops.KernelError, match="decode kernel needs"):
        _attention_case(ops, nh=8, nkv=2, d=64, page=64, lens=[(5, 70)], **DEC)
    with pytest.raises(ops.KernelError, match="decode kernel needs"):
        _attention_case(ops, nh=8, nkv=2, d=64, page=32, lens=[(1, 70)], **DEC)


@pytest.mark.parametrize("splits", [1, 3])
def test_short_portions_beside_decode_tokens_share_two_kernels(ops, splits):
    # no portion long enough for tcgen05: portions of more than 16 rows on the four-warp flash kernel, decode
    # tokens on the decode kernel, and one combine kernel for the slices of both
    before = ops.launch_count
    _attention_case(ops, dtype=torch.bfloat16, nh=32, nkv=8, d=64, page=64,
                    lens=[(10, 300), (1, 500), (4, 100), (5, 64), (1, 1), (20, 20), (1, 1500)], splits=splits, planted=True)
    assert ops.launch_count - before == (2 if splits == 1 else 3)


def test_attention_picks_its_kernels_for_a_mixed_step(ops):
    # "auto": prompt portions on tcgen05, short portions beside them on the flash kernel, decode tokens
    # (and portions of at most 16 rows) on the decode kernel
    before = ops.launch_count
    _attention_case(ops, dtype=torch.bfloat16, nh=32, nkv=8, d=64, page=64,
                    lens=[(1, 500), (300, 300), (1, 64), (31, 95), (32, 96), (1, 1), (64, 1000), (4, 200), (5, 201), (1, 2000)],
                    splits=1, planted=True)
    assert ops.launch_count - before == 3
    with pytest.raises(ops.KernelError, match="tcgen05 kernel needs"):
        _attention_case(ops, nh=4, nkv=2, d=128, page=64, lens=[(70, 70)], **T5)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("L,bias,hidden", [(3, False, 72), (4, True, 96), (2, True, 40), (1, False, 64), (8, False, 130), (3, True, 2048)])
def test_shortconv_portions_and_state(ops, dtype, L, bias, hidden):
    """Several steps over the same requests: portions shorter than the state, single tokens,
    a fresh request in a slot another one used (stale state must not leak in)."""
    torch.manual_seed(5)
    slots_n = 5
    state_ref = torch.full((slots_n, max(L - 1, 1), hidden), 9.0).to(dtype)[:, :L - 1]
    state_gpu = dev(state_ref.clone())
    taps = torch.randn(L, hidden)
    in_b = torch.randn(3 * hidden) if bias else None
    cv_b = torch.randn(hidden) if bias else None
    # (slot, start position, portion length) per sequence and step
    steps = [
        [(2, 0, 1), (0, 0, 7), (4, 0, 2)],
        [(2, 1, 1), (0, 7, 2), (4, 2, 1), (1, 0, 3)],
        [(2, 2, 5), (0, 9, 1), (4, 3, 2)],
        [(2, 0, 4), (3, 0, 1)],          # slot 2 starts over: a new request in a used slot
        [(2, 4, 1), (3, 1, 1)],
    ]
    for step in steps:
        n = sum(q for _, _, q in step)
        h3 = torch.randn(n, 3 * hidden).to(dtype)
        cu, pos, tseq = [0], [], []
        for i, (_, p0, q) in enumerate(step):
            cu.append(cu[-1] + q)
            pos += list(range(p0, p0 + q))
            tseq += [i] * q
        ss = torch.tensor([s for s, _, _ in step], dtype=torch.int32)
        cu_t, pos_t, ts_t = (torch.tensor(v, dtype=torch.int32) for v in (cu, pos, tseq))
        want = plain_ops.shortconv(h3, in_b, taps, cv_b, state_ref, ss, ts_t, cu_t, pos_t)
        got = ops.shortconv(dev(h3), dev(in_b), dev(taps), dev(cv_b), state_gpu if L > 1 else None, dev(ss),
                            dev(ts_t), dev(cu_t), dev(pos_t))
        torch.testing.assert_close(got.cpu().float(), want.float(), **tol(dtype))
        if L > 1:
            torch.testing.assert_close(state_gpu.cpu().float(), state_ref.float(), **tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("L,bias,hidden", [(3, False, 2048), (4, True, 96), (2, False, 72), (5, True, 264), (8, False, 64),
                                           (3, False, 100)])
def test_shortconv_prompt_sized_steps(ops, dtype, L, bias, hidden):
    """Steps of hundreds of tokens (token tiles for everything past the first L-1 tokens of a
    portion, the per-token kernel for those and the state): portions that start in the middle
    of a tile, a portion shorter than the state beside long ones, a second step that continues
    from the state the first one left."""
    torch.manual_seed(15)
    state_ref = torch.full((4, max(L - 1, 1), hidden), 9.0).to(dtype)[:, :L - 1]
    state_gpu = dev(state_ref.clone())
    taps = torch.randn(L, hidden)
    in_b = torch.randn(3 * hidden) if bias else None
    cv_b = torch.randn(hidden) if bias else None
    steps = [[(0, 0, 301), (1, 5, 2), (2, 0, 99)], [(0, 301, 257), (2, 99, 1), (1, 7, 43), (3, 0, 6)]]
    for step in steps:
        n = sum(q for _, _, q in step)
        h3 = torch.randn(n, 3 * hidden).to(dtype)
        cu, pos, tseq = [0], [], []
        for i, (_, p0, q) in enumerate(step):
            cu.append(cu[-1] + q)
            pos += list(range(p0, p0 + q))
            tseq += [i] * q
        ss = torch.tensor([s for s, _, _ in step], dtype=torch.int32)
        cu_t, pos_t, ts_t = (torch.tensor(v, dtype=torch.int32) for v in (cu, pos, tseq))
        want = plain_ops.shortconv(h3, in_b, taps, cv_b, state_ref, ss, ts_t, cu_t, pos_t)
        got = ops.shortconv(dev(h3), dev(in_b), dev(taps), dev(cv_b), state_gpu, dev(ss), dev(ts_t), dev(cu_t),
                            dev(pos_t))
        torch.testing.assert_close(got.cpu().float(), want.float(), **tol(dtype))
        torch.testing.assert_close(state_gpu.cpu().float(), state_ref.float(), **tol(dtype))


def test_sample_rows_greedy_ties_and_gumbel(ops):
    torch.manual_seed(6)
    V = 1000
    logits = torch.randn(6, V)
    logits[0, 17] = logits[0, 900] = 50.0                  # a tie: the lowest id wins
    got = ops.sample_rows(dev(logits)).cpu()
    assert got.tolist() == plain_ops.sample_rows(logits).tolist()
    assert got[0] == 17
    mode = torch.tensor([1, 2, 2, 0, 2, 2], dtype=torch.int32)
    inv_t = torch.tensor([1.0, 1.25, 0.5, 1.0, 2.0, 1.0])
    seeds = torch.tensor([0, 3, 3, 0, 2 ** 62 + 5, -7], dtype=torch.int64)
    draws = torch.tensor([0, 0, 1, 0, 9, 4], dtype=torch.int64)
    out = torch.full((6,), -1, dtype=torch.int32)
    got = ops.sample_rows(dev(logits), dev(mode), dev(inv_t), dev(seeds), dev(draws), dev(out)).cpu()
    want = plain_ops.sample_rows(logits, mode, inv_t, seeds, draws, torch.full((6,), -1, dtype=torch.int32))
    assert got.tolist() == want.tolist()
    assert got[3] == -1                                     # mode 0: untouched
    # same (seed, draw) -> same token, whatever row it sits in
    again = ops.sample_rows(dev(logits[[2, 1]].contiguous()), dev(mode[[2, 1]].contiguous()),
                            dev(inv_t[[2, 1]].contiguous()), dev(seeds[[2, 1]].contiguous()),
                            dev(draws[[2, 1]].contiguous())).cpu()
    assert again.tolist() == [int(got[2]), int(got[1])]


def test_gumbel_follows_the_tempered_softmax(ops):
    """Frequencies of many draws against softmax(logits / T), within 4 sigma per token
    (the reference's own check, crates/vapi-backend-candle/src/fused.rs:767-857)."""
    logits = torch.tensor([[2.0, 1.0, 0.0, -1.0, 0.5, -3.0, 1.5, 0.0]])
    T, N = 0.7, 4000
    big = logits.repeat(N, 1).contiguous()
    mode = torch.full((N,), 2, dtype=torch.int32)
    inv_t = torch.full((N,), 1.0 / T)
    seeds = torch.full((N,), 11, dtype=torch.int64)
    draws = torch.arange(N, dtype=torch.int64)
    toks = ops.sample_rows(dev(big), dev(mode), dev(inv_t), dev(seeds), dev(draws)).cpu()
    p = torch.softmax(logits[0] / T, 0)
    freq = torch.bincount(toks.long(), minlength=8).float() / N
    sigma = torch.sqrt(p * (1 - p) / N)
    assert torch.all((freq - p).abs() <= 4 * sigma + 1e-3), (freq, p)


def test_apply_penalties(ops):
    torch.manual_seed(7)
    logits = torch.randn(3, 50)
    rows = torch.tensor([0, 0, 2, 2], dtype=torch.int32)
    toks = torch.tensor([4, 9, 4, 30], dtype=torch.int32)
    counts = torch.tensor([1.0, 3.0, 2.0, 1.0])
    rep, freq, pres = torch.tensor([1.3, 1.0, 0.8]), torch.tensor([0.1, 0.0, 0.5]), torch.tensor([0.2, 0.0, 0.0])
    want = logits.clone()
    plain_ops.apply_penalties(want, rows, toks, counts, rep, freq, pres)
    got = dev(logits.clone())
    ops.apply_penalties(got, dev(rows), dev(toks), dev(counts), dev(rep), dev(freq), dev(pres))
    torch.testing.assert_close(got.cpu(), want, atol=1e-6, rtol=1e-6)


@pytest.mark.parametrize("dtype", DTYPES)
def test_linear_is_not_reduced_precision(ops, dtype):
    torch.manual_seed(8)
    ops.strict_fp32()
    x = torch.randn(9, 300).to(dtype)
    w = torch.randn(70, 300).to(dtype)
    b = torch.randn(70)
    got = ops.linear(dev(x), dev(w), dev(b.to(dtype)))
    want = plain_ops.linear(x, w, b.to(dtype))
    t = dict(atol=1e-4, rtol=1e-5) if dtype == torch.float32 else dict(atol=0.3, rtol=2e-2)
    torch.testing.assert_close(got.cpu().float(), want.float(), **t)
    if dtype == torch.bfloat16:
        got32 = ops.linear(dev(x), dev(w), None, torch.float32)
        assert got32.dtype == torch.float32
        torch.testing.assert_close(got32.cpu(), plain_ops.linear(x, w, None, torch.float32), atol=2e-3, rtol=1e-4)
        # a weight kept in float32 beside bfloat16 activations multiplies in float32
        got_mixed = ops.linear(dev(x), dev(w.float()))
        torch.testing.assert_close(got_mixed.cpu().float(), plain_ops.linear(x, w).float(), atol=0.3, rtol=2e-2)


# ---- the weight-streaming product of decode steps ---------------------------------------------
@pytest.mark.parametrize("M", [1, 3, 8, 9, 16])
@pytest.mark.parametrize("N,K", [(72, 96), (2048, 2048), (1000, 320), (6144, 1536), (520, 4096), (300, 2560), (48, 2080)])
def test_skinny_linear_plain_products(ops, M, N, K):
    # (inner sizes up to 2048: the tokens' rows live in registers; above: in the copy queue)
    torch.manual_seed(20)
    w = (torch.randn(N, K) * 0.05).to(torch.bfloat16)
    a = torch.randn(M, K).to(torch.bfloat16)
    b = torch.randn(N)
    want = a.float() @ w.float().t()
    for rpb in (8, 16):
        got = ops.skinny_linear(dev(w), act=dev(a), epilogue="f32", rows_per_block=rpb)
        torch.testing.assert_close(got.cpu(), want, atol=2e-3, rtol=1e-3)
    got = ops.skinny_linear(dev(w), act=dev(a), epilogue="bf16", bias=dev(b))
    torch.testing.assert_close(got.cpu().float(), (want + b).to(torch.bfloat16).float(), atol=2e-2, rtol=2e-2)
    # and `linear` sends decode-sized bfloat16 products there
    before = ops.launch_count
    got = ops.linear(dev(a), dev(w), None, torch.float32)
    assert ops.launch_count == before + 1
    torch.testing.assert_close(got.cpu(), want, atol=2e-3, rtol=1e-3)


@pytest.mark.parametrize("M", [1, 8, 13])
def test_skinny_linear_fusions(ops, M):
    """Deferred-norm prologue, SwiGLU epilogue, residual epilogue that prepares the next norm: a
    feed-forward of a decode step as two launches."""
    torch.manual_seed(21)
    H, F, eps = 96, 200, 1e-6
    x = torch.randn(M, H) * 2
    nw = 1 + 0.1 * torch.randn(H)
    w13 = (torch.randn(2 * F, H) * 0.2).to(torch.bfloat16)
    w2 = (torch.randn(H, 224) * 0.2).to(torch.bfloat16)
    # what a producer with 5 blocks would leave: partial sums of squares and bfloat16(x * weight)
    parts = torch.stack([(x[:, i * 20:(i + 1) * 20] ** 2).sum(1) for i in range(4)] + [(x[:, 80:] ** 2).sum(1)]).contiguous()
    xw = (x * nw).to(torch.bfloat16)
    s = ops.skinny_linear(dev(w13), xw=dev(xw), ss_in=dev(parts), eps=eps, epilogue="swiglu")
    inv = torch.rsqrt((x ** 2).mean(1, keepdim=True) + eps)
    gu = (xw.float() @ w13.float().t()) * inv
    want_s = (gu[:, :F] / (1 + torch.exp(-gu[:, :F]))) * gu[:, F:]
    torch.testing.assert_close(s.cpu().float(), want_s.to(torch.bfloat16).float(), atol=3e-2, rtol=3e-2)
    # and against the norm done the ordinary way (rounding the normed row instead of x * w)
    xn = (x * inv * nw).to(torch.bfloat16).float()
    gu2 = xn @ w13.float().t()
    torch.testing.assert_close(s.cpu().float(), ((gu2[:, :F] / (1 + torch.exp(-gu2[:, :F]))) * gu2[:, F:]), atol=6e-2, rtol=6e-2)
    # down projection (inner size 224 = 7 * 32) added into the stream, preparing the next norm
    s2 = torch.randn(M, 224).to(torch.bfloat16)
    bias, nw2 = torch.randn(H), 1 + 0.1 * torch.randn(H)
    for rpb in (8, 16):
        xr = dev(x.clone())
        ss, xw2 = ops.skinny_linear(dev(w2), act=dev(s2), epilogue="resid", resid=xr, bias=dev(bias),
                                    next_weight=dev(nw2), rows_per_block=rpb)
        want_x = x + s2.float() @ w2.float().t() + bias
        torch.testing.assert_close(xr.cpu(), want_x, atol=2e-3, rtol=1e-3)
        assert ss.shape == (ops.skinny_blocks(H, "resid", rpb), M)
        torch.testing.assert_close(ss.sum(0).cpu(), (want_x ** 2).sum(1), atol=1e-2, rtol=1e-3)
        torch.testing.assert_close(xw2.cpu().float(), (want_x * nw2).to(torch.bfloat16).float(), atol=3e-2, rtol=2e-2)
    none = ops.skinny_linear(dev(w2), act=dev(s2), epilogue="resid", resid=dev(x.clone()))
    assert none == (None, None)
    # the same call twice gives the same bits (fixed reduction order, no atomics)
    a = ops.skinny_linear(dev(w13), xw=dev(xw), ss_in=dev(parts), eps=eps, epilogue="swiglu")
    assert torch.equal(a, s)
    # logits epilogue through the deferred norm
    wv = (torch.randn(300, H) * 0.2).to(torch.bfloat16)
    lg = ops.skinny_linear(dev(wv), xw=dev(xw), ss_in=dev(parts), eps=eps, epilogue="f32")
    torch.testing.assert_close(lg.cpu(), (xw.float() @ wv.float().t()) * inv, atol=2e-3, rtol=1e-3)


@pytest.mark.parametrize("M", [8, 11, 16])
def test_skinny_linear_fusions_with_more_tiles_than_blocks(ops, M):
    """The same fusions where a product has more tiles than the device has SMs: with 9..16 rows a block's
    sixteen warps then walk the tiles as two groups of eight, each with its own sums and barriers."""
    torch.manual_seed(23)
    H, F, eps = 2432, 1304, 1e-5                      # 152 tiles of 16 rows, 163 tiles of 8 gate/up pairs
    x = torch.randn(M, H)
    nw = 1 + 0.1 * torch.randn(H)
    w13 = (torch.randn(2 * F, H) * 0.05).to(torch.bfloat16)
    w2 = (torch.randn(H, 1312) * 0.05).to(torch.bfloat16)
    parts = torch.stack([(x[:, i::7] ** 2).sum(1) for i in range(7)]).contiguous()
    xw = (x * nw).to(torch.bfloat16)
    inv = torch.rsqrt((x ** 2).mean(1, keepdim=True) + eps)
    s_ = ops.skinny_linear(dev(w13), xw=dev(xw), ss_in=dev(parts), eps=eps, epilogue="swiglu")
    gu = (xw.float() @ w13.float().t()) * inv
    want_s = (gu[:, :F] / (1 + torch.exp(-gu[:, :F]))) * gu[:, F:]
    torch.testing.assert_close(s_.cpu().float(), want_s, atol=3e-2, rtol=3e-2)
    s2 = torch.randn(M, 1312).to(torch.bfloat16)
    nw2 = 1 + 0.1 * torch.randn(H)
    xr = dev(x.clone())
    ss, xw2 = ops.skinny_linear(dev(w2), act=dev(s2), epilogue="resid", resid=xr, next_weight=dev(nw2))
    want_x = x + s2.float() @ w2.float().t()
    torch.testing.assert_close(xr.cpu(), want_x, atol=3e-3, rtol=1e-3)
    assert ss.shape == (152, M)
    torch.testing.assert_close(ss.sum(0).cpu(), (want_x ** 2).sum(1), atol=5e-2, rtol=1e-3)
    torch.testing.assert_close(xw2.cpu().float(), (want_x * nw2).to(torch.bfloat16).float(), atol=4e-2, rtol=2e-2)
    lg = ops.skinny_linear(dev(w13), xw=dev(xw), ss_in=dev(parts), eps=eps, epilogue="f32")
    torch.testing.assert_close(lg.cpu(), gu, atol=5e-3, rtol=2e-3)
    assert torch.equal(ops.skinny_linear(dev(w13), xw=dev(xw), ss_in=dev(parts), eps=eps, epilogue="swiglu"), s_)


@pytest.fixture()
def tma_weights(ops):
    """The decode product in its second form: weights by TMA into mbarrier rings."""
    was = ops.skinny_use_tma(True)
    yield
    ops.skinny_use_tma(was)


@pytest.mark.parametrize("M", [1, 3, 8])
@pytest.mark.parametrize("N,K", [(72, 96), (2048, 2048), (1000, 320), (6144, 1536), (48, 2016), (4100, 64)])
def test_skinny_linear_with_weights_by_tma(ops, tma_weights, M, N, K):
    """Every prologue and epilogue of the decode product in the form whose weights come by TMA:
    bit for bit what the form with per-lane copies gives (the sums are formed in the same order)."""
    torch.manual_seed(26)
    w = (torch.randn(N, K) * 0.05).to(torch.bfloat16)
    a = torch.randn(M, K).to(torch.bfloat16)
    b = torch.randn(N)
    x = torch.randn(M, K) * 2
    nw = 1 + 0.1 * torch.randn(K)
    parts = torch.stack([(x[:, i::5] ** 2).sum(1) for i in range(5)]).contiguous()
    xw = (x * nw).to(torch.bfloat16)
    nw2 = 1 + 0.1 * torch.randn(N)

    def run():
        out = [ops.skinny_linear(dev(w), act=dev(a), epilogue="f32"),
               ops.skinny_linear(dev(w), act=dev(a), epilogue="bf16", bias=dev(b)),
               ops.skinny_linear(dev(w), xw=dev(xw), ss_in=dev(parts), eps=1e-5, epilogue="f32"),
               ops.skinny_linear(dev(w), xw=dev(xw), ss_in=dev(parts), eps=1e-5, epilogue="bf16")]
        if N % 2 == 0:
            out.append(ops.skinny_linear(dev(w), xw=dev(xw), ss_in=dev(parts), eps=1e-5, epilogue="swiglu"))
            out.append(ops.skinny_linear(dev(w), act=dev(a), epilogue="swiglu"))
        r = dev(torch.arange(M * N, dtype=torch.float32).reshape(M, N) / 100)
        ss, xw2 = ops.skinny_linear(dev(w), act=dev(a), epilogue="resid", resid=r, bias=dev(b), next_weight=dev(nw2))
        return out + [r, ss, xw2]

    got = run()
    ops.skinny_use_tma(False)
    want = run()
    ops.skinny_use_tma(True)
    torch.testing.assert_close(got[0].cpu(), a.float() @ w.float().t(), atol=2e-3, rtol=1e-3)
    for i, (g_, w_) in enumerate(zip(got, want)):
        assert torch.equal(g_, w_), f"output {i} differs between the two forms"


@pytest.mark.parametrize("M", [2, 8, 14])
@pytest.mark.parametrize("N,K", [(2048, 8192), (1536, 6912), (256, 4096), (2048, 2048)])
def test_skinny_linear_residual_epilogue_over_a_long_inner_size(ops, M, N, K):
    """The down projection's shapes: a long inner size with no more tiles than SMs takes the deeper
    copy queue; the residual stream is read early and must still be this call's own element."""
    torch.manual_seed(24)
    w = (torch.randn(N, K) * 0.02).to(torch.bfloat16)
    a = torch.randn(M, K).to(torch.bfloat16)
    x = torch.randn(M, N)
    nw = 1 + 0.1 * torch.randn(N)
    xr = dev(x.clone())
    ss, xw = ops.skinny_linear(dev(w), act=dev(a), epilogue="resid", resid=xr, next_weight=dev(nw))
    want = x + a.float() @ w.float().t()
    torch.testing.assert_close(xr.cpu(), want, atol=3e-3, rtol=1e-3)
    torch.testing.assert_close(ss.sum(0).cpu(), (want ** 2).sum(1), atol=5e-2, rtol=1e-3)
    torch.testing.assert_close(xw.cpu().float(), (want * nw).to(torch.bfloat16).float(), atol=4e-2, rtol=2e-2)
    # twice in a row on the same stream: the second call adds to what the first left
    ops.skinny_linear(dev(w), act=dev(a), epilogue="resid", resid=xr)
    torch.testing.assert_close(xr.cpu(), want + a.float() @ w.float().t(), atol=6e-3, rtol=1e-3)


@pytest.mark.parametrize("M", [1, 3, 8, 11, 16])
@pytest.mark.parametrize("N,K", [(70, 96), (2048, 2048), (1003, 324), (515, 8192), (6, 4)])
def test_skinny_linear_float32_is_plain_float_arithmetic(ops, M, N, K):
    """The decode product of the 32-bit path: float weights, FMA only.  Against a float64 product
    the error must be that of float32 sums (a product rounded to 19 or 10 bits of mantissa, as the
    tensor cores' reduced modes would give, is a hundred times off), a token's result must not
    depend on what else is in the batch, and `linear` must send decode-sized float products there."""
    torch.manual_seed(30)
    w = torch.randn(N, K)
    a = torch.randn(M, K)
    b = torch.randn(N)
    want = (a.double() @ w.double().t() + b.double())
    got = ops.skinny_linear_f32(dev(w), dev(a), dev(b))
    err = (got.cpu().double() - want).abs().max().item()
    assert err < 3e-7 * K ** 0.5 * max(1.0, want.abs().max().item()) + 1e-6, err
    alone = ops.skinny_linear_f32(dev(w), dev(a[M - 1:]), dev(b))
    assert torch.equal(alone[0], got[M - 1]), "a token's row must not depend on the batch"
    before = ops.launch_count
    via = ops.linear(dev(a), dev(w), dev(b))
    assert ops.launch_count == before + 1 and torch.equal(via, got)


def test_embed_and_residual_add_prepare_the_next_norm(ops):
    torch.manual_seed(22)
    table = torch.randn(50, 72).to(torch.bfloat16)
    toks = torch.tensor([3, 49, 0, 3], dtype=torch.int32)
    nw = 1 + 0.1 * torch.randn(72)
    x, ss, xw = ops.embed(dev(table), dev(toks), None, dev(nw))
    want = table[toks.long()].float()
    torch.testing.assert_close(x.cpu(), want, atol=0, rtol=0)
    torch.testing.assert_close(ss.cpu(), (want ** 2).sum(1)[None], atol=1e-4, rtol=1e-5)
    torch.testing.assert_close(xw.cpu().float(), (want * nw).to(torch.bfloat16).float(), atol=1e-2, rtol=1e-2)
    delta = torch.randn(4, 72).to(torch.bfloat16)
    ss2, xw2 = ops.add_residual_ss(x, dev(delta), dev(nw))
    want2 = want + delta.float()
    torch.testing.assert_close(x.cpu(), want2, atol=1e-6, rtol=1e-6)
    torch.testing.assert_close(ss2.cpu(), (want2 ** 2).sum(1)[None], atol=1e-4, rtol=1e-5)
    torch.testing.assert_close(xw2.cpu().float(), (want2 * nw).to(torch.bfloat16).float(), atol=2e-2, rtol=1e-2)


def test_skinny_shortconv_with_weights_by_tma(ops, tma_weights):
    """The conv epilogue in the TMA form against the form with per-lane copies, state included."""
    torch.manual_seed(27)
    for M, H, K, L, bias in ((8, 2048, 2048, 3, False), (3, 72, 96, 4, True), (5, 200, 160, 2, True)):
        w = (torch.randn(3 * H, K) * 0.05).to(torch.bfloat16)
        x = torch.randn(M, K)
        nw = 1 + 0.1 * torch.randn(K)
        parts = torch.stack([(x[:, i::3] ** 2).sum(1) for i in range(3)]).contiguous()
        xw = (x * nw).to(torch.bfloat16)
        taps, cb, ib = torch.randn(L, H) * 0.5, torch.randn(H) * 0.1, torch.randn(3 * H) * 0.1
        state0 = torch.randn(M + 2, max(L - 1, 1), H).to(torch.bfloat16)
        slots = torch.randperm(M + 2)[:M].to(torch.int32)
        pos = torch.tensor([0, 1, 5, 2, 9, 1, 0, 3][:M], dtype=torch.int32)

        def run():
            st = dev(state0.clone())
            y = ops.skinny_shortconv(dev(w), xw=dev(xw), ss_in=dev(parts), eps=1e-5, in_bias=dev(ib) if bias else None,
                                     taps=dev(taps), conv_bias=dev(cb) if bias else None, state_layer=st if L > 1 else None,
                                     state_slots=dev(slots), positions=dev(pos))
            return y, st

        got = run()
        ops.skinny_use_tma(False)
        want = run()
        ops.skinny_use_tma(True)
        assert torch.equal(got[0], want[0]) and torch.equal(got[1], want[1]), (M, H, K, L)


@pytest.mark.parametrize("M,H,K,L,bias", [(8, 2048, 2048, 3, False), (1, 72, 96, 4, True), (11, 200, 160, 2, True),
                                          (16, 64, 64, 5, False), (3, 40, 32, 1, False), (12, 1280, 128, 3, True)])
def test_skinny_shortconv_is_in_proj_then_the_conv_kernel(ops, M, H, K, L, bias):
    """The decode form of the short-conv mixer in one launch, against the two steps it replaces
    (in_proj rounded to bfloat16, then the conv kernel's plain restatement), over two steps on the
    same slots so that the state it leaves is the state it reads, with one request starting over."""
    torch.manual_seed(31)
    bf = torch.bfloat16
    w_in = (torch.randn(3 * H, K) / math.sqrt(K)).to(bf)
    taps = torch.randn(L, H)
    in_b = torch.randn(3 * H) if bias else None
    cv_b = torch.randn(H) if bias else None
    nw = 1 + 0.1 * torch.randn(K)
    slots_n = M + 2
    state_ref = torch.full((slots_n, max(L - 1, 1), H), 9.0).to(bf)[:, :L - 1]
    state_gpu = dev(state_ref.clone())
    slots = torch.randperm(slots_n)[:M].to(torch.int32)
    pos0 = torch.randint(0, 4, (M,), dtype=torch.int32)
    for step in range(3):
        pos = pos0 + step
        if step == 2:
            pos[0] = 0                                     # a new request in a used slot
        x = torch.randn(M, K) * 2
        xw = (x * nw).to(bf)
        parts = 5
        ss = torch.stack([(x[:, j::parts] ** 2).sum(1) for j in range(parts)])
        inv = torch.rsqrt(ss.sum(0) / K + 1e-5)
        h3 = ((xw.float() @ w_in.float().t()) * inv[:, None]).to(bf)
        ar = torch.arange(M + 1, dtype=torch.int32)
        want = plain_ops.shortconv(h3, in_b, taps, cv_b, state_ref, slots, ar[:M].clone(), ar, pos)
        got = ops.skinny_shortconv(dev(w_in), xw=dev(xw), ss_in=dev(ss), eps=1e-5, in_bias=dev(in_b), taps=dev(taps),
                                   conv_bias=dev(cv_b), state_layer=state_gpu if L > 1 else None,
                                   state_slots=dev(slots), positions=dev(pos))
        torch.testing.assert_close(got.cpu().float(), want.float(), atol=6e-2, rtol=4e-2)
        if L > 1:
            torch.testing.assert_close(state_gpu.cpu().float(), state_ref.float(), atol=6e-2, rtol=4e-2)


@pytest.mark.parametrize("vocab", [1000, 65536, 70001])
def test_sample_truncated_cuts_where_the_host_sampler_cuts(ops, vocab):
    """top-k, min-p and top-p on the device: the survivors are exactly the host sampler's (random
    logits have no ties), the drawn token is one of them, and the draw is keyed by (seed, draw)."""
    import numpy as np
    g = torch.Generator().manual_seed(40)
    cases = [(1.0, 5, 1.0, 0.0), (0.7, 0, 0.9, 0.0), (1.3, 0, 1.0, 0.05), (0.9, 50, 0.8, 0.01), (2.0, 0, 0.5, 0.0),
             (1.0, 1, 1.0, 0.0), (0.5, 0, 1.0, 0.0), (1.0, 3000, 0.999, 0.0), (1.0, 0, 0.02, 0.0)]
    R = len(cases)
    logits = torch.randn(R, vocab, generator=g) * 3
    logits[4, 17] += 9.0                                     # one row with a dominant token
    f = lambda v, dt: torch.tensor(v, dtype=dt).cuda()
    inv_t = f([1.0 / c[0] for c in cases], torch.float32)
    top_k = f([c[1] for c in cases], torch.int32)
    top_p = f([c[2] for c in cases], torch.float32)
    min_p = f([c[3] for c in cases], torch.float32)
    seeds = f(list(range(5, 5 + R)), torch.int64)
    draws = f([0] * R, torch.int64)
    out, tau, cnt = ops.sample_truncated(dev(logits), inv_t, top_k, top_p, min_p, seeds, draws, check=True)
    again = ops.sample_truncated(dev(logits), inv_t, top_k, top_p, min_p, seeds, draws)
    other = ops.sample_truncated(dev(logits), inv_t, top_k, top_p, min_p, seeds, draws + 1)
    assert torch.equal(out, again)
    assert not torch.equal(out[[1, 2, 6]], other[[1, 2, 6]]), "another draw should move at least one wide row"
    for r, (T, k, tp, mp) in enumerate(cases):
        ids, prob, scaled = plain_ops.truncated_survivors(logits[r].numpy(), 1.0 / T, k or None, tp, mp)
        assert int(cnt[r]) == len(ids), (r, int(cnt[r]), len(ids))
        assert int(out[r]) in set(ids.tolist())
        assert abs(float(tau[r]) - float(scaled[ids].min())) < 1e-5 or len(ids) == int((scaled >= float(tau[r])).sum())
    # a negative top_k leaves the row to another kernel
    keep = torch.full((R,), -7, dtype=torch.int32).cuda()
    ops.sample_truncated(dev(logits), inv_t, torch.full_like(top_k, -1), top_p, min_p, seeds, draws, out=keep)
    assert keep.tolist() == [-7] * R


def test_sample_truncated_draws_from_the_renormalised_distribution(ops):
    import numpy as np
    g = torch.Generator().manual_seed(41)
    vocab, N = 300, 20000
    row = torch.randn(1, vocab, generator=g) * 2
    ids, prob, _ = plain_ops.truncated_survivors(row[0].numpy(), 1.0 / 0.8, 12, 0.85, 0.0)
    want = prob / prob.sum()
    f = lambda v, dt: torch.tensor(v, dtype=dt).cuda()
    logits = dev(row).expand(N, vocab)                       # the same row N times, N draws
    out = ops.sample_truncated(logits, f([1.25] * N, torch.float32), f([12] * N, torch.int32), f([0.85] * N, torch.float32),
                               f([0.0] * N, torch.float32), f([9] * N, torch.int64), f(list(range(N)), torch.int64))
    got = np.bincount(out.cpu().numpy(), minlength=vocab) / N
    assert set(np.nonzero(got)[0].tolist()) <= set(ids.tolist())
    sigma = np.sqrt(want * (1 - want) / N)
    assert np.all(np.abs(got[ids] - want) < 5 * sigma + 1e-3), (got[ids], want)


@pytest.mark.parametrize("M", [1, 8, 9, 16])
def test_skinny_linear_long_k_residual_product(ops, M):
    """w2 of the 1.2B model: K = 8192 and no more tiles than SMs, which takes the deeper copy queue."""
    torch.manual_seed(33)
    N, K = 2048, 8192
    w = (torch.randn(N, K) * 0.02).to(torch.bfloat16)
    a = torch.randn(M, K).to(torch.bfloat16)
    x = torch.randn(M, N)
    nw = 1 + 0.1 * torch.randn(N)
    xg = dev(x.clone())
    ss, xw = ops.skinny_linear(dev(w), act=dev(a), epilogue="resid", resid=xg, next_weight=dev(nw))
    want = x + a.float() @ w.float().t()
    torch.testing.assert_close(xg.cpu(), want, atol=2e-2, rtol=1e-3)
    torch.testing.assert_close(ss.sum(0).cpu(), (want ** 2).sum(1), rtol=1e-3, atol=1e-2)
    torch.testing.assert_close(xw.cpu().float(), (want * nw).to(torch.bfloat16).float(), atol=3e-2, rtol=2e-2)


def test_skinny_linear_refuses_what_it_cannot_do(ops):
    w = torch.zeros(64, 80, dtype=torch.bfloat16).cuda()
    with pytest.raises(ops.KernelError, match="multiple of 32"):
        ops.skinny_linear(w, act=torch.zeros(2, 80, dtype=torch.bfloat16).cuda(), epilogue="bf16")
    w = torch.zeros(64, 96, dtype=torch.bfloat16).cuda()
    with pytest.raises(ops.KernelError, match="more than 16"):
        ops.skinny_linear(w, act=torch.zeros(17, 96, dtype=torch.bfloat16).cuda(), epilogue="bf16")
    assert not ops.skinny_applies(17, w) and not ops.skinny_applies(4, w.float()) and ops.skinny_applies(4, w)


# ---- the tcgen05 / TMA product of steps of 17..256 rows -------------------------------------
@pytest.mark.parametrize("M", [17, 32, 64, 100, 256])
@pytest.mark.parametrize("N,K", [(200, 96), (2048, 2048), (1000, 328), (384, 8192)])
def test_linear_tc_plain_products(ops, M, N, K):
    """Tiles that are not full (N no multiple of 128), K that is no multiple of 64, few tiles
    (split over K with the last-arriver sum), token counts that are not a power of two."""
    torch.manual_seed(30)
    w = (torch.randn(N, K) * 0.05).to(torch.bfloat16)
    a = torch.randn(M, K).to(torch.bfloat16)
    b = torch.randn(N)
    want = a.float() @ w.float().t()
    st = torch.zeros(1, dtype=torch.int32).cuda()
    got = ops.linear_tc(dev(w), act=dev(a), epilogue="f32", status=st)
    assert int(st.item()) == 0, "a bounded wait ran out"
    torch.testing.assert_close(got.cpu(), want, atol=3e-3 * math.sqrt(K / 96), rtol=1e-3)
    got = ops.linear_tc(dev(w), act=dev(a), epilogue="bf16", bias=dev(b), status=st)
    torch.testing.assert_close(got.cpu().float(), (want + b).to(torch.bfloat16).float(), atol=3e-2 * math.sqrt(K / 96), rtol=2e-2)
    again = ops.linear_tc(dev(w), act=dev(a), epilogue="bf16", bias=dev(b), status=st)
    assert torch.equal(got, again), "the split-K sum must not depend on arrival order"
    assert int(st.item()) == 0
    # the dispatcher sends up to TC_MAX_ROWS rows here and larger steps to the library's product
    before = ops.launch_count
    got = ops.linear(dev(a), dev(w), None, torch.float32)
    assert ops.launch_count == before + (1 if M <= ops.TC_MAX_ROWS else 0)
    torch.testing.assert_close(got.cpu(), want, atol=3e-3 * math.sqrt(K / 96), rtol=1e-3)


@pytest.mark.parametrize("M", [24, 64, 130])
def test_linear_tc_fusions(ops, M):
    torch.manual_seed(31)
    H, F, eps = 256, 328, 1e-6
    x = torch.randn(M, H) * 2
    nw = 1 + 0.1 * torch.randn(H)
    w13 = (torch.randn(2 * F, H) * 0.1).to(torch.bfloat16)
    w2 = (torch.randn(H, F) * 0.1).to(torch.bfloat16)
    parts = torch.stack([(x[:, i * 64:(i + 1) * 64] ** 2).sum(1) for i in range(4)]).contiguous()
    xw = (x * nw).to(torch.bfloat16)
    st = torch.zeros(1, dtype=torch.int32).cuda()
    s = ops.linear_tc(dev(w13), xw=dev(xw), ss_in=dev(parts), eps=eps, epilogue="swiglu", status=st)
    inv = torch.rsqrt((x ** 2).mean(1, keepdim=True) + eps)
    gu = (xw.float() @ w13.float().t()) * inv
    want_s = (gu[:, :F] / (1 + torch.exp(-gu[:, :F]))) * gu[:, F:]
    torch.testing.assert_close(s.cpu().float(), want_s.to(torch.bfloat16).float(), atol=4e-2, rtol=3e-2)
    s2 = torch.randn(M, F).to(torch.bfloat16)
    bias, nw2 = torch.randn(H), 1 + 0.1 * torch.randn(H)
    xr = dev(x.clone())
    ss, xw2 = ops.linear_tc(dev(w2), act=dev(s2), epilogue="resid", resid=xr, bias=dev(bias), next_weight=dev(nw2), status=st)
    want_x = x + s2.float() @ w2.float().t() + bias
    torch.testing.assert_close(xr.cpu(), want_x, atol=3e-3, rtol=1e-3)
    torch.testing.assert_close(ss.sum(0).cpu(), (want_x ** 2).sum(1), atol=2e-2, rtol=1e-3)
    torch.testing.assert_close(xw2.cpu().float(), (want_x * nw2).to(torch.bfloat16).float(), atol=3e-2, rtol=2e-2)
    lg = ops.linear_tc(dev(w13), xw=dev(xw), ss_in=dev(parts), eps=eps, epilogue="f32", status=st)
    torch.testing.assert_close(lg.cpu(), (xw.float() @ w13.float().t()) * inv, atol=3e-3, rtol=1e-3)
    assert int(st.item()) == 0


# ---- the persistent tcgen05 / TMA product of prompt-sized steps ------------------------------
@pytest.fixture(params=[(256, 2), (128, 2), (256, 1), (128, 1), (0, 0)], ids=["256x2", "128x2", "256x1", "128x1", "planned"])
def prompt_tiles(ops, request):
    """Every tile shape of the kernel (features a tile x blocks a tile), and the kernel's own choice."""
    ops.prompt_force(*request.param)
    yield request.param
    ops.prompt_force(0, 0)


@pytest.mark.parametrize("M", [33, 128, 300, 1031])
@pytest.mark.parametrize("N,K", [(200, 96), (2048, 2048), (1000, 328), (384, 8192)])
def test_prompt_linear_plain_products(ops, prompt_tiles, M, N, K):
    """Tiles that are not full along the features (N no multiple of 128) or the tokens, K that is no
    multiple of 64, fewer tiles than blocks and many tiles a block (the ring of stages and the two
    accumulators wrap around)."""
    torch.manual_seed(32)
    w = (torch.randn(N, K) * 0.05).to(torch.bfloat16)
    a = torch.randn(M, K).to(torch.bfloat16)
    b = torch.randn(N)
    want = a.float() @ w.float().t()
    st = torch.zeros(1, dtype=torch.int32).cuda()
    got = ops.prompt_linear(dev(w), act=dev(a), epilogue="f32", status=st)
    assert int(st.item()) == 0, "a bounded wait ran out"
    torch.testing.assert_close(got.cpu(), want, atol=3e-3 * math.sqrt(K / 96), rtol=1e-3)
    got = ops.prompt_linear(dev(w), act=dev(a), epilogue="bf16", bias=dev(b), status=st)
    torch.testing.assert_close(got.cpu().float(), (want + b).to(torch.bfloat16).float(), atol=3e-2 * math.sqrt(K / 96), rtol=2e-2)
    assert int(st.item()) == 0


@pytest.mark.parametrize("M", [35, 260])
def test_prompt_linear_rows_that_are_not_16_byte_aligned(ops, prompt_tiles, M):
    """Output rows whose pitch is no multiple of 8 elements take the value-by-value ends of the
    epilogues: 100 SwiGLU features, a residual stream and plain outputs of 204 features."""
    torch.manual_seed(34)
    K, F, N = 96, 100, 204
    a = torch.randn(M, K).to(torch.bfloat16)
    w13 = (torch.randn(2 * F, K) * 0.1).to(torch.bfloat16)
    w = (torch.randn(N, K) * 0.1).to(torch.bfloat16)
    st = torch.zeros(1, dtype=torch.int32).cuda()
    gu = a.float() @ w13.float().t()
    want_s = (gu[:, :F] / (1 + torch.exp(-gu[:, :F]))) * gu[:, F:]
    s = ops.prompt_linear(dev(w13), act=dev(a), epilogue="swiglu", status=st)
    torch.testing.assert_close(s.cpu().float(), want_s.to(torch.bfloat16).float(), atol=4e-2, rtol=3e-2)
    y = a.float() @ w.float().t()
    torch.testing.assert_close(ops.prompt_linear(dev(w), act=dev(a), epilogue="f32", status=st).cpu(), y, atol=3e-3, rtol=1e-3)
    torch.testing.assert_close(ops.prompt_linear(dev(w), act=dev(a), epilogue="bf16", status=st).cpu().float(),
                               y.to(torch.bfloat16).float(), atol=3e-2, rtol=2e-2)
    x, nw = torch.randn(M, N), 1 + 0.1 * torch.randn(N)
    xr = dev(x.clone())
    ss, xw = ops.prompt_linear(dev(w), act=dev(a), epilogue="resid", resid=xr, next_weight=dev(nw), status=st)
    torch.testing.assert_close(xr.cpu(), x + y, atol=3e-3, rtol=1e-3)
    torch.testing.assert_close(ss.sum(0).cpu(), ((x + y) ** 2).sum(1), atol=2e-2, rtol=1e-3)
    torch.testing.assert_close(xw.cpu().float(), ((x + y) * nw).to(torch.bfloat16).float(), atol=3e-2, rtol=2e-2)
    assert int(st.item()) == 0


@pytest.mark.parametrize("M", [40, 130, 700])
def test_prompt_linear_fusions(ops, prompt_tiles, M):
    torch.manual_seed(33)
    H, F, eps = 264, 328, 1e-6
    x = torch.randn(M, H) * 2
    nw = 1 + 0.1 * torch.randn(H)
    w13 = (torch.randn(2 * F, H) * 0.1).to(torch.bfloat16)
    w2 = (torch.randn(H, F) * 0.1).to(torch.bfloat16)
    parts = torch.stack([(x[:, i * 66:(i + 1) * 66] ** 2).sum(1) for i in range(4)]).contiguous()
    xw = (x * nw).to(torch.bfloat16)
    st = torch.zeros(1, dtype=torch.int32).cuda()
    s = ops.prompt_linear(dev(w13), xw=dev(xw), ss_in=dev(parts), eps=eps, epilogue="swiglu", status=st)
    inv = torch.rsqrt((x ** 2).mean(1, keepdim=True) + eps)
    gu = (xw.float() @ w13.float().t()) * inv
    want_s = (gu[:, :F] / (1 + torch.exp(-gu[:, :F]))) * gu[:, F:]
    torch.testing.assert_close(s.cpu().float(), want_s.to(torch.bfloat16).float(), atol=4e-2, rtol=3e-2)
    s2 = torch.randn(M, F).to(torch.bfloat16)
    bias, nw2 = torch.randn(H), 1 + 0.1 * torch.randn(H)
    xr = dev(x.clone())
    ss, xw2 = ops.prompt_linear(dev(w2), act=dev(s2), epilogue="resid", resid=xr, bias=dev(bias), next_weight=dev(nw2), status=st)
    want_x = x + s2.float() @ w2.float().t() + bias
    torch.testing.assert_close(xr.cpu(), want_x, atol=3e-3, rtol=1e-3)
    torch.testing.assert_close(ss.sum(0).cpu(), (want_x ** 2).sum(1), atol=2e-2, rtol=1e-3)
    torch.testing.assert_close(xw2.cpu().float(), (want_x * nw2).to(torch.bfloat16).float(), atol=3e-2, rtol=2e-2)
    lg = ops.prompt_linear(dev(w13), xw=dev(xw), ss_in=dev(parts), eps=eps, epilogue="f32", status=st)
    torch.testing.assert_close(lg.cpu(), (xw.float() @ w13.float().t()) * inv, atol=3e-3, rtol=1e-3)
    assert int(st.item()) == 0
