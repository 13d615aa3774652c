"""The attention entry point that allocates nothing (vapi_paged_attention_noalloc), called the
way a C program would call it: through the exported symbol, with raw device addresses.

Who needs it: code that must run attention but may not allocate device memory when it does: a
latency-critical loop that must stay out of the allocator, a program with a fixed memory budget,
a plug-in whose host owns all device memory.  The ordinary entry point asks such a caller for two
scratch buffers; this one keeps its scratch in a fixed 8 MiB array inside the library.

The test runs the same inputs through both entry points, twice in a row with different data, the
larger call first (the built-in array keeps the first call's leftovers, which must not show in
the second), in the forms that really go through the array (bfloat16 on the one-warp flash kernel
and with more slices than the decode kernel combines by itself; float32 on the general kernel),
compares with the plain restatement of attention as well, and checks the refusal of a call that
would not fit the array.  This file is collected last on purpose."""
import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _case(seed, dtype, n_seqs=5, nh=8, nkv=2, d=64, page=64, longest=600):
    g = torch.Generator().manual_seed(seed)
    lens = [int(x) for x in torch.randint(1, longest, (n_seqs,), generator=g)]
    need = [-(-k // page) for k in lens]
    pages = sum(need) + 2
    perm = torch.randperm(pages, generator=g).tolist()
    table = torch.zeros((n_seqs, max(need)), dtype=torch.int32)
    it = iter(perm)
    for s in range(n_seqs):
        for j in range(need[s]):
            table[s, j] = next(it)
    cache = torch.randn(pages, 2, nkv, page, d, generator=g).to(dtype)
    q = torch.randn(n_seqs, nh * d, generator=g).to(dtype)                 # one decode token per sequence
    cu = torch.arange(n_seqs + 1, dtype=torch.int32)
    kl = torch.tensor(lens, dtype=torch.int32)
    return dict(q=q.cuda(), cache=cache.cuda(), table=table.cuda(), cu=cu.cuda(), kl=kl.cuda(), n=n_seqs,
                max_k=max(lens), nh=nh, nkv=nkv, d=d)


def _noalloc(lib, c, splits, impl=0):
    out = torch.empty((c["n"], c["nh"] * c["d"]), dtype=c["q"].dtype, device="cuda")
    dt = 0 if c["q"].dtype == torch.float32 else 1
    P = ctypes.c_void_p
    rc = lib.vapi_paged_attention_noalloc(
        P(c["q"].data_ptr()), ctypes.c_longlong(c["nh"] * c["d"]), P(c["cache"].data_ptr()), dt,
        P(c["table"].data_ptr()), c["table"].stride(0), P(c["cu"].data_ptr()), P(c["kl"].data_ptr()),
        P(out.data_ptr()), c["n"], c["n"], 1, c["nh"], c["nkv"], c["d"], c["cache"].shape[3], c["cache"].shape[0],
        ctypes.c_float(1.0 / math.sqrt(c["d"])), 0, splits, impl, None,
        P(torch.cuda.current_stream().cuda_stream))
    return rc, out


_IMPL = {"auto": 0, "general": 1, "tensor_core": 2, "decode": 4}


# (dtype, kernel, slices): every case but the first writes its partial results to the built-in array
# and reads them back in the combine kernel; in the first the decode kernel's slices combine among
# themselves as a thread-block cluster, and the array stays untouched
@pytest.mark.parametrize("dtype,impl,splits", [(torch.bfloat16, "auto", 4), (torch.bfloat16, "tensor_core", 4),
                                               (torch.bfloat16, "auto", 32), (torch.float32, "auto", 4),
                                               (torch.float32, "general", 7)])
def test_attention_without_allocation_matches_the_ordinary_entry_point(dtype, impl, splits):
    import plain_ops
    from vapi_b200 import ops
    lib = ops._lib("attention")
    assert hasattr(lib, "vapi_paged_attention_noalloc")
    tol = dict(atol=3e-2, rtol=3e-2) if dtype == torch.bfloat16 else dict(atol=3e-5, rtol=3e-5)
    if dtype == torch.bfloat16 and impl == "auto":
        assert ops.decode_attention_combines(5, 2, splits) == (splits == 4)
    # two calls in a row share the built-in array; the first is the larger one (more sequences and
    # longer contexts), so the second runs over what the first left behind
    for call, (seed, n_seqs, longest) in enumerate(((40, 9, 3000), (41, 5, 600))):
        c = _case(seed, dtype, n_seqs=n_seqs, longest=longest)
        scale = 1.0 / math.sqrt(c["d"])
        want = ops.paged_attention(c["q"], c["nh"] * c["d"], c["cache"], c["table"], c["cu"], c["kl"], c["n"], c["n"],
                                   1, c["max_k"], c["nh"], c["nkv"], c["d"], scale, 0, splits, None, impl)
        torch.cuda.synchronize()
        before = torch.cuda.memory_allocated()
        rc, got = _noalloc(lib, c, splits=splits, impl=_IMPL[impl])
        torch.cuda.synchronize()
        assert rc == 0, lib.vapi_last_error().decode()
        grown = torch.cuda.memory_allocated() - before
        assert grown <= got.numel() * got.element_size() + 1024, "only the output was allocated (by the test itself)"
        torch.testing.assert_close(got.float().cpu(), want.float().cpu(), **tol)
        assert torch.isfinite(got.float()).all(), f"call {call}"
        plain = plain_ops.paged_attention(c["q"].cpu(), c["nh"] * c["d"], c["cache"].cpu(), c["table"].cpu(), c["cu"].cpu(),
                                          c["kl"].cpu(), c["n"], c["n"], 1, c["max_k"], c["nh"], c["nkv"], c["d"], scale, 0)
        torch.testing.assert_close(got.float().cpu(), plain.float(), **tol)


def test_attention_without_allocation_refuses_what_does_not_fit():
    from vapi_b200 import ops
    lib = ops._lib("attention")
    c = _case(42, torch.bfloat16, n_seqs=4, nh=8, nkv=2, d=64)
    # pretend a step of 40,000 tokens: 40000 * 8 * 4 * 66 floats is far beyond the 2 Mi floats of the array
    P = ctypes.c_void_p
    rc = lib.vapi_paged_attention_noalloc(
        P(c["q"].data_ptr()), ctypes.c_longlong(512), P(c["cache"].data_ptr()), 1, P(c["table"].data_ptr()),
        c["table"].stride(0), P(c["cu"].data_ptr()), P(c["kl"].data_ptr()), P(c["q"].data_ptr()), 40000, 4, 1, 8, 2, 64, 64,
        c["cache"].shape[0], ctypes.c_float(0.125), 0, 4, 0, None, P(torch.cuda.current_stream().cuda_stream))
    assert rc != 0
    msg = lib.vapi_last_error().decode()
    assert "floats" in msg and "built-in array" in msg
    rc, got = _noalloc(lib, c, splits=1)                   # one split: the array is not needed at all
    assert rc == 0
