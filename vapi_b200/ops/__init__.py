"""The kernels of the package as Python functions over torch tensors.

Every function here launches hand-written CUDA for sm_100a from ``vapi_b200/csrc`` on the
current torch stream (``linear`` alone is a library matrix product, as in the reference,
which calls cuBLAS through candle for every projection).  There is no CPU path: a tensor
that is not on a CUDA device is refused, and a missing or unbuildable extension raises.

Activation tensors are float32 (the true 32-bit path) or bfloat16 (the serving path); the
residual stream is always float32; small parameter vectors (norm weights, biases, conv
taps) are always float32.
"""
from __future__ import annotations

import ctypes
import os
import threading
from typing import Dict, Optional, Tuple

import torch

from ..csrc import build as _build

F32, BF16 = 0, 1
_DT = {torch.float32: F32, torch.bfloat16: BF16}

_libs: Dict[str, ctypes.CDLL] = {}
_lock = threading.Lock()
loaded_libraries: Dict[str, str] = {}


class KernelError(RuntimeError):
    pass


def _lib(name: str) -> ctypes.CDLL:
    lib = _libs.get(name)
    if lib is not None:
        return lib
    with _lock:
        lib = _libs.get(name)
        if lib is None:
            path = _build.build(name)
            lib = ctypes.CDLL(path)
            lib.vapi_last_error.restype = ctypes.c_char_p
            _libs[name] = lib
            loaded_libraries[name] = path
            if _trace is not None:
                _trace_attach(name, lib)
    return lib


# ---- time stamps from inside captured graphs (a build with VAPI_NVCC_FLAGS=-DVAPI_TRACE) ----------
_trace: Optional[Tuple[torch.Tensor, torch.Tensor, Dict[str, int]]] = None


def _trace_attach(name: str, lib: ctypes.CDLL) -> None:
    buf, count, ids = _trace
    if not hasattr(lib, "vapi_trace_set"):
        raise KernelError(f"lib{name} was built without -DVAPI_TRACE (set VAPI_NVCC_FLAGS before the first import)")
    ids.setdefault(name, len(ids))
    rc = lib.vapi_trace_set(ctypes.c_void_p(buf.data_ptr()), ctypes.c_void_p(count.data_ptr()), buf.numel() // 2, ids[name])
    if rc != 0:
        raise KernelError(lib.vapi_last_error().decode(errors="replace"))


def trace_start(capacity: int = 1 << 16, device: str = "cuda") -> None:
    """Start collecting the kernels' own time stamps (first block's start, return of its dependency
    wait): every library loaded from now on, and those loaded already, writes into one buffer."""
    global _trace
    buf = torch.zeros(2 * capacity, dtype=torch.int64, device=device)
    count = torch.zeros(1, dtype=torch.int32, device=device)
    _trace = (buf, count, {})
    for name, lib in list(_libs.items()):
        if name != "host":
            _trace_attach(name, lib)


def trace_read() -> list:
    """The stamps so far, in time order: dicts with ``ns``, ``kind`` ("start" | "released"), ``library``,
    ``threads`` and ``blocks`` of the kernel that wrote them."""
    if _trace is None:
        raise KernelError("trace_start() was not called")
    buf, count, ids = _trace
    torch.cuda.synchronize()
    n = min(int(count.item()), buf.numel() // 2)
    raw = buf[:2 * n].cpu().tolist()
    names = {v: k for k, v in ids.items()}
    out = []
    for i in range(n):
        t, meta = raw[2 * i], raw[2 * i + 1]
        out.append({"ns": t, "kind": "start" if (meta & 15) == 0 else "released", "library": names.get((meta >> 4) & 15, "?"),
                    "threads": (meta >> 8) & 0xffff, "blocks": meta >> 24})
    out.sort(key=lambda e: e["ns"])
    return out


#: how many of this package's own kernels have been launched (library products not counted)
launch_count = 0


def _check(lib: ctypes.CDLL, rc: int, launches: int = 1) -> None:
    global launch_count
    if rc != 0:
        raise KernelError(lib.vapi_last_error().decode(errors="replace") + f" (code {rc})")
    launch_count += launches


def _dt(t: torch.Tensor) -> int:
    try:
        return _DT[t.dtype]
    except KeyError:
        raise KernelError(f"dtype {t.dtype} is not supported by the kernels (float32, bfloat16)")


def _cuda(*ts: Optional[torch.Tensor]) -> None:
    for t in ts:
        if t is not None and not t.is_cuda:
            raise KernelError("vapi_b200 kernels run on CUDA tensors only; there is no CPU fallback")


def _p(t: Optional[torch.Tensor]) -> ctypes.c_void_p:
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


_held_stream = threading.local()


def _stream() -> ctypes.c_void_p:
    h = getattr(_held_stream, "handle", None)
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream if h is None else h)


class one_stream:
    """Within the block every kernel of this module launches on the stream that is current at its
    entry, looked up once instead of once per kernel (a step launches a few hundred).  The caller
    must not switch streams inside the block."""

    def __enter__(self):
        self.before = getattr(_held_stream, "handle", None)
        _held_stream.handle = torch.cuda.current_stream().cuda_stream if torch.cuda.is_available() else None
        return self

    def __exit__(self, *exc):
        _held_stream.handle = self.before
        return False


def _contig(t: torch.Tensor, what: str) -> None:
    if not t.is_contiguous():
        raise KernelError(f"{what} must be contiguous")


def _i32(t: Optional[torch.Tensor], what: str) -> None:
    if t is not None and t.dtype != torch.int32:
        raise KernelError(f"{what} must be int32")


def _f32(t: Optional[torch.Tensor], what: str) -> None:
    if t is not None and (t.dtype != torch.float32 or not t.is_contiguous()):
        raise KernelError(f"{what} must be contiguous float32")


_sm_counts: Dict[int, int] = {}


def sm_count() -> int:
    """Multiprocessors of the current CUDA device, asked of the device (once per device)."""
    if not torch.cuda.is_available():
        raise KernelError("vapi_b200 kernels need a CUDA device; there is no CPU fallback")
    dev = torch.cuda.current_device()
    n = _sm_counts.get(dev)
    if n is None:
        n = _sm_counts[dev] = int(torch.cuda.get_device_properties(dev).multi_processor_count)
    return n


# ---------------------------------------------------------------------------------------
def embed(table: torch.Tensor, tokens: torch.Tensor, status: Optional[torch.Tensor] = None,
          next_weight: Optional[torch.Tensor] = None):
    """Rows of ``table`` [V, H] for ``tokens`` [n] as the float32 residual stream [n, H].

    With ``next_weight`` (the weight of the norm that will read the stream) the call also
    returns what a deferred norm needs: the sums of squares of the rows, [1, n], and
    bfloat16(row * next_weight), [n, H]: ``(x, ss, xw)``."""
    _cuda(table, tokens, next_weight)
    _contig(table, "embedding table")
    _i32(tokens, "tokens")
    _f32(next_weight, "norm weight")
    n, (vocab, hidden) = tokens.numel(), table.shape
    out = torch.empty((n, hidden), dtype=torch.float32, device=table.device)
    ss = xw = None
    if next_weight is not None:
        ss = torch.empty((1, n), dtype=torch.float32, device=table.device)
        xw = torch.empty((n, hidden), dtype=torch.bfloat16, device=table.device)
    lib = _lib("elementwise")
    _check(lib, lib.vapi_embed(_p(table), _dt(table), _p(tokens), _p(out), _p(ss), _p(next_weight), _p(xw), n,
                               hidden, vocab, _p(status), _stream()))
    return (out, ss, xw) if next_weight is not None else out


def add_residual_ss(x: torch.Tensor, delta: torch.Tensor, next_weight: torch.Tensor):
    """``x += delta`` on the float32 stream; returns ``(ss, xw)`` for the norm that follows:
    the sums of squares of the new rows, [1, n], and bfloat16(new row * next_weight)."""
    _cuda(x, delta, next_weight)
    _f32(x, "residual stream")
    _f32(next_weight, "norm weight")
    _contig(delta, "delta")
    n, hidden = x.shape
    ss = torch.empty((1, n), dtype=torch.float32, device=x.device)
    xw = torch.empty((n, hidden), dtype=torch.bfloat16, device=x.device)
    lib = _lib("elementwise")
    _check(lib, lib.vapi_add_residual_ss(_p(x), _p(delta), _dt(delta), _p(ss), _p(next_weight), _p(xw), n, hidden,
                                         _stream()))
    return ss, xw


def resolve_tokens(tokens: torch.Tensor, src: torch.Tensor, prev: torch.Tensor,
                   status: Optional[torch.Tensor] = None) -> None:
    """In place: ``tokens[i] = prev[src[i]]`` wherever ``src[i] >= 0`` (tokens that the step before
    sampled and the host has not read yet)."""
    _cuda(tokens, src, prev)
    for t, w in ((tokens, "tokens"), (src, "token sources"), (prev, "sampled tokens")):
        if t.dtype != torch.int32 or not t.is_contiguous():
            raise KernelError(f"{w} must be contiguous int32")
    lib = _lib("elementwise")
    _check(lib, lib.vapi_resolve_tokens(_p(tokens), _p(src), _p(prev), tokens.numel(), prev.numel(), _p(status),
                                        _stream()))


def add_rmsnorm(x: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, eps: float,
                out_dtype: torch.dtype, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``x += delta`` (when given) and ``out = rmsnorm(x) * weight``; x is the float32 stream.

    With ``rows`` the output has one row per entry of ``rows`` and ``x`` is left untouched
    (the sum is formed on the fly): that is the form the final norm uses for the rows whose
    logits are wanted.
    """
    _cuda(x, delta, weight, rows)
    _f32(x, "residual stream")
    _f32(weight, "norm weight")
    _i32(rows, "rows")
    hidden = x.shape[-1]
    if weight.numel() != hidden:
        raise KernelError(f"norm weight has {weight.numel()} elements for rows of {hidden}")
    if delta is not None:
        _contig(delta, "delta")
        if delta.shape != x.shape or delta.dtype != out_dtype:
            raise KernelError("delta must have the stream's shape and the activation dtype")
    n_out = rows.numel() if rows is not None else x.shape[0]
    out = torch.empty((n_out, hidden), dtype=out_dtype, device=x.device)
    lib = _lib("elementwise")
    _check(lib, lib.vapi_add_rmsnorm(_p(x), _p(delta), _p(weight), ctypes.c_float(eps), _p(rows), _p(out),
                                     _dt(out), n_out, hidden, _stream()))
    return out


def add_residual(x: torch.Tensor, delta: torch.Tensor) -> None:
    """``x += delta`` on the float32 stream."""
    _cuda(x, delta)
    _f32(x, "residual stream")
    _contig(delta, "delta")
    lib = _lib("elementwise")
    _check(lib, lib.vapi_add_residual(_p(x), _p(delta), _dt(delta), ctypes.c_longlong(x.numel()), _stream()))


def swiglu(g: torch.Tensor) -> torch.Tensor:
    """``silu(g[:, :F]) * g[:, F:]`` for a stacked gate/up product [n, 2F]."""
    _cuda(g)
    _contig(g, "gate/up product")
    rows, two_f = g.shape
    if two_f % 2:
        raise KernelError("swiglu needs an even number of columns")
    out = torch.empty((rows, two_f // 2), dtype=g.dtype, device=g.device)
    lib = _lib("elementwise")
    _check(lib, lib.vapi_swiglu(_p(g), _p(out), _dt(g), rows, two_f // 2, _stream()))
    return out


SKINNY_MAX_ROWS = int(os.environ.get("VAPI_SKINNY_MAX_ROWS", "16"))
#: set False to send every product to the library (for comparisons)
use_skinny = os.environ.get("VAPI_SKINNY", "1") != "0"

_PRO = {"act": 0, "norm": 1}
_EPI = {"bf16": 0, "swiglu": 1, "resid": 2, "f32": 3}


def skinny_applies(rows: int, weight: torch.Tensor) -> bool:
    """Whether the weight-streaming kernel takes this product: bfloat16 weight, at most 16
    rows, inner size a multiple of 32."""
    return (use_skinny and weight.is_cuda and weight.dtype == torch.bfloat16 and 0 < rows <= SKINNY_MAX_ROWS
            and weight.dim() == 2 and weight.shape[1] % 32 == 0 and weight.is_contiguous())


def skinny_use_tma(on: bool) -> bool:
    """Choose the form of the decode product whose weight stream is moved by TMA into mbarrier
    rings (steps of at most 8 tokens, inner size up to 2048) instead of per-lane asynchronous
    copies; returns what was chosen before.  ``VAPI_GV_TMA=1`` chooses it from the start."""
    return bool(_lib("gemv").vapi_skinny_linear_use_tma(1 if on else 0))


def skinny_blocks(n_out: int, epilogue: str, rows_per_block: int = 16) -> int:
    if epilogue == "swiglu":
        return (n_out // 2 + 7) // 8
    return -(-n_out // rows_per_block)


def skinny_linear(weight: torch.Tensor, *, act: Optional[torch.Tensor] = None,
                  xw: Optional[torch.Tensor] = None, ss_in: Optional[torch.Tensor] = None, eps: float = 0.0,
                  epilogue: str = "bf16", bias: Optional[torch.Tensor] = None,
                  resid: Optional[torch.Tensor] = None, next_weight: Optional[torch.Tensor] = None,
                  rows_per_block: Optional[int] = None):
    """The weight-streaming product for decode steps (at most 16 rows), with its fusions.

    Token operand: ``act`` [M, K] bfloat16; or the residual stream seen through an RMSNorm not
    applied yet: ``xw`` [M, K] = bfloat16(stream * norm weight) with the partial sums of squares
    ``ss_in`` [parts, M] of the stream's rows (both left by whoever wrote the stream last) and the
    norm's ``eps``.  ``epilogue``: "bf16" -> [M, N] bfloat16; "f32" -> [M, N] float32; "swiglu" ->
    [M, N/2] bfloat16 = silu(first half) * second half; "resid" -> adds into ``resid`` [M, N]
    float32 in place and returns ``(ss, xw)`` of the new stream for the norm whose weight is
    ``next_weight`` (``(None, None)`` without it).
    """
    _cuda(weight, act, xw, ss_in, bias, resid, next_weight)
    N, K = weight.shape
    pro = "act" if act is not None else "norm"
    src = act if act is not None else xw
    if src is None:
        raise KernelError("skinny_linear needs a token operand (act or xw)")
    M = src.shape[0]
    if weight.dtype != torch.bfloat16 or not weight.is_contiguous():
        raise KernelError("skinny_linear needs a contiguous bfloat16 weight")
    if src.shape[1] != K or not src.is_contiguous() or src.dtype != torch.bfloat16:
        raise KernelError(f"skinny_linear: token operand {tuple(src.shape)} / {src.dtype} does not fit a weight of {N}x{K}")
    if pro == "norm":
        _f32(ss_in, "partial sums")
        if ss_in is None or ss_in.dim() != 2 or ss_in.shape[1] != M:
            raise KernelError("partial sums must be [parts, M]")
    _f32(bias, "bias")
    _f32(next_weight, "norm weight")
    rpb = rows_per_block or 16
    out_bf16 = out_f32 = sso = xwo = None
    out_stride = N
    if epilogue == "bf16":
        out_bf16 = torch.empty((M, N), dtype=torch.bfloat16, device=weight.device)
    elif epilogue == "f32":
        out_f32 = torch.empty((M, N), dtype=torch.float32, device=weight.device)
    elif epilogue == "swiglu":
        out_stride = N // 2
        out_bf16 = torch.empty((M, N // 2), dtype=torch.bfloat16, device=weight.device)
    elif epilogue == "resid":
        _f32(resid, "residual stream")
        if resid is None or tuple(resid.shape) != (M, N):
            raise KernelError("the residual stream must be [M, N]")
        if next_weight is not None:
            sso = torch.empty((skinny_blocks(N, epilogue, rpb), M), dtype=torch.float32, device=weight.device)
            xwo = torch.empty((M, N), dtype=torch.bfloat16, device=weight.device)
    else:
        raise KernelError(f"unknown epilogue {epilogue}")
    lib = _lib("gemv")
    _check(lib, lib.vapi_skinny_linear(
        _p(weight), N, K, M, _PRO[pro], _p(act), _p(xw), _p(ss_in), 0 if ss_in is None else ss_in.shape[0],
        ctypes.c_float(eps), _EPI[epilogue], _p(out_bf16), _p(out_f32), ctypes.c_longlong(out_stride), _p(bias),
        _p(resid), _p(sso), _p(next_weight), _p(xwo), rpb, _stream()))
    if epilogue == "resid":
        return sso, xwo
    return out_bf16 if out_bf16 is not None else out_f32


#: Steps of up to this many rows go to the tcgen05 product with its fused epilogues.  The kernel
#: itself takes up to 256 rows, but it has one tile per block and pays its fixed costs (cluster
#: reduction, epilogue) per launch: measured in the captured decode step of LFM2-1.2B sizes it
#: beats the library's product plus separate norm / SwiGLU / add kernels at 32 rows (1.26 vs 1.33
#: ms), loses narrowly at 64 (1.71 vs 1.68 ms) and clearly beyond (2-7x slower at 256 rows).
TC_MAX_ROWS = int(os.environ.get("VAPI_TC_MAX_ROWS", "32"))
#: set False to keep products of 17..TC_MAX_ROWS rows on the library
use_tc = os.environ.get("VAPI_TC", "1") != "0"


def skinny_shortconv_applies(rows: int, w_in: torch.Tensor, kernel: int, state_layer: Optional[torch.Tensor]) -> bool:
    """Whether :func:`skinny_shortconv` takes a decode step of ``rows`` single-token sequences."""
    return (skinny_applies(rows, w_in) and 1 <= kernel <= 8 and w_in.shape[0] % 3 == 0
            and (kernel == 1 or (state_layer is not None and state_layer.dtype == torch.bfloat16)))


def skinny_shortconv(w_in: torch.Tensor, *, xw: torch.Tensor, ss_in: torch.Tensor, eps: float,
                     in_bias: Optional[torch.Tensor], taps: torch.Tensor, conv_bias: Optional[torch.Tensor],
                     state_layer: Optional[torch.Tensor], state_slots: torch.Tensor, positions: torch.Tensor,
                     status: Optional[torch.Tensor] = None) -> torch.Tensor:
    """The short-conv mixer up to its out_proj for a decode step, in one launch: in_proj on the
    stream seen through a deferred norm (``xw``, ``ss_in``, ``eps`` as for :func:`skinny_linear`),
    gate, taps over each request's state, ``C * conv``, state update.  Every one of the M <= 16
    tokens must be a sequence of its own: token m uses ``state_slots[m]`` and ``positions[m]``.
    Returns y [M, H] bfloat16."""
    _cuda(w_in, xw, ss_in, in_bias, taps, conv_bias, state_layer, state_slots, positions)
    H3, K = w_in.shape
    H, M, L = H3 // 3, xw.shape[0], taps.shape[0]
    if w_in.dtype != torch.bfloat16 or not w_in.is_contiguous() or H3 != 3 * H:
        raise KernelError("skinny_shortconv needs a contiguous bfloat16 in_proj weight of 3H rows")
    if xw.dtype != torch.bfloat16 or tuple(xw.shape) != (M, K) or not xw.is_contiguous():
        raise KernelError("skinny_shortconv: the weighted stream must be [M, K] bfloat16")
    _f32(ss_in, "partial sums")
    if ss_in.dim() != 2 or ss_in.shape[1] != M:
        raise KernelError("partial sums must be [parts, M]")
    for t, w in ((in_bias, "in_proj bias"), (taps, "conv taps"), (conv_bias, "conv bias")):
        _f32(t, w)
    if tuple(taps.shape) != (L, H):
        raise KernelError("taps must be [L, H]")
    _i32(state_slots, "state slots")
    _i32(positions, "positions")
    if state_slots.numel() < M or positions.numel() < M:
        raise KernelError("skinny_shortconv: one state slot and one position per token are needed")
    slot_stride = num_slots = 0
    if L > 1:
        if state_layer is None or state_layer.dtype != torch.bfloat16 or tuple(state_layer.shape[1:]) != (L - 1, H):
            raise KernelError(f"state must be [slots, {L - 1}, {H}] bfloat16")
        if state_layer.stride(2) != 1 or state_layer.stride(1) != H:
            raise KernelError("state rows must be contiguous")
        slot_stride, num_slots = state_layer.stride(0), state_layer.shape[0]
    out = torch.empty((M, H), dtype=torch.bfloat16, device=w_in.device)
    lib = _lib("gemv")
    _check(lib, lib.vapi_skinny_linear_conv(
        _p(w_in), H, K, M, _p(xw), _p(ss_in), ss_in.shape[0], ctypes.c_float(eps), _p(in_bias), _p(taps), _p(conv_bias),
        L, _p(state_layer if L > 1 else None), ctypes.c_longlong(slot_stride), num_slots, _p(state_slots),
        _p(positions), _p(out), _p(status), _stream()))
    return out


def tc_applies(rows: int, weight: torch.Tensor) -> bool:
    """Whether the tcgen05 kernel takes this product: bfloat16 weight, 17..TC_MAX_ROWS rows, inner size
    a multiple of 8 (16-byte rows for TMA)."""
    return (use_tc and weight.is_cuda and weight.dtype == torch.bfloat16 and SKINNY_MAX_ROWS < rows <= TC_MAX_ROWS
            and weight.dim() == 2 and weight.shape[1] % 8 == 0 and weight.is_contiguous())


def _tc_plan(N: int, K: int, M: int, epi: int):
    lib = _lib("linear_tc")
    t, s, b = ctypes.c_int(), ctypes.c_int(), ctypes.c_int()
    lib.vapi_linear_tc_plan(N, K, M, epi, ctypes.byref(t), ctypes.byref(s), ctypes.byref(b))
    return t.value, s.value, b.value


def _fused_product(which: str, weight: torch.Tensor, act, xw, ss_in, eps: float, epilogue: str, bias, resid,
                   next_weight, status):
    """Operand checks, outputs and the call shared by :func:`linear_tc` and :func:`prompt_linear`."""
    _cuda(weight, act, xw, ss_in, bias, resid, next_weight)
    N, K = weight.shape
    pro = "act" if act is not None else "norm"
    src = act if act is not None else xw
    if src is None:
        raise KernelError(f"{which} needs a token operand (act or xw)")
    M = src.shape[0]
    if weight.dtype != torch.bfloat16 or not weight.is_contiguous():
        raise KernelError(f"{which} needs a contiguous bfloat16 weight")
    if src.shape[1] != K or not src.is_contiguous() or src.dtype != torch.bfloat16:
        raise KernelError(f"{which}: token operand {tuple(src.shape)} / {src.dtype} does not fit a weight of {N}x{K}")
    if pro == "norm":
        _f32(ss_in, "partial sums")
        if ss_in is None or ss_in.dim() != 2 or ss_in.shape[1] != M:
            raise KernelError("partial sums must be [parts, M]")
    _f32(bias, "bias")
    _f32(next_weight, "norm weight")
    if epilogue not in _EPI:
        raise KernelError(f"unknown epilogue {epilogue}")
    lib = _lib(which)
    if which == "linear_tc":
        parts = _tc_plan(N, K, M, _EPI[epilogue])[0]
        fn = lib.vapi_linear_tc
    else:
        parts = _prompt_plan(N, K, M, _EPI[epilogue])[2]
        fn = lib.vapi_prompt_linear
    out_bf16 = out_f32 = sso = xwo = None
    out_stride = N
    if epilogue == "bf16":
        out_bf16 = torch.empty((M, N), dtype=torch.bfloat16, device=weight.device)
    elif epilogue == "f32":
        out_f32 = torch.empty((M, N), dtype=torch.float32, device=weight.device)
    elif epilogue == "swiglu":
        out_stride = N // 2
        out_bf16 = torch.empty((M, N // 2), dtype=torch.bfloat16, device=weight.device)
    else:
        _f32(resid, "residual stream")
        if resid is None or tuple(resid.shape) != (M, N) or not resid.is_contiguous():
            raise KernelError("the residual stream must be a contiguous [M, N]")
        if next_weight is not None:
            sso = torch.empty((parts, M), dtype=torch.float32, device=weight.device)
            xwo = torch.empty((M, N), dtype=torch.bfloat16, device=weight.device)
    _check(lib, fn(
        _p(weight), N, K, M, _PRO[pro], _p(src), _p(ss_in), 0 if ss_in is None else ss_in.shape[0], ctypes.c_float(eps),
        _EPI[epilogue], _p(out_bf16), _p(out_f32), ctypes.c_longlong(out_stride), _p(bias), _p(resid), _p(sso),
        _p(next_weight), _p(xwo), _p(status), _stream()))
    if epilogue == "resid":
        return sso, xwo
    return out_bf16 if out_bf16 is not None else out_f32


def linear_tc(weight: torch.Tensor, *, act: Optional[torch.Tensor] = None, xw: Optional[torch.Tensor] = None,
              ss_in: Optional[torch.Tensor] = None, eps: float = 0.0, epilogue: str = "bf16",
              bias: Optional[torch.Tensor] = None, resid: Optional[torch.Tensor] = None,
              next_weight: Optional[torch.Tensor] = None, status: Optional[torch.Tensor] = None):
    """The tcgen05 / TMA product for 17..256 rows; same operands, epilogues and results as
    :func:`skinny_linear`."""
    return _fused_product("linear_tc", weight, act, xw, ss_in, eps, epilogue, bias, resid, next_weight, status)


#: steps of more rows than TC_MAX_ROWS go to the persistent tcgen05 product of csrc/linear_prompt.cu
#: (with its fused prologue and epilogues) from this many rows on; 0 keeps them on the library's
#: product with separate norm / SwiGLU / add kernels
PROMPT_MIN_ROWS = int(os.environ.get("VAPI_PROMPT_MIN_ROWS", "0"))


def prompt_applies(rows: int, weight: torch.Tensor) -> bool:
    """Whether the persistent tcgen05 product takes this product: bfloat16 weight, at least
    PROMPT_MIN_ROWS rows, inner size a multiple of 8 (16-byte rows for TMA)."""
    return (PROMPT_MIN_ROWS > 0 and rows >= PROMPT_MIN_ROWS and rows > TC_MAX_ROWS and weight.is_cuda
            and weight.dtype == torch.bfloat16 and weight.dim() == 2 and weight.shape[1] % 8 == 0
            and weight.shape[0] % 8 == 0 and weight.is_contiguous())


def _prompt_plan(N: int, K: int, M: int, epi: int):
    lib = _lib("linear_prompt")
    b, pr, parts = ctypes.c_int(), ctypes.c_int(), ctypes.c_int()
    lib.vapi_prompt_linear_plan(N, K, M, epi, ctypes.byref(b), ctypes.byref(pr), ctypes.byref(parts))
    return b.value, pr.value, parts.value


#: a feed-forward's gate|up product with SwiGLU as its epilogue goes to the persistent tcgen05 product
#: from this many rows on, also where the other products stay on the library (0: never)
PROMPT_SWIGLU_MIN_ROWS = int(os.environ.get("VAPI_PROMPT_SWIGLU_MIN_ROWS", "256"))


def linear_swiglu(x: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """``silu(x @ Wg.T) * (x @ Wu.T)`` for ``weight = [Wg; Wu]``: one kernel with SwiGLU as the
    product's epilogue for prompt-sized bfloat16 steps, else the product followed by :func:`swiglu`."""
    rows = x.shape[0]
    if (x.dtype == torch.bfloat16 and 0 < PROMPT_SWIGLU_MIN_ROWS <= rows and rows > TC_MAX_ROWS and weight.is_cuda
            and weight.dtype == torch.bfloat16 and weight.dim() == 2 and weight.shape[1] % 8 == 0 and weight.shape[0] % 16 == 0
            and weight.is_contiguous() and x.is_contiguous()):
        return prompt_linear(weight, act=x, epilogue="swiglu")
    return swiglu(linear(x, weight))


def prompt_force(bn: int = 0, pair: int = 0) -> None:
    """Fix the tile (128 | 256 features) and the blocks working on a tile (1 | 2) of
    :func:`prompt_linear` for the calls that follow; 0 gives the choice back to the kernel's plan."""
    lib = _lib("linear_prompt")
    _check(lib, lib.vapi_prompt_linear_force(bn, pair), launches=0)


def prompt_linear(weight: torch.Tensor, *, act: Optional[torch.Tensor] = None, xw: Optional[torch.Tensor] = None,
                  ss_in: Optional[torch.Tensor] = None, eps: float = 0.0, epilogue: str = "bf16",
                  bias: Optional[torch.Tensor] = None, resid: Optional[torch.Tensor] = None,
                  next_weight: Optional[torch.Tensor] = None, status: Optional[torch.Tensor] = None):
    """The persistent tcgen05 / TMA product for prompt-sized steps; same operands, epilogues and
    results as :func:`skinny_linear`."""
    return _fused_product("linear_prompt", weight, act, xw, ss_in, eps, epilogue, bias, resid, next_weight, status)


def few_rows_applies(rows: int, weight: torch.Tensor) -> bool:
    """Whether one of this package's own products (with their fused prologues and epilogues)
    takes a step of ``rows`` rows against ``weight``."""
    return skinny_applies(rows, weight) or tc_applies(rows, weight) or prompt_applies(rows, weight)


def few_rows_linear(weight: torch.Tensor, **kw):
    """:func:`skinny_linear` up to 16 rows, :func:`linear_tc` up to TC_MAX_ROWS, :func:`prompt_linear` above."""
    src = kw.get("act") if kw.get("act") is not None else kw.get("xw")
    if src.shape[0] <= SKINNY_MAX_ROWS:
        return skinny_linear(weight, **kw)
    if src.shape[0] <= TC_MAX_ROWS:
        return linear_tc(weight, **kw)
    return prompt_linear(weight, **kw)


def skinny_f32_applies(rows: int, weight: torch.Tensor) -> bool:
    """Whether the float32 weight-streaming kernel takes this product: float32 weight, at most 16
    rows, inner size a multiple of 4."""
    return (use_skinny and weight.is_cuda and weight.dtype == torch.float32 and 0 < rows <= SKINNY_MAX_ROWS
            and weight.dim() == 2 and weight.shape[1] % 4 == 0 and weight.is_contiguous() and weight.data_ptr() % 16 == 0)


def skinny_linear_f32(weight: torch.Tensor, act: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``act @ weight.T (+ bias)`` for at most 16 rows in true float32 (FMA only): the decode
    product of the 32-bit path, bound by reading the weight once."""
    _cuda(weight, act, bias)
    N, K = weight.shape
    M = act.shape[0]
    if weight.dtype != torch.float32 or not weight.is_contiguous():
        raise KernelError("skinny_linear_f32 needs a contiguous float32 weight")
    if act.dtype != torch.float32 or tuple(act.shape) != (M, K) or not act.is_contiguous():
        raise KernelError(f"skinny_linear_f32: token operand {tuple(act.shape)} / {act.dtype} does not fit a weight of {N}x{K}")
    _f32(bias, "bias")
    out = torch.empty((M, N), dtype=torch.float32, device=weight.device)
    lib = _lib("gemv")
    _check(lib, lib.vapi_skinny_linear_f32(_p(weight), N, K, M, _p(act), _p(bias), _p(out), ctypes.c_longlong(N), _stream()))
    return out


def linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None,
           out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """``x @ weight.T (+ bias)``.  The library matrix product, except for decode-sized
    bfloat16 products (at most 16 rows), which go to the weight-streaming kernel.

    float32 runs without any reduced-precision mode (see :func:`strict_fp32`).  A weight kept
    in float32 beside bfloat16 activations is multiplied in float32.
    """
    _cuda(x, weight)
    if x.dtype == torch.bfloat16 and skinny_applies(x.shape[0], weight) and x.is_contiguous():
        if out_dtype in (None, torch.bfloat16):
            return skinny_linear(weight, act=x, epilogue="bf16", bias=bias)
        if out_dtype == torch.float32:
            return skinny_linear(weight, act=x, epilogue="f32", bias=bias)
    if x.dtype == torch.bfloat16 and tc_applies(x.shape[0], weight) and x.is_contiguous():
        if out_dtype in (None, torch.bfloat16):
            return linear_tc(weight, act=x, epilogue="bf16", bias=bias)
        if out_dtype == torch.float32:
            return linear_tc(weight, act=x, epilogue="f32", bias=bias)
    if (x.dtype == torch.float32 and out_dtype in (None, torch.float32) and skinny_f32_applies(x.shape[0], weight)
            and x.is_contiguous() and x.data_ptr() % 16 == 0):
        return skinny_linear_f32(weight, x, bias)
    if weight.dtype != x.dtype:
        y = torch.mm(x.to(torch.float32), weight.to(torch.float32).t())
        if bias is not None:
            y = y + bias
        return y.to(out_dtype or x.dtype)
    if out_dtype is not None and out_dtype != x.dtype:
        if bias is not None:
            return (torch.mm(x, weight.t(), out_dtype=out_dtype) + bias.to(out_dtype))
        return torch.mm(x, weight.t(), out_dtype=out_dtype)
    if bias is not None:
        return torch.addmm(bias.to(x.dtype), x, weight.t())
    return torch.mm(x, weight.t())


def strict_fp32() -> None:
    """Switch off every reduced-precision matrix mode of the library products."""
    torch.backends.cuda.matmul.allow_tf32 = False
    torch.backends.cudnn.allow_tf32 = False
    torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False
    torch.backends.cuda.matmul.allow_fp16_reduced_precision_reduction = False
    try:
        torch.set_float32_matmul_precision("highest")
    except Exception:  # pragma: no cover
        pass


def rope_cos_sin(positions: torch.Tensor, inv_freq: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """cos and sin of ``position * inv_freq`` in float32: two [n, len(inv_freq)] tensors."""
    _cuda(positions, inv_freq)
    _i32(positions, "positions")
    _f32(inv_freq, "inv_freq")
    n, half = positions.numel(), inv_freq.numel()
    cos = torch.empty((n, half), dtype=torch.float32, device=positions.device)
    sin = torch.empty_like(cos)
    lib = _lib("rope")
    _check(lib, lib.vapi_rope_cos_sin(_p(positions), _p(inv_freq), _p(cos), _p(sin), n, half, _stream()))
    return cos, sin


def qk_norm_rope_write(qkv: torch.Tensor, nh: int, nkv: int, d: int,
                       q_weight: Optional[torch.Tensor], k_weight: Optional[torch.Tensor], eps: float,
                       cos: Optional[torch.Tensor], sin: Optional[torch.Tensor], rot: int,
                       cache_layer: Optional[torch.Tensor], slot_mapping: Optional[torch.Tensor],
                       status: Optional[torch.Tensor] = None) -> None:
    """Per-head RMSNorm and rotate-half RoPE of q and k in a fused ``qkv`` [n, (nh+2nkv)*d];
    q is rewritten in place, k (normed, roped) and v go to ``cache_layer``
    [pages, 2, nkv, page_size, d] at ``slot_mapping``.  ``cache_layer=None`` leaves the
    cache alone (a layer that reads another layer's cache)."""
    _cuda(qkv, q_weight, k_weight, cos, sin, cache_layer, slot_mapping)
    _contig(qkv, "qkv")
    _f32(q_weight, "q norm weight")
    _f32(k_weight, "k norm weight")
    _f32(cos, "cos")
    _f32(sin, "sin")
    _i32(slot_mapping, "slot mapping")
    n = qkv.shape[0]
    if qkv.shape[1] != (nh + 2 * nkv) * d:
        raise KernelError(f"qkv has {qkv.shape[1]} columns, expected {(nh + 2 * nkv) * d}")
    page_size = num_pages = 0
    if cache_layer is not None:
        _contig(cache_layer, "cache layer")
        if cache_layer.dtype != qkv.dtype or tuple(cache_layer.shape[1:3]) != (2, nkv) or cache_layer.shape[4] != d:
            raise KernelError(f"cache layer {tuple(cache_layer.shape)} / {cache_layer.dtype} does not fit "
                              f"nkv={nkv} d={d} {qkv.dtype}")
        num_pages, page_size = cache_layer.shape[0], cache_layer.shape[3]
    if cos is not None and (cos.shape != (n, rot // 2) or sin is None or sin.shape != cos.shape):
        raise KernelError("cos/sin must be [n, rot/2]")
    lib = _lib("rope")
    _check(lib, lib.vapi_qk_norm_rope_write(
        _p(qkv), _dt(qkv), _p(q_weight), _p(k_weight), ctypes.c_float(eps), _p(cos), _p(sin), rot,
        _p(cache_layer), _p(slot_mapping), n, nh, nkv, d, page_size, num_pages, _p(status), _stream()))


# "tma": decode steps at head size 64 on the TMA-fed decode kernel; "mma": on the one-warp flash kernel
DECODE_ATTENTION = os.environ.get("VAPI_DECODE_ATTENTION", "tma")
_decode_limits: Optional[Tuple[int, int]] = None


def decode_attention_limits() -> Tuple[int, int]:
    """(blocks of the decode kernel that the device holds at once, the most slices of the keys that
    it combines inside the kernel), as the library reports them."""
    global _decode_limits
    if _decode_limits is None:
        lib = _lib("attention")
        lib.vapi_attention_use_decode_kernel(1 if DECODE_ATTENTION == "tma" else 0)
        _decode_limits = (int(lib.vapi_decode_attention_slots()) or sm_count() * 3, int(lib.vapi_decode_attention_cluster()))
    return _decode_limits


def decode_attention_applies(dtype: torch.dtype, d: int, page_size: int, rows: int) -> bool:
    """Whether a step whose sequences bring at most ``rows`` rows (tokens x q heads per kv head)
    runs on the decode kernel (the library's own rule, restated)."""
    return (DECODE_ATTENTION == "tma" and dtype == torch.bfloat16 and d == 64 and page_size % 64 == 0
            and rows <= 16)


def decode_attention_combines(num_seqs: int, nkv: int, splits: int) -> bool:
    """Whether the decode kernel combines its slices itself (at most a cluster's worth of slices,
    the whole grid resident at once, and a cluster of that size fits the device): the library's answer."""
    if splits <= 1:
        return False
    decode_attention_limits()
    return bool(_lib("attention").vapi_decode_attention_combines(num_seqs, nkv, splits))


def attention_splits(num_seqs: int, max_q: int, max_k: int, nh: int, nkv: int, decode_kernel: bool = False) -> int:
    """How many blocks share the keys of one row tile: 1 unless the step is so small that
    the device would sit idle (decode of few sequences over long contexts).  A block of the
    one-warp flash kernel has 48 KB of shared memory, so 4 fit on a multiprocessor: aim at one
    full wave of 4 blocks on each, every block with at least 128 keys.

    The decode kernel (measured at head size 64, 8 kv heads, context 4096 and 32768): while the
    (sequence, kv head) pairs are fewer than two blocks per SM, slices up to that many blocks, and
    no more than the kernel combines itself unless a slice would then be longer than 32 tiles and
    there would be fewer blocks than SMs;
    a step with more pairs than the device holds blocks is cut for about four rounds of blocks, so
    that the last ones do not run alone."""
    n_rep = nh // nkv
    rows = max_q * n_rep
    tiles = -(-rows // (16 if rows <= 16 else 64))
    blocks = max(1, num_seqs * nkv * tiles)
    if decode_kernel:
        key_tiles = max(1, -(-max_k // 64))
        slots, cluster = decode_attention_limits()
        by_len = max(1, key_tiles // 2)
        if blocks > slots:
            return max(1, min(-(-4 * slots // blocks), by_len, 32))
        want = max(1, int(round(2 * slots / 3 / blocks)))
        if want > cluster and (key_tiles <= 32 * cluster or 3 * blocks * cluster >= slots):
            want = cluster
        return max(1, min(want, by_len, 32))
    sms = sm_count()
    if rows > 16 and blocks >= sms:
        return 1
    want = max(1, 4 * sms // blocks)
    by_len = max(1, max_k // 128)
    return max(1, min(want, by_len, 32))


def paged_attention(q: torch.Tensor, q_row_stride: int, cache_layer: torch.Tensor,
                    block_table: torch.Tensor, cu_q: torch.Tensor, seqlens_k: torch.Tensor,
                    n: int, num_seqs: int, max_q: int, max_k: int, nh: int, nkv: int, d: int,
                    scale: float, window: int = 0, splits: Optional[int] = None,
                    status: Optional[torch.Tensor] = None, impl: str = "auto") -> torch.Tensor:
    """Causal GQA attention of a mixed batch over the paged cache; returns [n, nh*d].

    ``q`` may be a view into a fused qkv tensor: head h of token t is at
    ``t*q_row_stride + h*d``.  ``window`` > 0 limits each query to the last ``window`` keys.
    ``impl``: "tcgen05" forces the kernel on the fifth-generation tensor cores (bfloat16, head_dim 64,
    pages of 64n, no split), which "auto" uses for steps with prompt portions of 64 tokens or more;
    "auto" otherwise picks the tensor-core kernel where it applies (bfloat16, head_dim 64 or
    128, page size a multiple of 64) and the general kernel elsewhere; "general" and
    "tensor_core" force one (the latter raises where it does not apply); "decode" forces the
    TMA-fed decode kernel (bfloat16, head_dim 64, at most 16 rows per sequence and kv head).
    """
    _cuda(q, cache_layer, block_table, cu_q, seqlens_k)
    _i32(block_table, "block table")
    _i32(cu_q, "cu_q")
    _i32(seqlens_k, "seqlens_k")
    _contig(cache_layer, "cache layer")
    if cache_layer.dtype != q.dtype:
        raise KernelError("q and the cache must have one dtype")
    if block_table.dim() != 2 or block_table.stride(1) != 1:
        raise KernelError("block table must be [S, width] with unit inner stride")
    num_pages, page_size = cache_layer.shape[0], cache_layer.shape[3]
    if splits is None:
        splits = 1 if impl == "tcgen05" else attention_splits(
            num_seqs, max_q, max_k, nh, nkv,
            impl == "decode" or (impl == "auto" and decode_attention_applies(q.dtype, d, page_size, max_q * (nh // nkv))))
    out = torch.empty((n, nh * d), dtype=q.dtype, device=q.device)
    part_o = part_ml = None
    if splits > 1:
        part_o = torch.empty((n * nh * splits * d,), dtype=torch.float32, device=q.device)
        part_ml = torch.empty((n * nh * splits * 2,), dtype=torch.float32, device=q.device)
    lib = _lib("attention")
    decode_attention_limits()             # (also tells the library whether the decode kernel is in use)
    # how many kernels the library launches (its own rule, restated for the launch count): the
    # tcgen05 kernel takes steps with prompt portions, beside the flash kernel and the decode kernel in a mixed step
    tc = impl == "tcgen05" or (impl == "auto" and q.dtype == torch.bfloat16 and d == 64 and page_size % 64 == 0
                               and splits == 1 and max_q >= 64 and q_row_stride % 8 == 0 and scale > 0)
    launches = (1 if impl == "tcgen05" or num_seqs == 1 else (3 if nh // nkv <= 16 and DECODE_ATTENTION == "tma" else 2)) \
        if tc else (2 if splits > 1 else 1)
    if (impl == "decode" or (impl == "auto" and decode_attention_applies(q.dtype, d, page_size, max_q * (nh // nkv)))) \
            and decode_attention_combines(num_seqs, nkv, splits):
        launches = 1                      # the decode kernel's slices combine among themselves
    elif (not tc and impl == "auto" and DECODE_ATTENTION == "tma" and max_q * (nh // nkv) > 16
            and decode_attention_applies(q.dtype, d, page_size, nh // nkv)):
        launches += 1                     # short portions on the flash kernel, decode tokens on the decode kernel
    code = {"auto": 0, "general": 1, "tensor_core": 2, "tcgen05": 3, "decode": 4}[impl]
    _check(lib, lib.vapi_paged_attention(
        _p(q), ctypes.c_longlong(q_row_stride), _p(cache_layer), _dt(q), _p(block_table),
        block_table.stride(0), _p(cu_q), _p(seqlens_k), _p(out), _p(part_o), _p(part_ml), n, num_seqs,
        max_q, nh, nkv, d, page_size, num_pages, ctypes.c_float(scale), window, splits,
        code, _p(status), _stream()), launches)
    return out


#: whether decode steps run q/k norm, RoPE and the cache write inside the decode attention kernel.  Off
#: unless asked for: it gives the same bits with one launch fewer per attention layer, but measured no
#: faster (batch 8) to 1 % slower (batch 1 and 64) than the two kernels, whose first one hides behind
#: the product before it.
FUSED_DECODE_ROPE = os.environ.get("VAPI_FUSED_DECODE_ROPE", "0") == "1"


def decode_attention_fused_applies(dtype: torch.dtype, d: int, page_size: int, rows: int, rot: Optional[int]) -> bool:
    """Whether :func:`decode_attention_fused` takes a step of this shape (``rot``: the rotated width, or
    None without a position encoding)."""
    return decode_attention_applies(dtype, d, page_size, rows) and (rot is None or rot == d)


def decode_attention_fused(qkv: torch.Tensor, nh: int, nkv: int, d: int,
                           q_weight: Optional[torch.Tensor], k_weight: Optional[torch.Tensor], eps: float,
                           cos: Optional[torch.Tensor], sin: Optional[torch.Tensor],
                           cache_layer: torch.Tensor, write_kv: bool, block_table: torch.Tensor,
                           cu_q: torch.Tensor, seqlens_k: torch.Tensor, n: int, num_seqs: int, max_q: int,
                           max_k: int, scale: float, window: int = 0, splits: Optional[int] = None,
                           status: Optional[torch.Tensor] = None) -> torch.Tensor:
    """:func:`qk_norm_rope_write` and :func:`paged_attention` of a decode step in one kernel: per-head
    RMSNorm and rotate-half RoPE of q and of the new keys, the new keys and values written to
    ``cache_layer`` (``write_kv``) at the places the block table gives for the sequences' last
    ``q`` positions, and attention over the cache.  ``qkv`` [n, (nh+2nkv)*d] is left as it was.
    bfloat16, head_dim 64, pages of 64n, at most 16 rows per sequence and kv head.  Gives exactly
    what the two calls give."""
    _cuda(qkv, q_weight, k_weight, cos, sin, cache_layer, block_table, cu_q, seqlens_k)
    _contig(qkv, "qkv")
    _contig(cache_layer, "cache layer")
    _f32(q_weight, "q norm weight")
    _f32(k_weight, "k norm weight")
    _f32(cos, "cos")
    _f32(sin, "sin")
    _i32(block_table, "block table")
    _i32(cu_q, "cu_q")
    _i32(seqlens_k, "seqlens_k")
    if qkv.dtype != torch.bfloat16 or cache_layer.dtype != torch.bfloat16:
        raise KernelError("the fused decode attention is for bfloat16")
    if qkv.shape[0] != n or qkv.shape[1] != (nh + 2 * nkv) * d:
        raise KernelError(f"qkv is {tuple(qkv.shape)}, expected ({n}, {(nh + 2 * nkv) * d})")
    if tuple(cache_layer.shape[1:3]) != (2, nkv) or cache_layer.shape[4] != d:
        raise KernelError(f"cache layer {tuple(cache_layer.shape)} does not fit nkv={nkv} d={d}")
    if block_table.dim() != 2 or block_table.stride(1) != 1:
        raise KernelError("block table must be [S, width] with unit inner stride")
    if cos is not None and (cos.shape != (n, d // 2) or sin is None or sin.shape != cos.shape or not cos.is_contiguous()
                            or not sin.is_contiguous()):
        raise KernelError("cos/sin must be contiguous [n, head_dim/2]")
    for w, name in ((q_weight, "q"), (k_weight, "k")):
        if w is not None and (w.numel() != d or not w.is_contiguous()):
            raise KernelError(f"the {name} norm weight must be [head_dim]")
    num_pages, page_size = cache_layer.shape[0], cache_layer.shape[3]
    if splits is None:
        splits = attention_splits(num_seqs, max_q, max_k, nh, nkv, True)
    out = torch.empty((n, nh * d), dtype=qkv.dtype, device=qkv.device)
    part_o = part_ml = None
    if splits > 1:
        part_o = torch.empty((n * nh * splits * d,), dtype=torch.float32, device=qkv.device)
        part_ml = torch.empty((n * nh * splits * 2,), dtype=torch.float32, device=qkv.device)
    lib = _lib("attention")
    decode_attention_limits()
    launches = 1 if splits == 1 or decode_attention_combines(num_seqs, nkv, splits) else 2
    _check(lib, lib.vapi_decode_attention_fused(
        _p(qkv), _p(q_weight), _p(k_weight), ctypes.c_float(eps), _p(cos), _p(sin), _p(cache_layer),
        1 if write_kv else 0, _p(block_table), block_table.stride(0), _p(cu_q), _p(seqlens_k), _p(out),
        _p(part_o), _p(part_ml), n, num_seqs, max_q, nh, nkv, d, page_size, num_pages, ctypes.c_float(scale),
        window, splits, _p(status), _stream()), launches)
    return out


def shortconv(h3: torch.Tensor, in_bias: Optional[torch.Tensor], taps: torch.Tensor,
              conv_bias: Optional[torch.Tensor], state_layer: Optional[torch.Tensor],
              state_slots: torch.Tensor, tok_seq: torch.Tensor, cu_q: torch.Tensor,
              positions: torch.Tensor, status: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Gating, causal depthwise convolution and state update of the short-conv mixer.

    ``h3`` [n, 3H] = B | C | x; ``taps`` [L, H] oldest first; ``state_layer`` is a view
    [slots, L-1, H] of the per-request state (any slot stride).  Returns y [n, H].
    """
    _cuda(h3, in_bias, taps, conv_bias, state_layer, state_slots, tok_seq, cu_q, positions)
    _contig(h3, "h3")
    _f32(in_bias, "in_proj bias")
    _f32(taps, "conv taps")
    _f32(conv_bias, "conv bias")
    for t, w in ((state_slots, "state slots"), (tok_seq, "tok_seq"), (cu_q, "cu_q"), (positions, "positions")):
        _i32(t, w)
    n, three_h = h3.shape
    hidden = three_h // 3
    L = taps.shape[0]
    if three_h != 3 * hidden or taps.shape[1] != hidden:
        raise KernelError("h3 must be [n, 3H] and taps [L, H]")
    slot_stride = num_slots = 0
    if L > 1:
        if state_layer is None or state_layer.dtype != h3.dtype or tuple(state_layer.shape[1:]) != (L - 1, hidden):
            raise KernelError(f"state must be [slots, {L - 1}, {hidden}] of {h3.dtype}")
        if state_layer.stride(2) != 1 or state_layer.stride(1) != hidden:
            raise KernelError("state rows must be contiguous")
        slot_stride, num_slots = state_layer.stride(0), state_layer.shape[0]
    out = torch.empty((n, hidden), dtype=h3.dtype, device=h3.device)
    num_seqs = cu_q.numel() - 1
    lib = _lib("shortconv")
    _check(lib, lib.vapi_shortconv(
        _p(h3), _dt(h3), _p(in_bias), _p(taps), _p(conv_bias), _p(state_layer if L > 1 else None),
        ctypes.c_longlong(slot_stride), _p(state_slots), _p(tok_seq), _p(cu_q), _p(positions), _p(out),
        n, num_seqs, hidden, L, num_slots, _p(status), _stream()))
    return out


_sample_bufs: Dict[str, Tuple[torch.Tensor, torch.Tensor, torch.Tensor]] = {}


def _sample_scratch(device, rows: int, slices: int):
    """Persistent scratch of the sliced argmax (the counters start at zero and every launch
    leaves them zero, so the buffer must not be handed out fresh each call)."""
    key = str(device)
    buf = _sample_bufs.get(key)
    need = rows * slices
    if buf is None or buf[0].numel() < need or buf[2].numel() < rows:
        cap_r, cap = max(rows, 256), max(need, 256 * 32)
        buf = (torch.empty(cap, dtype=torch.float32, device=device), torch.empty(cap, dtype=torch.int32, device=device),
               torch.zeros(cap_r, dtype=torch.int32, device=device))
        _sample_bufs[key] = buf
    return buf


def sample_rows(logits: torch.Tensor, mode: Optional[torch.Tensor] = None,
                inv_t: Optional[torch.Tensor] = None, seeds: Optional[torch.Tensor] = None,
                draws: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """One token per row of float32 ``logits`` [R, V]: greedy argmax (lowest id wins ties),
    or, where ``mode`` is 2, Gumbel-max temperature sampling keyed by (seed, draw)."""
    _cuda(logits, mode, inv_t, seeds, draws)
    if logits.dtype != torch.float32 or logits.stride(1) != 1:
        raise KernelError("logits must be float32 with unit inner stride")
    _i32(mode, "mode")
    _f32(inv_t, "inverse temperatures")
    for t in (seeds, draws):
        if t is not None and t.dtype != torch.int64:
            raise KernelError("seeds and draw counters must be int64")
    rows, vocab = logits.shape
    if out is None:
        out = torch.empty((rows,), dtype=torch.int32, device=logits.device)
    # few rows over a large vocabulary: cut each row into slices so that more than `rows` blocks work
    slices = 1
    wave = 4 * sm_count()
    if rows < wave and vocab >= 8192:
        slices = max(1, min(32, wave // rows, vocab // 2048))
    part_v = part_i = counters = None
    if slices > 1:
        part_v, part_i, counters = _sample_scratch(logits.device, rows, slices)
    lib = _lib("sampling")
    _check(lib, lib.vapi_sample_rows(_p(logits), rows, vocab, ctypes.c_longlong(logits.stride(0)), _p(mode),
                                     _p(inv_t), _p(seeds), _p(draws), _p(out), slices, _p(part_v), _p(part_i),
                                     _p(counters), _stream()))
    return out


def sample_truncated(logits: torch.Tensor, inv_t: torch.Tensor, top_k: Optional[torch.Tensor],
                     top_p: Optional[torch.Tensor], min_p: Optional[torch.Tensor], seeds: torch.Tensor,
                     draws: torch.Tensor, out: Optional[torch.Tensor] = None, check: bool = False):
    """One token per row from the temperature distribution cut by top-k (0: none; negative: leave
    the row alone), min-p (0: none) and top-p (1: none), drawn by Gumbel-max over the survivors
    with noise keyed by (seed, draw).  With ``check`` also returns the threshold on the scaled
    logits and the number of survivors per row."""
    _cuda(logits, inv_t, top_k, top_p, min_p, seeds, draws, out)
    if logits.dtype != torch.float32 or logits.stride(1) != 1:
        raise KernelError("logits must be float32 with unit inner stride")
    _f32(inv_t, "inverse temperatures")
    _f32(top_p, "top_p")
    _f32(min_p, "min_p")
    _i32(top_k, "top_k")
    for t in (seeds, draws):
        if t.dtype != torch.int64:
            raise KernelError("seeds and draw counters must be int64")
    rows, vocab = logits.shape
    if out is None:
        out = torch.empty((rows,), dtype=torch.int32, device=logits.device)
    tau = cnt = None
    if check:
        tau = torch.zeros((rows,), dtype=torch.float32, device=logits.device)
        cnt = torch.zeros((rows,), dtype=torch.int32, device=logits.device)
    lib = _lib("sampling")
    _check(lib, lib.vapi_sample_truncated(_p(logits), rows, vocab, ctypes.c_longlong(logits.stride(0)), _p(inv_t), _p(top_k),
                                          _p(top_p), _p(min_p), _p(seeds), _p(draws), _p(out), _p(tau), _p(cnt), _stream()))
    return (out, tau, cnt) if check else out


def apply_penalties(logits: torch.Tensor, rows: torch.Tensor, toks: torch.Tensor, counts: torch.Tensor,
                    rep: torch.Tensor, freq: torch.Tensor, pres: torch.Tensor) -> None:
    """Repetition / frequency / presence penalties on (row, token) pairs, in place."""
    _cuda(logits, rows, toks, counts, rep, freq, pres)
    _i32(rows, "rows")
    _i32(toks, "tokens")
    for t, w in ((counts, "counts"), (rep, "repetition"), (freq, "frequency"), (pres, "presence")):
        _f32(t, w)
    lib = _lib("sampling")
    _check(lib, lib.vapi_apply_penalties(_p(logits), logits.shape[1], ctypes.c_longlong(logits.stride(0)),
                                         _p(rows), _p(toks), _p(counts), _p(rep), _p(freq), _p(pres),
                                         rows.numel(), _stream()))
