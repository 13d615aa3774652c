"""Loader of the host runtime (``csrc/host.cpp``): page and slot pools, block tables, the step
packer and the scheduler, in C++ behind a C interface.  Built on first use like the kernel
libraries; there is no Python fallback for it.
"""
from __future__ import annotations

import ctypes
import threading
from typing import Optional

import numpy as np

from .csrc import build as _build

_lib: Optional[ctypes.CDLL] = None
_lock = threading.Lock()
path: Optional[str] = None

_I, _P = ctypes.c_int, ctypes.c_void_p

_SIGNATURES = {
    "vh_last_error": (ctypes.c_char_p, []),
    "vh_pool_new": (_P, [_I, _I]), "vh_pool_delete": (None, [_P]), "vh_pool_size": (_I, [_P]),
    "vh_pool_watermark": (_I, [_P]), "vh_pool_num_free": (_I, [_P]), "vh_pool_can_allocate": (_I, [_P, _I]),
    "vh_pool_allocate": (_I, [_P]), "vh_pool_release": (_I, [_P, _I]), "vh_pool_held": (_I, [_P, _P, _I]),
    "vh_pool_check": (_I, [_P]),
    "vh_cache_new": (_P, [_I, _I, _P, _P, _P, _I]), "vh_cache_delete": (None, [_P]),
    "vh_cache_group_pool": (_P, [_P, _I]), "vh_cache_slot_pool": (_P, [_P]),
    "vh_open": (_I, [_P]), "vh_close": (_I, [_P, _I]), "vh_reserve": (_I, [_P, _I, _I, _I]),
    "vh_commit": (_I, [_P, _I, _I]), "vh_can_admit": (_I, [_P, _I]), "vh_is_live": (_I, [_P, _I]),
    "vh_slot": (_I, [_P, _I]), "vh_num_tokens": (_I, [_P, _I]), "vh_first_live": (_I, [_P, _I, _I]),
    "vh_table": (_I, [_P, _I, _I, _P, _I]), "vh_commit_many": (_I, [_P, _I, _P, _P]),
    "vh_set_aside": (_I, [_P, _P]), "vh_cache_check": (_I, [_P]),
    "vh_layout_len": (_I, [_I]), "vh_layout": (None, [_I, _I, _I, _I, _I, _P]),
    "vh_pack": (_I, [_P, _I, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _P, _I, _P, _P]),
    "vs_new": (_P, [_P, _I, _I, _I, _I, _P, _I]), "vs_delete": (None, [_P]),
    "vs_admit": (_I, [_P, _P, _I, _I, _I, _P, _I]), "vs_schedule": (_I, [_P]),
    "vs_commit": (_I, [_P, _P, _I]), "vs_finish": (None, [_P, _I, _I]), "vs_fail_all": (_I, [_P, _P, _I]),
    "vs_list": (_I, [_P, _I, _P, _I]), "vs_plan_info": (None, [_P, _P]),
    "vs_pack_plan": (_I, [_P, _I, _I, _I, _I, _I, _P, _I, _P, _P]),
    "vs_advance": (_I, [_P]), "vs_resolve": (_I, [_P, _P, _P, _I, _P]), "vs_can_run_ahead": (_I, [_P]),
    "vs_commit_cache": (_I, [_P]), "vs_clear_finished": (None, [_P]), "vs_erase": (None, [_P, _I]), "vs_seq_get": (_I, [_P, _I, _I]),
    "vs_seq_tokens": (_I, [_P, _I, _I, _P, _I]), "vs_counts": (_I, [_P, _I]),
}


def lib() -> ctypes.CDLL:
    global _lib, path
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is None:
            path = _build.build("host")
            handle = ctypes.CDLL(path)
            for name, (res, args) in _SIGNATURES.items():
                fn = getattr(handle, name)
                fn.restype, fn.argtypes = res, args
            _lib = handle
    return _lib


def last_error() -> str:
    return lib().vh_last_error().decode(errors="replace")


def i32(values) -> np.ndarray:
    """A contiguous int32 array (kept alive by the caller for the duration of the call)."""
    return np.ascontiguousarray(values, dtype=np.int32)


def ptr(a: Optional[np.ndarray]) -> int:
    return 0 if a is None else a.ctypes.data
