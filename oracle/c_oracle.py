"""ctypes front end of the C restatement (oracle/kvattn_oracle.c).  Test infrastructure: used by
tests and by the benchmark's CPU-baseline leg only."""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

from . import build_c
from .oracle import KVCache, _table2d

_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        path = build_c.build()
        _lib = C.CDLL(path)
        _lib.kv_threads.restype = C.c_int
    return _lib


def _p(a: np.ndarray):
    return a.ctypes.data_as(C.c_void_p)


def set_threads(n: int) -> None:
    """Use n OpenMP threads (launchers such as torchrun export OMP_NUM_THREADS=1)."""
    lib().kv_set_threads(C.c_int(int(n)))


def threads() -> int:
    return int(lib().kv_threads())


def quantize_rows(x: np.ndarray):
    x = np.ascontiguousarray(x, np.float32)
    D = x.shape[-1]
    rows = x.size // D
    codes = np.empty(x.shape, np.int8)
    scales = np.empty(x.shape[:-1], np.float32)
    lib().kv_quantize_rows(_p(x), C.c_int64(rows), C.c_int(D), _p(codes), _p(scales))
    return codes, scales


def norm_rope(x, w, cos, sin, eps: float) -> np.ndarray:
    x = np.ascontiguousarray(x, np.float32)
    T, H, D = x.shape
    assert D == 128
    w = np.ascontiguousarray(w, np.float32)
    cos = np.ascontiguousarray(np.asarray(cos, np.float32).reshape(T, D // 2))
    sin = np.ascontiguousarray(np.asarray(sin, np.float32).reshape(T, D // 2))
    out = np.empty_like(x)
    lib().kv_norm_rope(_p(x), C.c_int64(T), C.c_int(H), _p(w), _p(cos), _p(sin), C.c_float(eps), _p(out))
    return out


def decode_attention(q, cache: KVCache, cached_lens, table, num_decoding: int, scale: float, out=None) -> np.ndarray:
    q = np.ascontiguousarray(q, np.float32)
    B, Hq, D = q.shape
    assert D == 128
    tab = np.ascontiguousarray(_table2d(table), np.int32)
    cl = np.ascontiguousarray(cached_lens, np.int32)
    if out is None:
        out = np.zeros((B, Hq, D), np.float32)
    for a in (cache.k, cache.v, cache.k_scale, cache.v_scale):
        assert a.flags.c_contiguous
    lib().kv_decode_attention(_p(q), _p(cache.k), _p(cache.v), _p(cache.k_scale), _p(cache.v_scale), _p(tab),
                              C.c_int(tab.shape[1]), _p(cl), C.c_int(B), C.c_int(int(num_decoding)), C.c_int(Hq),
                              C.c_int(cache.k.shape[1]), C.c_int(cache.page_size), C.c_float(scale), _p(out))
    return out
