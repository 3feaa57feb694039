"""ctypes binding of libb200kv.so (declared in include/b200kv.h).

Loading never falls back to anything: a missing or unloadable library raises, and every
wrapper raises on a negative return code."""
from __future__ import annotations

import ctypes as C
import os

from . import build as _build

c_void_p, c_int32, c_int64, c_float, c_size_t = C.c_void_p, C.c_int32, C.c_int64, C.c_float, C.c_size_t


class Cache(C.Structure):
    """struct b200kv_cache"""

    _fields_ = [
        ("k", c_void_p), ("v", c_void_p), ("k_scale", c_void_p), ("v_scale", c_void_p), ("k_calibration", c_void_p),
        ("stride_page", c_int64), ("stride_head", c_int64), ("stride_tok", c_int64),
        ("sstride_page", c_int64), ("sstride_head", c_int64),
        ("cstride_page", c_int64), ("cstride_head", c_int64),
        ("num_pages", c_int32), ("num_kv_heads", c_int32), ("page_size", c_int32), ("head_dim", c_int32),
    ]


class Table(C.Structure):
    """struct b200kv_table"""

    _fields_ = [("ids", c_void_p), ("stride", c_int32), ("max_pages", c_int32)]


P_CACHE, P_TABLE = C.POINTER(Cache), C.POINTER(Table)

# name -> (restype, argtypes); must list every function include/b200kv.h declares
SIGNATURES = {
    "b200kv_version": (c_int32, []),
    "b200kv_error_string": (C.c_char_p, [c_int32]),
    "b200kv_write_decode": (c_int32, [c_void_p, c_int64, c_int64, c_void_p, c_int64, c_int64, c_void_p, c_int64, c_int64,
                                      c_void_p, c_void_p, c_void_p, c_int64, c_void_p, c_int64, P_CACHE, P_TABLE,
                                      c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int32, c_int32, c_float,
                                      c_void_p, c_void_p]),
    "b200kv_norm_rope_prefill": (c_int32, [c_void_p, c_int64, c_int64, c_void_p, c_int64, c_int64, c_void_p, c_void_p,
                                           c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_int64, c_void_p,
                                           c_int64, c_int64, c_int32, c_int32, c_int32, c_int32, c_float, c_void_p]),
    "b200kv_quantize_prefill": (c_int32, [c_void_p, c_int64, c_int64, c_void_p, c_int64, c_int64, c_void_p, c_int32,
                                          P_CACHE, P_TABLE, c_void_p, c_void_p, c_int32, c_void_p, c_void_p]),
    "b200kv_write_prefill": (c_int32, [c_void_p, c_int64, c_int64, c_void_p, c_int64, c_int64, c_void_p, c_int64, c_int64,
                                       c_void_p, c_void_p, c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int32,
                                       P_CACHE, P_TABLE, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_void_p, c_int64,
                                       c_int64, c_int32, c_int32, c_float, c_void_p, c_void_p]),
    "b200kv_dequant_prefix": (c_int32, [P_CACHE, P_TABLE, c_void_p, c_int32, c_void_p, c_void_p, c_int64, c_int64,
                                        c_int32, c_void_p, c_void_p]),
    "b200kv_prefill_attn": (c_int32, [c_void_p, c_int64, c_int64, c_void_p, c_int64, c_int64, c_void_p, c_int64, c_int64,
                                      c_void_p, c_void_p, c_void_p, c_int32, c_int32, c_void_p, c_void_p, c_int64,
                                      c_int64, c_void_p, c_void_p, c_int64, c_int64, c_int32, c_int32, c_int32, c_int32,
                                      c_void_p]),
    "b200kv_prefill_attn_variant": (c_int32, [c_void_p, c_int64, c_int64, c_void_p, c_int64, c_int64, c_void_p, c_int64,
                                              c_int64, c_void_p, c_void_p, c_void_p, c_int32, c_int32, c_void_p, c_void_p,
                                              c_int64, c_int64, c_int32, c_void_p, c_void_p, c_int64, c_int64, c_int32,
                                              c_int32, c_int32, c_int32, c_int32, c_void_p, c_void_p]),
    "b200kv_silu_mul": (c_int32, [c_void_p, c_int64, c_void_p, c_int64, c_int32, c_int32, c_void_p]),
    "b200kv_add_rms_norm": (c_int32, [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_void_p, c_int64, c_void_p, c_int64,
                                      c_int32, c_int32, c_float, c_void_p]),
    "b200kv_sample_workspace_bytes": (c_size_t, [c_int32, c_int32]),
    "b200kv_sample": (c_int32, [c_void_p, c_int64, c_int32, c_void_p, c_float, c_void_p, c_size_t, c_void_p, c_int64,
                                c_int32, c_int32, c_void_p]),
    "b200kv_skinny_linear": (c_int32, [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_int32, c_int32, c_int32,
                                       c_int32, c_void_p, c_void_p]),
    "b200kv_set_chained_launch": (None, [c_int32]),
    "b200kv_get_chained_launch": (c_int32, []),
    "b200kv_decode_attn_workspace_bytes": (c_size_t, [c_int32, c_int32, c_int32, c_int32, c_int32]),
    "b200kv_decode_attn_workspace_zero_bytes": (c_size_t, [c_int32, c_int32]),
    "b200kv_decode_attn": (c_int32, [c_void_p, c_int64, c_int64, P_CACHE, P_TABLE, c_void_p, c_void_p, c_float, c_void_p,
                                     c_int64, c_int64, c_void_p, c_size_t, c_int32, c_int32, c_int32, c_int32, c_void_p,
                                     c_void_p]),
    "b200kv_decode_plan_bytes": (c_size_t, [c_int32]),
    "b200kv_decode_plan": (c_int32, [P_TABLE, c_void_p, c_void_p, c_int32, c_int32, c_int32, c_int32, c_void_p, c_size_t,
                                     c_void_p]),
    "b200kv_decode_attn_planned": (c_int32, [c_void_p, c_int64, c_int64, P_CACHE, P_TABLE, c_void_p, c_void_p, c_float,
                                             c_void_p, c_int64, c_int64, c_void_p, c_size_t, c_void_p, c_size_t, c_int32,
                                             c_int32, c_int32, c_int32, c_void_p, c_void_p]),
    "b200kv_decode_attn_static_limit": (c_size_t, []),
    "b200kv_decode_attn_static": (c_int32, [c_void_p, c_int64, c_int64, P_CACHE, P_TABLE, c_void_p, c_void_p, c_float,
                                            c_void_p, c_int64, c_int64, c_int32, c_int32, c_int32, c_void_p, c_void_p]),
}

_lib = None


class B200KVError(RuntimeError):
    pass


_path_override = None


def use_library(path: str) -> None:
    """Load this build of the library instead of the default one (the instrumented build of bench.py --phases).
    Must be called before the first op."""
    global _path_override
    if _lib is not None:
        raise B200KVError("a library is already loaded")
    _path_override = path


def load(build_if_needed: bool = True) -> C.CDLL:
    """Load (building first if sources are newer) the CUDA library.  Raises if impossible."""
    global _lib
    if _lib is not None:
        return _lib
    path = _build.LIB
    if build_if_needed and _build.needs_build():
        path = _build.build()
    if _path_override is not None:
        path = _path_override
    elif os.environ.get("B200KV_LIBRARY"):  # another build of the same sources (an experiment with other tile constants)
        path = os.environ["B200KV_LIBRARY"]
    if not os.path.exists(path):
        raise B200KVError(f"{path} is missing: the CUDA extension is required, there is no fallback path")
    lib = C.CDLL(path)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name, None)
        if fn is None:
            continue  # entry points are added unit by unit; exported_symbols() reports what exists
        fn.restype, fn.argtypes = res, args
    _lib = lib
    return lib


def check(rc: int, what: str) -> None:
    if rc != 0:
        msg = load().b200kv_error_string(rc)
        raise ValueError(f"{what}: {msg.decode() if msg else rc}")
