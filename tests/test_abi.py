"""CPU-side checks of the C-ABI boundary: the library builds/loads without a GPU and exports
every function include/b200kv.h declares; the Python binding lists each of them; and the
drop-in module exports every name the reference's architecture.py / engine.py import."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_functions():
    text = open(os.path.join(ROOT, "include", "b200kv.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(b200kv_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_path():
    names = declared_functions()
    for must in ("b200kv_write_decode", "b200kv_decode_attn", "b200kv_decode_attn_workspace_bytes",
                 "b200kv_norm_rope_prefill", "b200kv_quantize_prefill", "b200kv_dequant_prefix", "b200kv_prefill_attn",
                 "b200kv_prefill_attn_variant"):
        assert must in names


def test_library_exports_every_declared_symbol():
    from inference_engine_b200 import _lib, build

    path = build.build()
    lib = ctypes.CDLL(path)
    for name in declared_functions():
        assert hasattr(lib, name), f"{name} is declared in include/b200kv.h but not exported"
        assert name in _lib.SIGNATURES, f"{name} has no ctypes signature"
    assert lib.b200kv_version() == 2
    lib.b200kv_error_string.restype = ctypes.c_char_p
    assert b"workspace" in lib.b200kv_error_string(-4)


def test_workspace_size_is_pure_host_arithmetic():
    from inference_engine_b200 import _lib

    lib = _lib.load()
    n64 = lib.b200kv_decode_attn_workspace_bytes(64, 16, 8, 128, 148)
    n1 = lib.b200kv_decode_attn_workspace_bytes(1, 16, 8, 128, 148)
    assert n64 > n1 > 0 and n64 % 256 == 0
    assert lib.b200kv_decode_attn_workspace_bytes(64, 16, 8, 64, 148) == 0  # head_dim 64 unsupported
    assert lib.b200kv_decode_attn_workspace_bytes(64, 15, 8, 128, 148) == 0


def test_invalid_arguments_launch_nothing():
    """Argument validation happens before any CUDA call, so it can be exercised without a GPU."""
    from inference_engine_b200 import _lib

    lib = _lib.load()
    cache, table = _lib.Cache(), _lib.Table()
    rc = lib.b200kv_decode_attn(None, 0, 0, ctypes.byref(cache), ctypes.byref(table), None, None, 1.0, None, 0, 0, None,
                                0, 1, 16, 148, 0, None, None)
    assert rc == -1
    rc = lib.b200kv_dequant_prefix(ctypes.byref(cache), ctypes.byref(table), 8, 1, 8, 8, 128, 128, 4, None, None)
    assert rc == -1  # cache pointers are NULL


def test_cache_strides_must_fit_32_bits():
    """The kernels form offsets from 32 x 32 -> 64 bit products: a stride of 2^31 or more is refused on the host
    (made-up aligned addresses: validation never dereferences them and nothing is launched)."""
    from inference_engine_b200 import _lib

    lib = _lib.load()
    fake = 0x10000
    cache = _lib.Cache(fake, fake, fake, fake, fake, 8 * 16 * 128, 16 * 128, 128, 8 * 16, 16, 8 * 128, 128, 4, 8, 16, 128)
    table = _lib.Table(fake, 4, 4)
    args = (ctypes.byref(cache), ctypes.byref(table), fake, 1, fake, fake, 128, 1024, 4, None, None)
    # in range: validation passes and the call goes on to launch, which is not done without a GPU here
    cache.stride_page = 1 << 31
    assert lib.b200kv_dequant_prefix(*args) == -6
    cache.stride_page = 8 * 16 * 128
    cache.sstride_page = -4
    assert lib.b200kv_dequant_prefix(*args) == -6


def test_dropin_module_exports_reference_names():
    from inference_engine_b200 import kernels

    for name in ("LayerKVCache", "decode_attention", "fused_rope_kv_decode", "fused_norm_rope_prefill",
                 "quantize_kv_prefill", "dequantize_kv_prefix", "prefill_attention", "silu_mul", "add_rms_norm",
                 "linear", "sample", "tune_linear"):
        assert hasattr(kernels, name)


def test_ops_refuse_cpu_tensors():
    import torch

    from inference_engine_b200 import kernels as K

    cache = K.make_layer_cache(2, 8, 16, 128, device="cpu")
    q = torch.zeros(1, 16, 128, dtype=torch.bfloat16)
    i = torch.zeros(1, dtype=torch.int32)
    with pytest.raises(RuntimeError):
        K.decode_attention(q, cache, i, i, i, 0.088)
