"""The allocation-free decode-attention entry point (b200kv_decode_attn_static) against the regular
one, through the C ABI.  Kept in a file that pytest collects last: if it fails under -x every
other test has already run.  It must pass alone in a fresh process and after the other tests, so
it builds all of its inputs itself and assumes nothing about the built-in scratch's contents."""
import ctypes

import numpy as np
import pytest
import torch

from tests import helpers as H
from tests.helpers import D, HKV, HQ

pytestmark = pytest.mark.gpu
SCALE = D ** -0.5


def make_case(seed, lens):
    rng = np.random.default_rng(seed)
    num_pages = sum((n + 15) // 16 for n in lens) + 2
    table = H.i32(H.random_block_table(rng, lens, 16, num_pages))
    cache = H.cache_to_torch(H.random_filled_cache(rng, num_pages, 16, gauss=True))
    q = H.bf16_tensor(H.randn_bf16(rng, len(lens), HQ, D))
    cached = H.i32([n - 1 for n in lens])
    return q, cache, cached, table, H.i32([len(lens)])


def call_static(K, q, cache, cached, table, nd):
    """Straight through the C ABI: no workspace argument, output buffer supplied by the caller."""
    from inference_engine_b200 import _lib

    lib = _lib.load()
    out = torch.full(q.shape, 3.0, dtype=torch.bfloat16, device=q.device)
    cs, ts = K._cache_struct(cache), K._table_struct(table)
    rc = lib.b200kv_decode_attn_static(q.data_ptr(), q.stride(0), q.stride(1), ctypes.byref(cs), ctypes.byref(ts),
                                       cached.data_ptr(), nd.data_ptr(), SCALE, out.data_ptr(), out.stride(0),
                                       out.stride(1), q.shape[0], HQ, K.num_sms(q.device),
                                       K.status_word(q.device).data_ptr(), torch.cuda.current_stream().cuda_stream)
    return rc, out


def test_static_scratch_matches_workspace_entry_point():
    from inference_engine_b200 import kernels as K

    # two different batches back to back: the second must not be disturbed by what the first left
    # in the shared built-in scratch (sequences split over many warps, and ones a single warp owns)
    for seed, lens in ((11, [4096, 1, 700, 33, 2048]), (12, [130] * 40 + [3000])):
        q, cache, cached, table, nd = make_case(seed, lens)
        want = K.decode_attention(q, cache, cached, table, nd, SCALE)
        for _ in range(2):  # and the same call twice in a row
            rc, got = call_static(K, q, cache, cached, table, nd)
            assert rc == 0
            torch.cuda.synchronize()
            mx, mean = H.attn_errors(H.to_f32(got), H.to_f32(want))
            assert mx <= 2e-2 and mean <= 2e-3, (mx, mean)  # the tolerance of the attention tests
            assert torch.equal(got, want)  # same kernel and same split: in fact the same bits
    assert K.check_status() == 0


def test_static_scratch_rejects_oversized_requests():
    from inference_engine_b200 import _lib, kernels as K

    lib = _lib.load()
    assert lib.b200kv_decode_attn_static_limit() == 8 << 20
    q, cache, cached, table, nd = make_case(13, [64, 64])
    cs, ts = K._cache_struct(cache), K._table_struct(table)
    out = torch.empty_like(q)
    # a fictitious device with 4000 SMs would need ~100 MB of partials: refused, nothing launched
    rc = lib.b200kv_decode_attn_static(q.data_ptr(), q.stride(0), q.stride(1), ctypes.byref(cs), ctypes.byref(ts),
                                       cached.data_ptr(), nd.data_ptr(), SCALE, out.data_ptr(), out.stride(0),
                                       out.stride(1), 2, HQ, 4000, None, None)
    assert rc == -7
    assert b"8 MiB" in lib.b200kv_error_string(rc)
