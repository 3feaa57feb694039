"""GPU parity of the quantize-on-write kernels: bit-exact against the reference's own outputs
(golden fixtures) and against the CPU oracle on seeded random inputs, through the drop-in
Python API (which calls the C ABI)."""
import numpy as np
import pytest
import torch

from oracle import oracle as O
from tests import helpers as H
from tests.helpers import D, HKV, HQ

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def K():
    from inference_engine_b200 import kernels

    return kernels


def golden_cache(g, prefix):
    return O.KVCache(g[prefix + "k"].copy(), g[prefix + "v"].copy(), g[prefix + "k_scale"].copy(),
                     g[prefix + "v_scale"].copy(), g[prefix + "k_calibration"].copy())


def split_views(qkv: torch.Tensor):
    n = qkv.shape[0]
    q, k, v = qkv.split([HQ * D, HKV * D, HKV * D], dim=-1)
    return q.view(n, HQ, D), k.view(n, HKV, D), v.view(n, HKV, D)


def test_write_decode_golden(K, golden):
    g = golden
    q, k, v = split_views(H.bits_tensor(g["wd_qkv_bf16"]))
    cache = H.cache_to_torch(golden_cache(g, "wd_in_"))
    nd = int(g["wd_nd"][0])
    out = K.fused_rope_kv_decode(q, k, v, H.bits_tensor(g["wd_qw_bf16"]), H.bits_tensor(g["wd_kw_bf16"]),
                                 H.bits_tensor(g["wd_cos_bf16"]), H.bits_tensor(g["wd_sin_bf16"]), H.i32(g["wd_slots"]),
                                 cache, H.i32(g["wd_cached"]), H.i32(g["wd_nd"]), 1e-6)
    assert np.array_equal(H.to_bits(out[:nd]), g["wd_out_q_bf16"])
    H.assert_cache_equal(H.cache_to_numpy(cache), golden_cache(g, "wd_out_"), "write_decode ")
    assert K.check_status() == 0


def test_prefill_write_golden(K, golden):
    g = golden
    q, k, v = split_views(H.bits_tensor(g["pf_qkv_bf16"]))
    q_p, k_p = K.fused_norm_rope_prefill(q, k, H.bits_tensor(g["wd_qw_bf16"]), H.bits_tensor(g["wd_kw_bf16"]),
                                         H.bits_tensor(g["pf_cos_bf16"]), H.bits_tensor(g["pf_sin_bf16"]), 1e-6)
    assert np.array_equal(H.to_bits(q_p), g["pf_q_p_bf16"])
    assert np.array_equal(H.to_bits(k_p), g["pf_k_p_bf16"])
    cache = H.cache_to_torch(golden_cache(g, "pf_in_"))
    K.quantize_kv_prefill(k_p, v, H.i32(g["pf_cu"]), H.i32(g["pf_slots"]), H.i32(g["pf_cached"]), H.i32(g["pf_nd"]), cache)
    H.assert_cache_equal(H.cache_to_numpy(cache), golden_cache(g, "pf_out_"), "quantize_prefill ")
    k_out = torch.zeros(g["pf_k_prefix_bf16"].shape, dtype=torch.bfloat16, device="cuda")
    v_out = torch.zeros_like(k_out)
    K.dequantize_kv_prefix(cache, H.i32(g["pf_cu_cached"]), H.i32(g["pf_slots"]), k_out, v_out)
    assert np.array_equal(H.to_bits(k_out), g["pf_k_prefix_bf16"])
    assert np.array_equal(H.to_bits(v_out), g["pf_v_prefix_bf16"])
    assert K.check_status() == 0


def make_write_inputs(rng, T):
    qkv = H.randn_bf16(rng, T, (HQ + 2 * HKV) * D)
    qw = O.bf16_round((1 + 0.02 * rng.standard_normal(D)).astype(np.float32))
    kw = O.bf16_round((1 + 0.02 * rng.standard_normal(D)).astype(np.float32))
    pos = rng.integers(0, 32768, T).astype(np.int32)
    cos, sin = O.rope_tables(pos)
    return qkv, qw, kw, pos, cos, sin


def np_views(qkv):
    n = qkv.shape[0]
    return (qkv[:, : HQ * D].reshape(n, HQ, D), qkv[:, HQ * D : (HQ + HKV) * D].reshape(n, HKV, D),
            qkv[:, (HQ + HKV) * D :].reshape(n, HKV, D))


@pytest.mark.parametrize("T", [1, 64, 1024])
@pytest.mark.parametrize("calibrated", [False, True])
def test_write_decode_paged_random(K, T, calibrated):
    """T new tokens written at random free (page, row) slots of a 16-token paged cache; codes,
    scales and rotated q must equal the oracle bit for bit."""
    rng = np.random.default_rng(1000 + T + int(calibrated))
    P = 16
    qkv, qw, kw, pos, cos, sin = make_write_inputs(rng, T)
    # token b sits at position pos[b] of its own sequence; only the page holding it (and page 0,
    # whose calibration row is used) must exist, so the table is wide and sparse
    max_pages = 32768 // P
    num_pages = 2 * T + 2
    table = np.full((T, max_pages), -1, np.int32)
    perm = rng.permutation(num_pages)
    for b in range(T):
        table[b, 0] = perm[2 * b]
        table[b, pos[b] // P] = perm[2 * b + 1] if pos[b] // P else perm[2 * b]
    cache = O.make_cache(num_pages, HKV, P, D)
    if calibrated:
        cache.k_calibration[...] = (0.5 + 2 * rng.random(cache.k_calibration.shape)).astype(np.float32)
    dev_cache = H.cache_to_torch(cache)
    q, k, v = np_views(qkv)
    want_q = O.write_decode(q, k, v, qw, kw, cos, sin, table, cache, pos, T, 1e-6)
    tq, tk, tv = split_views(H.bf16_tensor(qkv))
    got_q = K.fused_rope_kv_decode(tq, tk, tv, H.bf16_tensor(qw), H.bf16_tensor(kw), H.bf16_tensor(cos)[:, None, :],
                                   H.bf16_tensor(sin)[:, None, :], H.i32(table), dev_cache, H.i32(pos), H.i32([T]), 1e-6)
    assert np.array_equal(H.to_bits(got_q), O.bf16_bits(want_q))
    H.assert_cache_equal(H.cache_to_numpy(dev_cache), cache, f"T={T} ")
    assert K.check_status() == 0


@pytest.mark.parametrize("fused", [False, True])
@pytest.mark.parametrize("T", [64, 1024, 1500])
@pytest.mark.parametrize("first_chunk", [True, False])
def test_prefill_write_paged_random(K, T, first_chunk, fused):
    """One T-token prefill chunk behind two decoding entries, paged cache: bf16 q/k outputs,
    calibration, codes and scales equal the oracle; then the dequantized prefix does too.  fused = the single
    write_prefill call instead of fused_norm_rope_prefill + quantize_kv_prefill.  T = 1500: more rows than the
    first-chunk kernel keeps in registers."""
    rng = np.random.default_rng(2000 + T + int(first_chunk))
    P = 16
    prior = 0 if first_chunk else 48
    chunk = [1, 1, T, 0]
    N = sum(chunk)
    cached = np.array([7, 33, prior, 0], np.int32)
    cu = np.concatenate([[0], np.cumsum(chunk)]).astype(np.int32)
    qkv = H.randn_bf16(rng, N, (HQ + 2 * HKV) * D)
    qw = O.bf16_round((1 + 0.02 * rng.standard_normal(D)).astype(np.float32))
    kw = O.bf16_round((1 + 0.02 * rng.standard_normal(D)).astype(np.float32))
    pos = np.concatenate([np.arange(c, c + L) for c, L in zip(cached, chunk)]).astype(np.int32)
    cos, sin = O.rope_tables(pos)
    lens = [int(c + L) for c, L in zip(cached, chunk)]
    num_pages = sum((n + P - 1) // P for n in lens) + 3
    table = H.random_block_table(rng, lens, P, num_pages)
    table[3, 0] = table[2, 0]  # unused entry: any valid page
    cache = H.random_filled_cache(rng, num_pages, P)
    cache.k_calibration[...] = (0.5 + 2 * rng.random(cache.k_calibration.shape)).astype(np.float32)
    dev_cache = H.cache_to_torch(cache)
    q, k, v = np_views(qkv)
    want_qp, want_kp = O.norm_rope_prefill(q, k, qw, kw, cos, sin, 1e-6)
    O.quantize_prefill(want_kp, v, cu, table, cached, 2, cache)

    tq, tk, tv = split_views(H.bf16_tensor(qkv))
    if fused:
        got_qp, got_kp = K.write_prefill(tq, tk, tv, H.bf16_tensor(qw), H.bf16_tensor(kw), H.bf16_tensor(cos)[:, None, :],
                                         H.bf16_tensor(sin)[:, None, :], H.i32(cu), H.i32(table), H.i32(cached), H.i32([2]),
                                         dev_cache, 1e-6)
    else:
        got_qp, got_kp = K.fused_norm_rope_prefill(tq, tk, H.bf16_tensor(qw), H.bf16_tensor(kw), H.bf16_tensor(cos)[:, None, :],
                                                   H.bf16_tensor(sin)[:, None, :], 1e-6)
    assert np.array_equal(H.to_bits(got_qp), O.bf16_bits(want_qp))
    assert np.array_equal(H.to_bits(got_kp), O.bf16_bits(want_kp))
    if not fused:
        K.quantize_kv_prefill(got_kp, tv, H.i32(cu), H.i32(table), H.i32(cached), H.i32([2]), dev_cache)
    H.assert_cache_equal(H.cache_to_numpy(dev_cache), cache, f"T={T} first={first_chunk} ")

    # dequantize what is now cached for the prefilling entry (prior + T tokens)
    cu_cached = np.array([0, 0, 0, prior + T, prior + T], np.int32)
    want_k = np.zeros((HKV, prior + T + 5, D), np.float32)
    want_v = np.zeros_like(want_k)
    O.dequantize_prefix(cache, cu_cached, table, want_k, want_v)
    got_k = torch.zeros(want_k.shape, dtype=torch.bfloat16, device="cuda")
    got_v = torch.zeros_like(got_k)
    K.dequantize_kv_prefix(dev_cache, H.i32(cu_cached), H.i32(table), got_k, got_v)
    assert np.array_equal(H.to_bits(got_k), O.bf16_bits(want_k))
    assert np.array_equal(H.to_bits(got_v), O.bf16_bits(want_v))
    assert K.check_status() == 0


def test_quantizer_known_answers(K):
    """Hand-made rows through the decode write's V branch (no norm/rope): all zeros -> scale
    1e-6/127 and zero codes; +-absmax -> +-127 (never -128); exact .5 ties round to even."""
    T = 4
    v = np.zeros((T, HKV, D), np.float32)
    v[1, :, 0], v[1, :, 1] = 2.0, -2.0  # absmax elements
    v[2, :, 0] = 127.0  # scale = 1: x/scale = x
    v[2, :, 1:5] = [2.5, 3.5, -2.5, -0.5]  # ties -> 2, 4, -2, -0
    v[3, :, 0] = 1e-30  # far below the scale floor
    v = O.bf16_round(v)
    cache = O.make_cache(T, HKV, 16, D)
    dev_cache = H.cache_to_torch(cache)
    qk = np.zeros((T, HQ + HKV, D), np.float32)
    qk[..., 0] = 1.0
    ones = np.ones(D, np.float32)
    cos, sin = O.rope_tables(np.zeros(T, np.int32))
    table = np.arange(T, dtype=np.int32)[:, None]
    lens = np.zeros(T, np.int32)
    O.write_decode(qk[:, :HQ], qk[:, HQ:], v, ones, ones, cos, sin, table, cache, lens, T, 1e-6)
    K.fused_rope_kv_decode(H.bf16_tensor(qk[:, :HQ]), H.bf16_tensor(qk[:, HQ:]), H.bf16_tensor(v), H.bf16_tensor(ones),
                           H.bf16_tensor(ones), H.bf16_tensor(cos)[:, None, :], H.bf16_tensor(sin)[:, None, :],
                           H.i32(table), dev_cache, H.i32(lens), H.i32([T]), 1e-6)
    got = H.cache_to_numpy(dev_cache)
    H.assert_cache_equal(got, cache, "known answers ")
    assert got.v_scale[0, 0, 0] == np.float32(1e-6) / np.float32(127) and not got.v[0].any()
    assert got.v[1, 0, 0, 0] == 127 and got.v[1, 0, 0, 1] == -127
    assert list(got.v[2, 0, 0, :5]) == [127, 2, 4, -2, 0] and got.v_scale[2, 0, 0] == np.float32(1.0)
    assert got.v.min() >= -127


def test_bad_page_sets_status_and_skips(K):
    """An out-of-range page id is reported through the status word and nothing is written."""
    rng = np.random.default_rng(5)
    qkv, qw, kw, pos, cos, sin = make_write_inputs(rng, 2)
    cache = O.make_cache(3, HKV, 16, D)
    dev_cache = H.cache_to_torch(cache)
    table = np.array([[0], [99]], np.int32)
    tq, tk, tv = split_views(H.bf16_tensor(qkv))
    K.fused_rope_kv_decode(tq, tk, tv, H.bf16_tensor(qw), H.bf16_tensor(kw), H.bf16_tensor(cos)[:, None, :],
                           H.bf16_tensor(sin)[:, None, :], H.i32(table), dev_cache, H.i32([3, 3]), H.i32([2]), 1e-6)
    assert K.check_status() & 1
    got = H.cache_to_numpy(dev_cache)
    assert got.k[0, :, 3].any() and not got.k[1:].any()
