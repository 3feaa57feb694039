"""GPU parity of chunked-prefill attention against the reference kernel's output (golden) and
the CPU oracle."""
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


@pytest.mark.parametrize("variant", [0, 1, 2])
def test_reference_golden(K, golden, variant):
    g = golden
    v = O.from_bf16_bits(g["pf_qkv_bf16"])[:, (HQ + HKV) * D :].reshape(-1, HKV, D)
    nd = int(g["pf_nd"][0])
    out = K.prefill_attention(H.bits_tensor(g["pf_q_p_bf16"]), H.bits_tensor(g["pf_k_p_bf16"]), H.bf16_tensor(v),
                              H.i32(g["pf_seq_ids"]), H.i32(g["pf_cu"]), H.i32(g["pf_tile_start"]),
                              H.bits_tensor(g["pf_k_prefix_bf16"]), H.bits_tensor(g["pf_v_prefix_bf16"]),
                              H.i32(g["pf_cu_cached"]), int(g["pf_block_m"][0]), variant=variant)
    assert K.check_status() == 0
    lo = int(g["pf_cu"][nd])
    mx, mean = H.attn_errors(H.to_f32(out)[lo:], O.from_bf16_bits(g["pf_attn_out_bf16"])[lo:])
    assert mx <= 8e-3 and mean <= 4e-4, (mx, mean)


@pytest.mark.parametrize("variant", [1, 2])
@pytest.mark.parametrize("block_m", [16, 128])
def test_random_mixed_batch(K, block_m, variant):
    """Two decoding rows, a 200-row chunk on a 300-token prefix, a 77-row first chunk, padding."""
    rng = np.random.default_rng(31 + block_m)
    chunk = [1, 1, 200, 77, 9, 0]
    prefix = [0, 0, 300, 0, 0, 0]
    nd = 2
    N = sum(chunk)
    cu = np.concatenate([[0], np.cumsum(chunk)]).astype(np.int32)
    cu_cached = np.concatenate([[0], np.cumsum(prefix)]).astype(np.int32)
    seq_ids = np.concatenate([np.full(L, b) for b, L in enumerate(chunk)]).astype(np.int32)
    q, k, v = H.randn_bf16(rng, N, HQ, D), H.randn_bf16(rng, N, HKV, D), H.randn_bf16(rng, N, HKV, D)
    k_pre, v_pre = H.randn_bf16(rng, HKV, 300 + 4, D), H.randn_bf16(rng, HKV, 300 + 4, D)
    tiles = [r for b in range(nd, len(chunk)) for r in range(cu[b], cu[b + 1], block_m)] + [-1, -1]
    want = O.prefill_attention(q, k, v, cu, k_pre, v_pre, cu_cached, nd)
    out = K.prefill_attention(H.bf16_tensor(q), H.bf16_tensor(k), H.bf16_tensor(v), H.i32(seq_ids), H.i32(cu),
                              H.i32(tiles), H.bf16_tensor(k_pre), H.bf16_tensor(v_pre), H.i32(cu_cached), block_m,
                              variant=variant)
    assert K.check_status() == 0
    mx, mean = H.attn_errors(H.to_f32(out)[nd:], want[nd:])
    assert mx <= 2e-2 and mean <= 2e-3
    assert mx <= 8e-3 and mean <= 4e-4, (mx, mean)


@pytest.mark.parametrize("variant", [1, 2])
@pytest.mark.parametrize("prior", [0, 333])
def test_long_chunk_on_prefix(K, prior, variant):
    """One 700-row chunk (block_m 128: five full tiles and a ragged one) on a prefix that is not a
    multiple of the key block, plus a decoding row and a padding entry; strided q/k/v views of one
    projection buffer as the engine passes them."""
    rng = np.random.default_rng(900 + prior)
    chunk, prefix, nd = [1, 700, 67, 0], [0, prior, 0, 0], 1
    N = sum(chunk)
    cu = np.concatenate([[0], np.cumsum(chunk)]).astype(np.int32)
    cu_cached = np.concatenate([[0], np.cumsum(prefix)]).astype(np.int32)
    seq_ids = np.concatenate([np.full(L, b) for b, L in enumerate(chunk)]).astype(np.int32)
    qkv = H.randn_bf16(rng, N, (HQ + 2 * HKV) * D)
    q = qkv[:, : HQ * D].reshape(N, HQ, D)
    k = qkv[:, HQ * D : (HQ + HKV) * D].reshape(N, HKV, D)
    v = qkv[:, (HQ + HKV) * D :].reshape(N, HKV, D)
    k_pre, v_pre = H.randn_bf16(rng, HKV, prior + 8, D), H.randn_bf16(rng, HKV, prior + 8, D)
    tiles = [r for b in range(nd, len(chunk)) for r in range(cu[b], cu[b + 1], 128)] + [-1, -1]
    want = O.prefill_attention(q, k, v, cu, k_pre, v_pre, cu_cached, nd)
    t = H.bf16_tensor(qkv)
    tq, tk, tv = t.split([HQ * D, HKV * D, HKV * D], dim=-1)
    out = K.prefill_attention(tq.view(N, HQ, D), tk.view(N, HKV, D), tv.view(N, HKV, D), H.i32(seq_ids), H.i32(cu),
                              H.i32(tiles), H.bf16_tensor(k_pre), H.bf16_tensor(v_pre), H.i32(cu_cached), 128,
                              variant=variant)
    assert K.check_status() == 0
    mx, mean = H.attn_errors(H.to_f32(out)[nd:], want[nd:])
    assert mx <= 8e-3 and mean <= 4e-4, (mx, mean)


@pytest.mark.parametrize("variant", [1, 2])
def test_rows_behind_the_prefix_are_never_used(K, variant):
    """The prefix scratch is uninitialised behind the last entry's rows (the engine allocates it with
    torch.empty): NaNs there must not reach any output, also when the prefix ends inside a key block."""
    rng = np.random.default_rng(4242)
    chunk, prefix, nd = [150, 40], [200, 70], 0
    N = sum(chunk)
    cu = np.concatenate([[0], np.cumsum(chunk)]).astype(np.int32)
    cu_cached = np.concatenate([[0], np.cumsum(prefix)]).astype(np.int32)
    seq_ids = np.concatenate([np.full(L, b) for b, L in enumerate(chunk)]).astype(np.int32)
    q, k, v = H.randn_bf16(rng, N, HQ, D), H.randn_bf16(rng, N, HKV, D), H.randn_bf16(rng, N, HKV, D)
    k_pre, v_pre = H.randn_bf16(rng, HKV, 270 + 200, D), H.randn_bf16(rng, HKV, 270 + 200, D)
    want = O.prefill_attention(q, k, v, cu, k_pre, v_pre, cu_cached, nd)
    k_pre[:, 270:], v_pre[:, 270:] = np.nan, np.nan
    tiles = [r for b in range(len(chunk)) for r in range(cu[b], cu[b + 1], 128)] + [-1]
    out = K.prefill_attention(H.bf16_tensor(q), H.bf16_tensor(k), H.bf16_tensor(v), H.i32(seq_ids), H.i32(cu),
                              H.i32(tiles), H.bf16_tensor(k_pre), H.bf16_tensor(v_pre), H.i32(cu_cached), 128,
                              variant=variant)
    assert K.check_status() == 0
    got = H.to_f32(out)
    assert np.isfinite(got).all()
    mx, mean = H.attn_errors(got, want)
    assert mx <= 8e-3 and mean <= 4e-4, (mx, mean)


@pytest.mark.parametrize("seed", range(24))
def test_tcgen05_kernel_agrees_with_mma_kernel_on_random_batches(K, seed):
    """Random packed batches (chunk lengths 1..700, prefixes 0..900, 1..5 prefilling entries, decoding rows and a
    padding entry in front / behind, block_m 64 / 128 / 256, GQA groups of 1, 2, 4 and 8): the tcgen05 kernel
    against the mma.sync kernel, which the oracle tests pin.  Exercises every count of key blocks per warpgroup
    (0, 1, 2, 3, many), ragged last tiles and prefixes that end inside a key block."""
    rng = np.random.default_rng(1000 + seed)
    block_m = int(rng.choice([64, 128, 256]))
    hkv = int(rng.choice([1, 2, 4, 8]))
    hq = hkv * int(rng.choice([1, 2, 4, 8]))
    while hq > 16:
        hq //= 2
    nd = int(rng.integers(0, 3))
    npf = int(rng.integers(1, 6))
    small = seed % 3 == 0  # every third case: only short chunks and prefixes (few key blocks)
    chunk = [1] * nd + [int(rng.integers(1, 60 if small else 700)) for _ in range(npf)] + [int(rng.integers(0, 40))]
    prefix = [0] * nd + [int(rng.choice([0, rng.integers(1, 130 if small else 900)])) for _ in range(npf)] + [0]
    N = sum(chunk)
    cu = np.concatenate([[0], np.cumsum(chunk)]).astype(np.int32)
    cu_cached = np.concatenate([[0], np.cumsum(prefix)]).astype(np.int32)
    seq_ids = np.concatenate([np.full(L, b) for b, L in enumerate(chunk)]).astype(np.int32)
    q, k, v = H.randn_bf16(rng, N, hq, D), H.randn_bf16(rng, N, hkv, D), H.randn_bf16(rng, N, hkv, D)
    cap = int(cu_cached[-1]) + int(rng.integers(1, 70))
    k_pre, v_pre = H.randn_bf16(rng, hkv, cap, D), H.randn_bf16(rng, hkv, cap, D)
    tiles = [r for b in range(nd, len(chunk)) for r in range(cu[b], cu[b + 1], block_m)] + [-1] * int(rng.integers(0, 4))
    args = (H.bf16_tensor(q), H.bf16_tensor(k), H.bf16_tensor(v), H.i32(seq_ids), H.i32(cu), H.i32(tiles),
            H.bf16_tensor(k_pre), H.bf16_tensor(v_pre), H.i32(cu_cached), block_m)
    a = K.prefill_attention(*args, variant=1)
    b = K.prefill_attention(*args, variant=2)
    assert K.check_status() == 0
    lo = int(cu[nd])
    ga, gb = H.to_f32(a)[lo:], H.to_f32(b)[lo:]
    assert np.isfinite(gb).all()
    mx, mean = H.attn_errors(gb, ga)
    assert mx <= 1.6e-2 and mean <= 6e-4, (mx, mean)  # two bf16 roundings of the same fp32 value: one step apart at most


def test_bounded_waits_run_out_cleanly(K):
    """variant 3: the tcgen05 kernel with idle issuing warps and short wait limits.  Every wait inside the kernel
    gives up; the call must return, report B200KV_S_TIMEOUT (4) in the status word, write no output row and leave
    the GPU in a state where the next call works."""
    from inference_engine_b200 import _lib

    rng = np.random.default_rng(77)
    chunk, prefix = [300, 0], [200, 0]
    N = sum(chunk)
    cu = np.concatenate([[0], np.cumsum(chunk)]).astype(np.int32)
    cu_cached = np.concatenate([[0], np.cumsum(prefix)]).astype(np.int32)
    q, k, v = H.randn_bf16(rng, N, HQ, D), H.randn_bf16(rng, N, HKV, D), H.randn_bf16(rng, N, HKV, D)
    k_pre, v_pre = H.randn_bf16(rng, HKV, 208, D), H.randn_bf16(rng, HKV, 208, D)
    tiles = list(range(0, N, 128)) + [-1]
    tq, tk, tv = H.bf16_tensor(q), H.bf16_tensor(k), H.bf16_tensor(v)
    tkp, tvp = H.bf16_tensor(k_pre), H.bf16_tensor(v_pre)
    out = torch.full((N, HQ, D), 7.0, dtype=torch.bfloat16, device="cuda")
    status = K.status_word(torch.device("cuda", 0))
    rc = _lib.load().b200kv_prefill_attn_variant(
        tq.data_ptr(), tq.stride(0), tq.stride(1), tk.data_ptr(), tk.stride(0), tk.stride(1), tv.data_ptr(), tv.stride(0),
        tv.stride(1), H.i32(np.zeros(N)).data_ptr(), H.i32(cu).data_ptr(), H.i32(tiles).data_ptr(), len(tiles), 128,
        tkp.data_ptr(), tvp.data_ptr(), tkp.stride(0), tkp.stride(1), 208, H.i32(cu_cached).data_ptr(), out.data_ptr(),
        out.stride(0), out.stride(1), N, HQ, HKV, D, 3, status.data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()
    assert K.check_status() == 4  # B200KV_S_TIMEOUT, and the word is cleared by the read
    assert torch.all(out == 7.0)
    # the same inputs through the working kernel
    want = O.prefill_attention(q, k, v, cu, k_pre, v_pre, cu_cached, 0)
    good = K.prefill_attention(tq, tk, tv, H.i32(np.zeros(N)), H.i32(cu), H.i32(tiles), tkp, tvp, H.i32(cu_cached), 128,
                               variant=2)
    assert K.check_status() == 0
    mx, mean = H.attn_errors(H.to_f32(good), want)
    assert mx <= 8e-3 and mean <= 4e-4, (mx, mean)
