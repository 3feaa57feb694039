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


def test_reference_golden(K, golden):
    g = golden
    v = O.from_bf16_bits(g["pf_qkv_bf16"])[:, (HQ + HKV) * D :].reshape(-1, HKV, D)
    nd = int(g["pf_nd"][0])
    out = K.prefill_attention(H.bits_tensor(g["pf_q_p_bf16"]), H.bits_tensor(g["pf_k_p_bf16"]), H.bf16_tensor(v),
                              H.i32(g["pf_seq_ids"]), H.i32(g["pf_cu"]), H.i32(g["pf_tile_start"]),
                              H.bits_tensor(g["pf_k_prefix_bf16"]), H.bits_tensor(g["pf_v_prefix_bf16"]),
                              H.i32(g["pf_cu_cached"]), int(g["pf_block_m"][0]))
    lo = int(g["pf_cu"][nd])
    mx, mean = H.attn_errors(H.to_f32(out)[lo:], O.from_bf16_bits(g["pf_attn_out_bf16"])[lo:])
    assert mx <= 8e-3 and mean <= 4e-4, (mx, mean)


@pytest.mark.parametrize("block_m", [16, 128])
def test_random_mixed_batch(K, block_m):
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
                              H.i32(tiles), H.bf16_tensor(k_pre), H.bf16_tensor(v_pre), H.i32(cu_cached), block_m)
    mx, mean = H.attn_errors(H.to_f32(out)[nd:], want[nd:])
    assert mx <= 2e-2 and mean <= 2e-3
    assert mx <= 8e-3 and mean <= 4e-4, (mx, mean)
