"""GPU parity of the decoder block's element-wise ops (silu_mul, add_rms_norm) against the reference kernels'
own outputs (golden) and against the CPU oracle on other shapes.  The residual stream must be exact; the
normalised / activated outputs may differ by one bf16 step where exp / rsqrt differ in their last place."""
import os

import numpy as np
import pytest
import torch

from oracle import oracle as O
from tests import helpers as H
from tests.test_oracle_block_ops import GOLD, ulps

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def K():
    from inference_engine_b200 import kernels

    return kernels


def close(got_bits, want_bits, frac=0.01):
    d = ulps(got_bits, want_bits)
    assert d.max() <= 1 and (d > 0).mean() < frac, (int(d.max()), float((d > 0).mean()))


def test_reference_golden(K):
    g = dict(np.load(GOLD))
    y = K.silu_mul(H.bits_tensor(g["sm_in_bf16"]))
    close(H.to_bits(y), g["sm_out_bf16"])
    r, n = K.add_rms_norm(H.bits_tensor(g["arn_res_bf16"]), H.bits_tensor(g["arn_delta_bf16"]),
                          H.bits_tensor(g["arn_w_bf16"]), 1e-6)
    assert np.array_equal(H.to_bits(r), g["arn_new_res_bf16"])
    close(H.to_bits(n), g["arn_normed_bf16"])


@pytest.mark.parametrize("N,D", [(1, 8), (3, 2048), (33, 6144), (1024, 2048), (2, 8192)])
def test_add_rms_norm_vs_oracle(K, N, D):
    rng = np.random.default_rng(N * 7 + D)
    res, delta = H.randn_bf16(rng, N, D) * 4, H.randn_bf16(rng, N, D)
    res = O.bf16_round(res)
    w = O.bf16_round((1 + 0.1 * rng.standard_normal(D)).astype(np.float32))
    want_r, want_n = O.add_rms_norm(res, delta, w, 1e-6)
    r, n = K.add_rms_norm(H.bf16_tensor(res), H.bf16_tensor(delta), H.bf16_tensor(w), 1e-6)
    assert np.array_equal(H.to_bits(r), O.bf16_bits(want_r))
    close(H.to_bits(n), O.bf16_bits(want_n))


@pytest.mark.parametrize("N,D", [(1, 8), (5, 1536), (64, 6144), (7, 12288)])
def test_silu_mul_vs_oracle_strided(K, N, D):
    rng = np.random.default_rng(N + D)
    buf = O.bf16_round(H.randn_bf16(rng, N, 2 * D + 64) * 3)
    t = H.bf16_tensor(buf)[:, : 2 * D]  # a strided view, like a slice of a wider projection
    y = K.silu_mul(t)
    close(H.to_bits(y), O.bf16_bits(O.silu_mul(buf[:, : 2 * D])))


def test_argument_checks(K):
    x = torch.zeros(4, 2 * 12, dtype=torch.bfloat16, device="cuda")  # D = 12: not a multiple of 8
    with pytest.raises(ValueError):
        K.silu_mul(x)
    big = torch.zeros(2, 8200, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(ValueError):
        K.add_rms_norm(big, big, torch.ones(8200, dtype=torch.bfloat16, device="cuda"), 1e-6)
