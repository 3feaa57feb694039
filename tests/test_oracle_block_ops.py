"""The oracle's restatement of the decoder block's element-wise ops against vectors produced by the
reference's own kernels (tests/golden/make_golden_block_ops.py)."""
import os

import numpy as np
import pytest

from oracle import oracle as O

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "reference_block_ops.npz")


@pytest.fixture(scope="module")
def g():
    return dict(np.load(GOLD))


def ulps(a_bits, b_bits):
    """Distance in bf16 steps between two arrays of bf16 bit patterns (same sign assumed where it matters)."""
    def key(u):
        u = u.astype(np.int32)
        return np.where(u & 0x8000, 0x8000 - (u & 0x7FFF) - 1, 0x8000 + (u & 0x7FFF))
    return np.abs(key(a_bits) - key(b_bits))


def test_silu_mul(g):
    got = O.bf16_bits(O.silu_mul(O.from_bf16_bits(g["sm_in_bf16"])))
    d = ulps(got, g["sm_out_bf16"])
    # exp differs in the last place between libraries: at most one bf16 step, and rarely
    assert d.max() <= 1 and (d > 0).mean() < 0.01, (d.max(), (d > 0).mean())


def test_add_rms_norm(g):
    res, normed = O.add_rms_norm(O.from_bf16_bits(g["arn_res_bf16"]), O.from_bf16_bits(g["arn_delta_bf16"]),
                                 O.from_bf16_bits(g["arn_w_bf16"]), 1e-6)
    assert np.array_equal(O.bf16_bits(res), g["arn_new_res_bf16"])  # the residual stream is exact
    d = ulps(O.bf16_bits(normed), g["arn_normed_bf16"])
    assert d.max() <= 1 and (d > 0).mean() < 0.01, (d.max(), (d > 0).mean())
