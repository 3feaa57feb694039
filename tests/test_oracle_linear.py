"""The oracle's matmul against the reference's skinny_matmul kernel (run unmodified under Triton's interpreter by
tests/golden/make_golden_linear.py): equal up to the last bf16 bit, which the order of the fp32 sums decides."""
import os

import numpy as np

from oracle import oracle as O

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "reference_linear.npz")


def test_linear_matches_the_reference_kernel():
    g = np.load(GOLD)
    for tag in "abc":
        x, w = O.from_bf16_bits(g[f"{tag}_x_bf16"]), O.from_bf16_bits(g[f"{tag}_w_bf16"])
        want = O.from_bf16_bits(g[f"{tag}_y_bf16"])
        got = O.linear(x, w)
        step = np.maximum(np.abs(want), 2.0 ** -6) * 2.0 ** -7  # one bf16 step at the value's magnitude
        assert np.all(np.abs(got - want) <= step), (tag, float(np.abs(got - want).max()))
        assert np.mean(got == want) > 0.9, tag
