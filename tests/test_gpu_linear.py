"""The weight-streaming matmul for few rows (b200kv_skinny_linear behind kernels.skinny_matmul / linear /
tune_linear) against the oracle's fp32 matmul and against the reference kernel's own outputs, at the five weight
shapes of the decoder (qkv, o, gate_up, down, lm_head) and at every cluster size each shape allows."""
import os

import numpy as np
import pytest
import torch

from oracle import oracle as O
from tests import helpers as H

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "reference_linear.npz")
SHAPES = {"qkv": (4096, 2048), "o": (2048, 2048), "gate_up": (12288, 2048), "down": (2048, 6144), "lm_head": (151936, 2048)}


@pytest.fixture(scope="module")
def K():
    from inference_engine_b200 import kernels

    return kernels


def close(got, want):
    """fp32 sums in another order: equal up to one bf16 step at the value's magnitude."""
    step = np.maximum(np.abs(want), 2.0 ** -6) * 2.0 ** -7
    bad = np.abs(got - want) > step
    assert not bad.any(), (int(bad.sum()), float(np.abs(got - want).max()))


def test_reference_golden(K):
    g = np.load(GOLD)
    for tag in "abc":
        x, w = H.bits_tensor(g[f"{tag}_x_bf16"]), H.bits_tensor(g[f"{tag}_w_bf16"])
        want = O.from_bf16_bits(g[f"{tag}_y_bf16"])
        for s in K.skinny_supported(x.shape[0], w.shape[0], w.shape[1]):
            close(H.to_f32(K.skinny_matmul(x, w, s)), want)
    assert K.check_status() == 0


@pytest.mark.parametrize("name", list(SHAPES))
@pytest.mark.parametrize("M", [1, 8, 17, 64])
def test_decoder_shapes(K, name, M):
    N, Kd = SHAPES[name]
    g = torch.Generator(device="cuda").manual_seed(N + M)
    w = (torch.randn(N, Kd, generator=g, device="cuda") * 0.02).to(torch.bfloat16)
    x = torch.randn(M, Kd, generator=g, device="cuda").to(torch.bfloat16)
    want = O.bf16_round((x.double() @ w.double().T).float().cpu().numpy())  # the oracle's formula, on the device for speed
    assert np.array_equal(want[:1, :256], O.linear(H.to_f32(x[:1]), H.to_f32(w[:256])))
    options = K.skinny_supported(M, N, Kd)
    assert options and options[0] == 1
    for s in options:
        y = K.skinny_matmul(x, w, s)
        torch.cuda.synchronize()
        close(H.to_f32(y), want)
    assert K.check_status() == 0


def test_strided_inputs_and_small_k(K):
    """x as a view into a wider buffer (rows 16-byte aligned), K of a single pipeline step, N of a single row block."""
    g = torch.Generator(device="cuda").manual_seed(5)
    buf = torch.randn(9, 64 + 192, generator=g, device="cuda").to(torch.bfloat16)
    x = buf[:, :64]
    w = torch.randn(128, 64, generator=g, device="cuda").to(torch.bfloat16)
    close(H.to_f32(K.skinny_matmul(x, w, 1)), O.linear(H.to_f32(x), H.to_f32(w)))
    with pytest.raises(ValueError):
        K.skinny_matmul(x, w, 2)  # a single K step cannot be split
    with pytest.raises(ValueError):
        K.skinny_matmul(buf[:, :96], torch.zeros(128, 96, device="cuda", dtype=torch.bfloat16), 1)  # K % 64
    assert K.check_status() == 0


def test_tune_linear_picks_per_shape_and_linear_dispatches(K):
    g = torch.Generator(device="cuda").manual_seed(9)
    w = (torch.randn(2048, 2048, generator=g, device="cuda") * 0.02).to(torch.bfloat16)
    K.use_skinny.clear()
    K.tune_linear([w], [1, 64, 128])
    assert (2048, 2048, 1) in K.use_skinny and (2048, 2048, 64) in K.use_skinny and (2048, 2048, 128) not in K.use_skinny
    for M in (1, 64, 128):
        x = torch.randn(M, 2048, generator=g, device="cuda").to(torch.bfloat16)
        close(H.to_f32(K.linear(x, w)), O.bf16_round((x.double() @ w.double().T).float().cpu().numpy()))
    # forcing each backend gives the same values up to summation order
    x = torch.randn(8, 2048, generator=g, device="cuda").to(torch.bfloat16)
    K.use_skinny[(2048, 2048, 8)] = 4
    a = K.linear(x, w)
    K.use_skinny[(2048, 2048, 8)] = 0
    b = K.linear(x, w)
    close(H.to_f32(a), H.to_f32(b))
    K.use_skinny.clear()
    assert K.check_status() == 0
