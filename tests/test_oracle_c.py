"""The C restatement must agree with the numpy one: bit for bit on the quantizer and on
norm+rope, within fp32 summation noise on attention."""
import numpy as np

from oracle import c_oracle as C
from oracle import oracle as O
from tests import helpers as H


def test_quantizer_bit_equal():
    rng = np.random.default_rng(0)
    x = rng.standard_normal((300, 128)).astype(np.float32) * rng.uniform(1e-4, 50, (300, 1)).astype(np.float32)
    x[7] = 0
    x[8, :4] = [2.5, 3.5, -2.5, 127.0]
    c0, s0 = O.quantize_rows(x)
    c1, s1 = C.quantize_rows(x)
    assert np.array_equal(c0, c1) and np.array_equal(s0.view(np.uint32), s1.view(np.uint32))


def test_norm_rope_bit_equal():
    rng = np.random.default_rng(1)
    x = H.randn_bf16(rng, 40, 24, 128)
    w = O.bf16_round((1 + 0.02 * rng.standard_normal(128)).astype(np.float32))
    cos, sin = O.rope_tables(rng.integers(0, 32768, 40))
    a = O.norm_rope(x, w, cos, sin, 1e-6)
    b = C.norm_rope(x, w, cos, sin, 1e-6)
    assert np.array_equal(a.view(np.uint32), b.view(np.uint32))


def test_decode_attention_close():
    rng = np.random.default_rng(2)
    lens = [1, 17, 300, 64]
    table = H.random_block_table(rng, lens, 16, 40)
    cache = H.random_filled_cache(rng, 40, 16, gauss=True)
    q = H.randn_bf16(rng, 4, 16, 128)
    cached = np.array([n - 1 for n in lens], np.int32)
    a = O.decode_attention(q, cache, cached, table, 3, 128 ** -0.5)
    b = C.decode_attention(q, cache, cached, table, 3, 128 ** -0.5)
    assert np.all(b[3] == 0)
    assert np.abs(a - b).max() <= 2e-3  # at most one bf16 ulp of the small outputs
    assert C.threads() >= 1
