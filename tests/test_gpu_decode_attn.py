"""GPU parity of split-K paged decode attention (C ABI via the drop-in Python API) against the
CPU oracle (dequantize, fp32 softmax) and against the reference kernel's own output."""
import numpy as np
import pytest
import torch

from oracle import oracle as O
from tests import helpers as H
from tests.helpers import D, HKV, HQ

pytestmark = pytest.mark.gpu
SCALE = D ** -0.5
# Gate stated for the path: max-abs 2e-2, mean-abs 2e-3 (relative to max(1,|want|), see helpers).
# Tight gate: the kernel keeps P*v_scale in fp16 and everything else in fp32, so it must sit
# well inside one bf16 output ulp of the fp32 oracle.
GATE, TIGHT = (2e-2, 2e-3), (8e-3, 4e-4)


@pytest.fixture(scope="module")
def K():
    from inference_engine_b200 import kernels

    return kernels


def run_case(K, rng, lens, page_size, paged, variant=0, gauss=False, nd=None, extra_pages=3):
    B = len(lens)
    nd = B if nd is None else nd
    if paged:
        num_pages = sum((n + page_size - 1) // page_size for n in lens) + extra_pages
        table = H.random_block_table(rng, lens, page_size, num_pages)
    else:
        num_pages = B + 1
        table = rng.permutation(num_pages)[:B].astype(np.int32)
    cache = H.random_filled_cache(rng, num_pages, page_size, gauss=gauss)
    q = H.randn_bf16(rng, B, HQ, D)
    cached = np.array([n - 1 for n in lens], np.int32)
    want = O.decode_attention(q, cache, cached, table, nd, SCALE)
    out = torch.full((B, HQ, D), 7.0, dtype=torch.bfloat16, device="cuda")
    K.decode_attention(H.bf16_tensor(q), H.cache_to_torch(cache), H.i32(cached), H.i32(table), H.i32([nd]), SCALE,
                       out=out, variant=variant)
    got = H.to_f32(out)
    assert K.check_status() == 0
    assert np.all(got[nd:] == 7.0), "rows of non-decoding entries must not be written"
    return got[:nd], want[:nd]


def check(got, want, tight=TIGHT):
    assert np.isfinite(got).all()
    mx, mean = H.attn_errors(got, want)
    assert mx <= GATE[0] and mean <= GATE[1], (mx, mean)
    assert mx <= tight[0] and mean <= tight[1], (mx, mean)


@pytest.mark.parametrize("variant", [0, 1])
def test_reference_golden(K, golden, variant):
    g = golden
    cache = O.KVCache(g["da_k"], g["da_v"], g["da_k_scale"], g["da_v_scale"], g["da_k_calibration"])
    nd = int(g["da_nd"][0])
    out = K.decode_attention(H.bits_tensor(g["da_q_bf16"]), H.cache_to_torch(cache), H.i32(g["da_cached"]),
                             H.i32(g["da_slots"]), H.i32(g["da_nd"]), SCALE, variant=variant)
    want = O.from_bf16_bits(g["da_out_bf16"])
    mx, mean = H.attn_errors(H.to_f32(out)[:nd], want)
    # the reference rounds P*v_scale to bf16 (kernels.py:186); that alone is ~one bf16 ulp
    assert mx <= 8e-3 and mean <= 1.5e-3, (mx, mean)
    check(H.to_f32(out)[:nd], O.decode_attention(O.from_bf16_bits(g["da_q_bf16"]), cache, g["da_cached"], g["da_slots"], nd, SCALE)[:nd])


@pytest.mark.parametrize("variant", [0, 1, 2])
@pytest.mark.parametrize("paged", [True, False])
def test_boundaries(K, variant, paged):
    """Context lengths on every tile, page and split boundary, in both cache layouts."""
    rng = np.random.default_rng(10 + variant + 2 * int(paged))
    lens = [1, 2, 15, 16, 17, 31, 32, 33, 63, 64, 65, 127, 128, 129, 130, 255, 256, 257, 1000]
    got, want = run_case(K, rng, lens, 16 if paged else 1008, paged, variant)
    check(got, want)


@pytest.mark.parametrize("variant", [0, 1])
def test_quantized_gaussian_four_sequences(K, variant):
    """B=4, contexts 128..1024, N(0,1) K/V quantized per token per head, 16-token pages, permuted
    page table: the stated tolerance and the tight one."""
    rng = np.random.default_rng(0)
    got, want = run_case(K, rng, [128, 256, 512, 1024], 16, True, variant, gauss=True)
    err = np.abs(got - want)
    assert err.max() <= 2e-2 and err.mean() <= 2e-3
    assert err.max() <= 2e-3 and err.mean() <= 2e-4, (err.max(), err.mean())


@pytest.mark.parametrize("variant", [0, 2])
@pytest.mark.parametrize("B,n", [(1, 4096), (3, 2048), (64, 512), (256, 128), (37, 700)])
def test_split_shapes(K, B, n, variant):
    """Shapes where sequences are split over many warps (B small) and where one warp owns many
    sequences (B large)."""
    rng = np.random.default_rng(B * 100003 + n)
    got, want = run_case(K, rng, [n] * B, 16, True, variant, gauss=True)
    err = np.abs(got - want)
    # outputs are below 1 in magnitude: 4e-3 is one bf16 ulp there (a rounding flip), the mean is the real gate
    assert err.max() <= 4e-3 and err.mean() <= 1e-4, (err.max(), err.mean())


def test_ragged_batch_and_page_sizes(K):
    rng = np.random.default_rng(77)
    lens = [int(x) for x in rng.integers(1, 3000, 23)]
    for page_size in (16, 64, 256):
        got, want = run_case(K, rng, lens, page_size, True, 0)
        check(got, want)


def test_num_decoding_subset_and_zero(K):
    rng = np.random.default_rng(3)
    got, want = run_case(K, rng, [100, 200, 300, 400], 16, True, 0, nd=2)
    check(got, want)
    got, want = run_case(K, rng, [100, 200], 16, True, 0, nd=0)
    assert got.shape[0] == 0


def test_batch_invariance_of_unsplit_sequences(K):
    """A sequence whose tiles all land in one warp gives the same bits alone and inside a batch of
    equal sequences (the work split depends only on the batch's tile count)."""
    rng = np.random.default_rng(9)
    P, n = 16, 64
    cache = H.random_filled_cache(rng, 40, P, gauss=True)
    q = H.randn_bf16(rng, 8, HQ, D)
    table = H.random_block_table(rng, [n] * 8, P, 40)
    cached = np.full(8, n - 1, np.int32)
    dev = H.cache_to_torch(cache)
    full = K.decode_attention(H.bf16_tensor(q), dev, H.i32(cached), H.i32(table), H.i32([8]), SCALE)
    one = K.decode_attention(H.bf16_tensor(q[3:4]), dev, H.i32(cached[3:4]), H.i32(table[3:4]), H.i32([1]), SCALE)
    assert torch.equal(full[3], one[0])


def test_one_hot_values_reveal_attended_tokens(K):
    """V = scale * one-hot(token index mod 128): the output is the softmax mass per residue, so a
    token skipped or read twice shows up; a single huge score makes it a one-hot."""
    rng = np.random.default_rng(21)
    n, P = 300, 16
    cache = O.make_cache(32, HKV, P, D)
    table = H.random_block_table(rng, [n], P, 32)
    pages, rows = O.locate(cache, table, 0, np.arange(n))
    cache.k[...] = rng.integers(-20, 21, cache.k.shape, dtype=np.int8)
    cache.k_scale[...] = 0.01
    cache.v_scale[...] = 1.0 / 127
    for t in range(n):
        cache.v[pages[t], :, rows[t], t % D] = 127
    q = H.randn_bf16(rng, 1, HQ, D)
    cached = np.array([n - 1], np.int32)
    want = O.decode_attention(q, cache, cached, table, 1, SCALE)
    got = H.to_f32(K.decode_attention(H.bf16_tensor(q), H.cache_to_torch(cache), H.i32(cached), H.i32(table), H.i32([1]), SCALE))
    check(got, want)
    assert np.allclose(got.sum(-1), 1.0, atol=2e-2)
    # one dominant key: token 77 for every head
    cache.k[pages[77], :, rows[77], :] = np.sign(O.bf16_round(q[0, ::2])).astype(np.int8) * 127
    cache.k_scale[pages[77], :, rows[77]] = 1.0
    q2 = np.repeat(q[0, ::2], 2, axis=0)[None]
    got = H.to_f32(K.decode_attention(H.bf16_tensor(q2), H.cache_to_torch(cache), H.i32(cached), H.i32(table), H.i32([1]), SCALE))
    assert np.all(got[0, :, 77] > 0.99)


def test_argument_validation(K):
    rng = np.random.default_rng(1)
    cache = H.cache_to_torch(H.random_filled_cache(rng, 4, 24))  # 24-token pages: not a multiple of 16
    q = H.bf16_tensor(H.randn_bf16(rng, 2, HQ, D))
    table = H.i32([[0, 1], [2, 3]])
    with pytest.raises(ValueError):
        K.decode_attention(q, cache, H.i32([30, 30]), table, H.i32([2]), SCALE)
    with pytest.raises(RuntimeError):
        K.decode_attention(q.cpu(), cache, H.i32([30, 30]), table, H.i32([2]), SCALE)


def test_repeated_calls_leave_the_workspace_reusable(K):
    """The arrival counters must be back at zero after every call: the same inputs give the same
    bits on three consecutive calls, and a different batch in between does not disturb them."""
    rng = np.random.default_rng(5)
    lens = [3000, 70, 1500, 16]
    table = H.random_block_table(rng, lens, 16, 300)
    cache = H.cache_to_torch(H.random_filled_cache(rng, 300, 16, gauss=True))
    q = H.bf16_tensor(H.randn_bf16(rng, 4, HQ, D))
    cached, tab, nd = H.i32([n - 1 for n in lens]), H.i32(table), H.i32([4])
    first = K.decode_attention(q, cache, cached, tab, nd, SCALE).clone()
    K.decode_attention(q[:2], cache, cached[:2], tab[:2], H.i32([2]), SCALE)
    for _ in range(2):
        again = K.decode_attention(q, cache, cached, tab, nd, SCALE)
        assert torch.equal(first, again)
    ws = K.decode_workspace(q.device, 4, HQ, HKV, 1)
    counters = ws[: 4096].view(torch.int32)
    torch.cuda.synchronize()
    assert int(counters[64:128].abs().sum()) == 0  # the arrival counters follow the 256-byte prefix area


def test_early_start_after_quantize_on_write(K):
    """Decode attention launched with programmatic early start right behind the write kernel whose
    new token it must see, several layers back to back on one stream: every layer's output must
    equal the oracle's, i.e. the kernel really waited for the write before reading the cache."""
    rng = np.random.default_rng(17)
    lens = [257, 16, 1000, 64, 3]
    B, P, layers = len(lens), 16, 4
    pages = sum((n + P - 1) // P for n in lens) + 2
    table = H.random_block_table(rng, lens, P, pages)
    cached = np.array([n - 1 for n in lens], np.int32)
    cos, sin = O.rope_tables(cached)
    w = O.bf16_round((1 + 0.02 * rng.standard_normal(D)).astype(np.float32))
    caches, dev_caches, qkvs, wants = [], [], [], []
    for _ in range(layers):
        cache = H.random_filled_cache(rng, pages, P, gauss=True)
        dev_caches.append(H.cache_to_torch(cache))
        qkv = H.randn_bf16(rng, B, (HQ + 2 * HKV) * D)
        q, k, v = (qkv[:, : HQ * D].reshape(B, HQ, D), qkv[:, HQ * D : (HQ + HKV) * D].reshape(B, HKV, D),
                   qkv[:, (HQ + HKV) * D :].reshape(B, HKV, D))
        qr = O.write_decode(q, k, v, w, w, cos, sin, table, cache, cached, B, 1e-6)
        wants.append(O.decode_attention(qr, cache, cached, table, B, SCALE))
        qkvs.append(H.bf16_tensor(qkv))
    tw, tcos, tsin = H.bf16_tensor(w), H.bf16_tensor(cos)[:, None, :], H.bf16_tensor(sin)[:, None, :]
    ttab, tcl, tnd = H.i32(table), H.i32(cached), H.i32([B])
    K.set_early_start(True)
    try:
        for rep in range(3):
            outs = []
            for l in range(layers):
                tq, tk, tv = qkvs[l].split([HQ * D, HKV * D, HKV * D], dim=-1)
                qr = K.fused_rope_kv_decode(tq.view(B, HQ, D), tk.view(B, HKV, D), tv.view(B, HKV, D), tw, tw, tcos, tsin,
                                            ttab, dev_caches[l], tcl, tnd, 1e-6)
                outs.append(K.decode_attention(qr, dev_caches[l], tcl, ttab, tnd, SCALE))
            torch.cuda.synchronize()
            for l in range(layers):
                check(H.to_f32(outs[l]), wants[l])
    finally:
        K.set_early_start(False)
    assert K.check_status() == 0
