"""Parity at the sizes the benchmark quotes, not only at sizes the numpy oracle is quick at: the headline
sweep cell (64 sequences x 4096 tokens) and the two cells above it, the full-size chunked-prefill step
(32 decoding sequences + a 992-row chunk on 3072 cached tokens) and one GPU's share of the sequence-sharded
decode configuration (256 sequences, contexts log-uniform in [512, 32768]).  The checker is the
multi-threaded C restatement of the reference math (oracle/kvattn_oracle.c); caches are filled on the
device and copied back for it, so a case costs seconds."""
import os

import numpy as np
import pytest
import torch

from oracle import c_oracle as C
from oracle import oracle as O
from tests import helpers as H
from tests.helpers import D, HKV, HQ

pytestmark = pytest.mark.gpu
SCALE = D ** -0.5
PAGE = 16


@pytest.fixture(scope="module")
def K():
    from inference_engine_b200 import kernels

    return kernels


def device_cache(K, num_pages, gen, gauss_scales=True):
    """Random codes and positive scales, made on the device (a host-made 2 GB cache would take minutes)."""
    c = K.make_layer_cache(num_pages, HKV, PAGE, D, device="cuda")
    c.k.copy_(torch.randint(-127, 128, c.k.shape, generator=gen, device="cuda", dtype=torch.int8))
    c.v.copy_(torch.randint(-127, 128, c.v.shape, generator=gen, device="cuda", dtype=torch.int8))
    c.k_scale.copy_(0.01 + 0.03 * torch.rand(c.k_scale.shape, generator=gen, device="cuda"))
    c.v_scale.copy_(0.01 + 0.03 * torch.rand(c.v_scale.shape, generator=gen, device="cuda"))
    return c


def ragged_table(lens, seed):
    need = [(int(n) + PAGE - 1) // PAGE for n in lens]
    total = sum(need)
    perm = np.random.default_rng(seed).permutation(total).astype(np.int32)
    table = np.zeros((len(lens), max(need)), np.int32)
    at = 0
    for b, k in enumerate(need):
        table[b, :k] = perm[at:at + k]
        at += k
    return table, total


def check(got, want, gate=(2e-2, 2e-3), tight=(8e-3, 4e-4)):
    assert np.isfinite(got).all()
    mx, mean = H.attn_errors(got, want)
    assert mx <= gate[0] and mean <= gate[1], (mx, mean)  # the tolerance stated for the path
    assert mx <= tight[0] and mean <= tight[1], (mx, mean)  # one bf16 output step


@pytest.mark.parametrize("B", [64, 128, 256])
def test_sweep_cells_at_ctx_4096(K, B):
    """The cell the metric is quoted on and the two above it: ~74 tiles per warp, every sequence cut over
    3-4 warps, CTA-level pre-merge and the last-arriver merge all in one call.  Fused reduction, two-kernel
    reduction and the planned call against the oracle; the three must also agree bit for bit."""
    n = 4096
    gen = torch.Generator(device="cuda").manual_seed(64 + B)
    table, pages = ragged_table([n] * B, B)
    cache = device_cache(K, pages + 1, gen)
    q = torch.randn(B, HQ, D, generator=gen, device="cuda").to(torch.bfloat16)
    cached, nd, tab = H.i32([n - 1] * B), H.i32([B]), H.i32(table)
    C.set_threads(os.cpu_count() or 1)
    want = C.decode_attention(H.to_f32(q), H.cache_to_numpy(cache), np.full(B, n - 1, np.int32), table, B, SCALE)
    outs = []
    for variant, planned in ((0, False), (2, False), (0, True), (0, True)):
        out = torch.full((B, HQ, D), 7.0, dtype=torch.bfloat16, device="cuda")
        plan = K.plan_decode_step(cached, tab, nd, cache) if planned else None
        for _ in range(2):
            K.decode_attention(q, cache, cached, tab, nd, SCALE, out=out, variant=variant, plan=plan)
        torch.cuda.synchronize()
        assert K.check_status() == 0
        check(H.to_f32(out), want)
        outs.append(out)
    assert torch.equal(outs[2], outs[3]), "calls must be reproducible bit for bit"
    assert torch.equal(outs[0], outs[2]), "planned and unplanned calls share one work split"


def test_one_shard_of_the_sequence_sharded_decode(K):
    """256 sequences with contexts log-uniform in [512, 32768] (what one of eight GPUs serves of 2048), one layer
    (about 4 GB of cache, block-table rows of up to 2048 pages): quantize-on-write of the new tokens, bit-exact,
    then attention over the written cache, planned and unplanned."""
    rng = np.random.default_rng(4)
    B = 256
    lens = np.exp(rng.uniform(np.log(512), np.log(32768), B)).astype(np.int64)
    table, pages = ragged_table(lens, 4)
    gen = torch.Generator(device="cuda").manual_seed(4)
    cache = device_cache(K, pages + 1, gen)
    cached_np = (lens - 1).astype(np.int32)
    cached, nd, tab = H.i32(cached_np), H.i32([B]), H.i32(table)
    qkv = H.randn_bf16(rng, B, (HQ + 2 * HKV) * D)
    q, k, v = (qkv[:, : HQ * D].reshape(B, HQ, D), qkv[:, HQ * D : (HQ + HKV) * D].reshape(B, HKV, D),
               qkv[:, (HQ + HKV) * D :].reshape(B, HKV, D))
    w = O.bf16_round((1 + 0.02 * rng.standard_normal(D)).astype(np.float32))
    cos, sin = O.rope_tables(cached_np)

    host = H.cache_to_numpy(cache)  # before the write: the oracle writes the same rows into its copy
    want_q = O.write_decode(q, k, v, w, w, cos, sin, table, host, cached_np, B, 1e-6)
    t = H.bf16_tensor(qkv)
    tq, tk, tv = t.split([HQ * D, HKV * D, HKV * D], dim=-1)
    got_q = K.fused_rope_kv_decode(tq.view(B, HQ, D), tk.view(B, HKV, D), tv.view(B, HKV, D), H.bf16_tensor(w),
                                   H.bf16_tensor(w), H.bf16_tensor(cos)[:, None, :], H.bf16_tensor(sin)[:, None, :],
                                   tab, cache, cached, nd, 1e-6)
    assert np.array_equal(H.to_bits(got_q), O.bf16_bits(want_q)), "rotated q differs from the oracle"
    # the rows the write touched, gathered on the device and compared with the oracle's bytes
    page = torch.from_numpy(table[np.arange(B), cached_np // PAGE].astype(np.int64)).cuda()
    row = torch.from_numpy((cached_np % PAGE).astype(np.int64)).cuda()
    hp, hr = page.cpu().numpy(), row.cpu().numpy()
    for name in ("k", "v", "k_scale", "v_scale"):
        got = getattr(cache, name)[page, :, row].cpu().numpy()
        assert np.array_equal(got.view(np.uint8), getattr(host, name)[hp, :, hr].view(np.uint8)), name

    C.set_threads(os.cpu_count() or 1)
    want = C.decode_attention(want_q, host, cached_np, table, B, SCALE)
    plain = K.decode_attention(got_q, cache, cached, tab, nd, SCALE)
    planned = K.decode_attention(got_q, cache, cached, tab, nd, SCALE, plan=K.plan_decode_step(cached, tab, nd, cache))
    torch.cuda.synchronize()
    assert K.check_status() == 0
    check(H.to_f32(plain), want)
    assert torch.equal(plain, planned), "planned and unplanned calls share one work split"


@pytest.mark.parametrize("prior", [3072])
def test_full_size_chunked_prefill_step(K, prior):
    """The chunked-prefill configuration at full size through the six ops in the engine's call order: 32 decoding
    sequences with contexts ~U[128, 4096] and one 992-row chunk on `prior` cached tokens, 1024 packed rows, query
    tiles of 128 rows (the tcgen05 kernel), against the same composition of the oracle."""
    from inference_engine_b200 import scaffold as S

    rng = np.random.default_rng(3)
    n_dec, chunk, n_tokens = 32, 992, 1024
    ctx = [int(x) for x in rng.integers(128, 4097, n_dec)]
    plan = S.plan_step(ctx, [(prior, chunk)], n_tokens, n_dec + 2)
    table_t, pages = S.assign_pages(plan, PAGE, (4096 + PAGE) // PAGE + 1, generator=torch.Generator().manual_seed(3))
    table = table_t.numpy()
    E = n_dec + 2
    gen = torch.Generator(device="cuda").manual_seed(3)
    dev_cache = device_cache(K, pages, gen)
    # the entry that continues a prompt carries the calibration of its first chunk
    dev_cache.k_calibration[int(table[n_dec, 0])] = (0.5 + 1.5 * torch.rand(HKV, 1, D, generator=gen, device="cuda"))
    cache = H.cache_to_numpy(dev_cache)
    cache = O.KVCache(*(a.copy() for a in (cache.k, cache.v, cache.k_scale, cache.v_scale, cache.k_calibration)))
    q, k, v = H.randn_bf16(rng, n_tokens, HQ, D), H.randn_bf16(rng, n_tokens, HKV, D), H.randn_bf16(rng, n_tokens, HKV, D)
    qw = O.bf16_round((1 + 0.02 * rng.standard_normal(D)).astype(np.float32))
    kw = O.bf16_round((1 + 0.02 * rng.standard_normal(D)).astype(np.float32))
    cos, sin = O.rope_tables(np.asarray(plan["positions"], np.int32))
    cu, cached, cu_cached = plan["cu_seqlens"], plan["cached"], plan["cu_cached"]
    inp = S.upload_step(plan, table_t, [0] * n_tokens, "cuda", 128)
    cap = cu_cached[-1] + 8
    prefix = S.PrefixScratch(torch.full((HKV, cap, D), float("nan"), device="cuda", dtype=torch.bfloat16),
                             torch.full((HKV, cap, D), float("nan"), device="cuda", dtype=torch.bfloat16), inp.cu_cached)
    step_plan = K.plan_decode_step(inp.cached_lens, inp.block_table, inp.num_decoding, dev_cache)
    out = S.attention_ops(H.bf16_tensor(q), H.bf16_tensor(k), H.bf16_tensor(v), H.bf16_tensor(qw), H.bf16_tensor(kw),
                          H.bf16_tensor(cos)[:, None, :], H.bf16_tensor(sin)[:, None, :], dev_cache, inp,
                          inp.cached_lens, inp.block_table, inp.num_decoding, prefix, step_plan)
    torch.cuda.synchronize()
    assert K.check_status() == 0

    nd = n_dec
    q_p, k_p = O.norm_rope_prefill(q, k, qw, kw, cos, sin, 1e-6)
    O.quantize_prefill(k_p, v, cu, table, cached, nd, cache)
    kpre = np.zeros((HKV, cap, D), np.float32)
    vpre = np.zeros_like(kpre)
    O.dequantize_prefix(cache, cu_cached, table, kpre, vpre)
    want = O.prefill_attention(q_p, k_p, v, cu, kpre, vpre, cu_cached, nd)
    q_d = O.write_decode(q[:E], k[:E], v[:E], qw, kw, cos[:E], sin[:E], table, cache, cached, nd, 1e-6)
    C.set_threads(os.cpu_count() or 1)
    want[:nd] = C.decode_attention(q_d, cache, np.asarray(cached, np.int32), table, nd, SCALE)[:nd]
    H.assert_cache_equal(H.cache_to_numpy(dev_cache), cache, "full-size mixed step: ")
    live = cu_cached[-1]
    assert np.array_equal(H.to_bits(prefix.k[:, :live]), O.bf16_bits(kpre[:, :live]))
    assert np.array_equal(H.to_bits(prefix.v[:, :live]), O.bf16_bits(vpre[:, :live]))
    got = H.to_f32(out)
    rows = cu[n_dec + 1]  # decoding rows and the chunk's rows; the padding entry's rows are junk nobody reads
    mx, mean = H.attn_errors(got[:rows], want[:rows])
    assert mx <= 2e-2 and mean <= 2e-3, (mx, mean)
