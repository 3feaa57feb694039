"""Buffers the kernels may only partly touch, checked with poison and canaries through the C ABI.

Decode attention: the split partials of the workspace hold NaNs before the call (only the arrival counters are
zero, as the header demands), a guard band follows the workspace, `out` has rows past num_decoding and a guard
band behind it.  The result must be the oracle's and bit-equal to a run on a clean workspace, the counters must
be back at zero, and no guard byte may change.  Chunked prefill: the dequantized-prefix scratch is NaN wherever
dequantize_kv_prefix has no row to write; it must write exactly its rows, and prefill_attention must not read
any other.  The allocation-free entry is checked against the oracle as well (its own file only compares it with
the regular entry)."""
import ctypes

import numpy as np
import pytest
import torch

from oracle import c_oracle as CO
from oracle import oracle as O
from tests import helpers as H
from tests.helpers import D, HKV, HQ

pytestmark = pytest.mark.gpu
SCALE = D ** -0.5
GUARD = 4096


def decode_case(seed, lens, page_size=16):
    rng = np.random.default_rng(seed)
    num_pages = sum((n + page_size - 1) // page_size for n in lens) + 2
    table = H.random_block_table(rng, lens, page_size, num_pages)
    cache = H.random_filled_cache(rng, num_pages, page_size, gauss=True)
    q = H.randn_bf16(rng, len(lens), HQ, D)
    cached = np.array([n - 1 for n in lens], np.int32)
    return q, cache, cached, table


def oracle_decode(q, cache, cached, table, nd):
    return CO.decode_attention(q, cache, cached, table, nd, SCALE)  # the C restatement: seconds at these sizes


@pytest.mark.parametrize("planned", [False, True])
@pytest.mark.parametrize("lens", [[4096, 1, 700, 33, 2048], [130] * 40 + [3000], [17]], ids=["ragged", "many", "one"])
def test_decode_workspace_poison_and_guards(lens, planned):
    from inference_engine_b200 import _lib, kernels as K

    lib = _lib.load()
    q, cache, cached, table = decode_case(5 + len(lens), lens)
    B = len(lens)
    nd = max(B - 2, 1)
    dev = torch.device("cuda", 0)
    sms = K.num_sms(dev)
    nbytes = lib.b200kv_decode_attn_workspace_bytes(B, HQ, HKV, D, sms)
    zero = lib.b200kv_decode_attn_workspace_zero_bytes(B, HKV)
    assert 0 < zero < nbytes
    tq, tc, tcl, ttab, tnd = H.bf16_tensor(q), H.cache_to_torch(cache), H.i32(cached), H.i32(table), H.i32([nd])
    cs, ts = K._cache_struct(tc), K._table_struct(ttab)
    plan = K.plan_decode_step(tcl, ttab, tnd, tc) if planned else None

    def run(poison):
        ws = torch.zeros(nbytes + GUARD, dtype=torch.uint8, device=dev)
        ws[nbytes:] = 0xA5
        if poison:
            ws[zero:nbytes] = 0xFF  # fp32 NaN in every partial and every (m, l) pair
        rows = B + 3
        buf = torch.full((rows * HQ * D + GUARD // 2,), 7.0, dtype=torch.bfloat16, device=dev)
        out = buf[: rows * HQ * D].view(rows, HQ, D)
        args = [tq.data_ptr(), tq.stride(0), tq.stride(1), ctypes.byref(cs), ctypes.byref(ts), tcl.data_ptr(),
                tnd.data_ptr(), SCALE, out.data_ptr(), out.stride(0), out.stride(1), ws.data_ptr(), nbytes]
        tail = [B, HQ, sms, 0, K.status_word(dev).data_ptr(), torch.cuda.current_stream().cuda_stream]
        for _ in range(2):  # the second call runs on what the first left behind
            if planned:
                rc = lib.b200kv_decode_attn_planned(*args, plan.data_ptr(), plan.numel(), *tail)
            else:
                rc = lib.b200kv_decode_attn(*args, *tail)
            assert rc == 0
        torch.cuda.synchronize()
        assert bool((ws[nbytes:] == 0xA5).all()), "bytes behind the workspace were written"
        assert bool((ws[:zero] == 0).all()), "arrival counters not returned to zero"
        assert bool((buf[nd * HQ * D:] == 7.0).all()), "rows past num_decoding or the guard behind out were written"
        return out[:nd].clone()

    clean, dirty = run(False), run(True)
    assert K.check_status() == 0
    assert torch.equal(clean, dirty)
    assert not bool(torch.isnan(dirty.float()).any())
    want = oracle_decode(q, cache, cached, table, nd)[:nd]
    mx, mean = H.attn_errors(H.to_f32(dirty), want)
    assert mx <= 2e-2 and mean <= 2e-3, (mx, mean)


@pytest.mark.parametrize("lens", [[4096, 1, 700, 33, 2048], [130] * 40 + [3000]], ids=["ragged", "many"])
def test_static_entry_against_the_oracle(lens):
    from inference_engine_b200 import kernels as K

    q, cache, cached, table = decode_case(21 + len(lens), lens)
    B = len(lens)
    tq, tc = H.bf16_tensor(q), H.cache_to_torch(cache)
    for nd in (B, B - 1):
        out = torch.full((B, HQ, D), 3.0, dtype=torch.bfloat16, device="cuda")
        K.decode_attention_static(tq, tc, H.i32(cached), H.i32(table), H.i32([nd]), SCALE, out)
        torch.cuda.synchronize()
        assert bool((out[nd:] == 3.0).all())
        want = oracle_decode(q, cache, cached, table, nd)[:nd]
        mx, mean = H.attn_errors(H.to_f32(out[:nd]), want)
        assert mx <= 2e-2 and mean <= 2e-3, (mx, mean)
    assert K.check_status() == 0


@pytest.mark.parametrize("variant", [1, 2])
def test_prefix_scratch_poison(variant):
    """A decoding entry, a 200-row chunk on 300 cached tokens, a first chunk, a 40-row chunk on 129 cached tokens."""
    from inference_engine_b200 import kernels as K

    rng = np.random.default_rng(77)
    page = 16
    chunk, prior, nd = [1, 200, 77, 40], [55, 300, 0, 129], 1
    B, N = len(chunk), sum(chunk)
    lens = [p + c for p, c in zip(prior, chunk)]
    num_pages = sum((n + page - 1) // page for n in lens) + 2
    table = H.random_block_table(rng, lens, page, num_pages)
    cache = H.random_filled_cache(rng, num_pages, page, gauss=True)
    cu = np.concatenate([[0], np.cumsum(chunk)]).astype(np.int32)
    prefix = [0 if b < nd else p for b, p in enumerate(prior)]
    cu_cached = np.concatenate([[0], np.cumsum(prefix)]).astype(np.int32)
    total = int(cu_cached[-1])
    seq_ids = np.concatenate([np.full(L, b) for b, L in enumerate(chunk)]).astype(np.int32)
    q, k, v = H.randn_bf16(rng, N, HQ, D), H.randn_bf16(rng, N, HKV, D), H.randn_bf16(rng, N, HKV, D)
    tiles = [r for b in range(nd, B) for r in range(cu[b], cu[b + 1], 128)] + [-1, -1]

    rows = total + 37  # the engine's scratch is sized for the longest prefix, not for this step's
    kpre = torch.full((HKV, rows, D), float("nan"), dtype=torch.bfloat16, device="cuda")
    vpre = torch.full_like(kpre, float("nan"))
    tc = H.cache_to_torch(cache)
    K.dequantize_kv_prefix(tc, H.i32(cu_cached), H.i32(table), kpre, vpre)
    torch.cuda.synchronize()
    for t in (kpre, vpre):
        assert not bool(torch.isnan(t[:, :total].float()).any()), "a prefix row was not written"
        assert bool(torch.isnan(t[:, total:].float()).all()), "rows past the last prefix were written"
    wk = np.zeros((HKV, rows, D), np.float32)
    wv = np.zeros_like(wk)
    O.dequantize_prefix(cache, cu_cached, table, wk, wv)
    assert np.array_equal(H.to_f32(kpre)[:, :total], wk[:, :total])
    assert np.array_equal(H.to_f32(vpre)[:, :total], wv[:, :total])

    out = K.prefill_attention(H.bf16_tensor(q), H.bf16_tensor(k), H.bf16_tensor(v), H.i32(seq_ids), H.i32(cu),
                              H.i32(tiles), kpre, vpre, H.i32(cu_cached), 128, variant=variant)
    assert K.check_status() == 0
    got = H.to_f32(out)[cu[nd]:]
    assert not np.isnan(got).any(), "prefill attention read a row outside its prefix"
    want = O.prefill_attention(q, k, v, cu, wk, wv, cu_cached, nd)[cu[nd]:]
    mx, mean = H.attn_errors(got, want)
    assert mx <= 8e-3 and mean <= 4e-4, (mx, mean)
