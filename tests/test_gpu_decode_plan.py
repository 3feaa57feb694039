"""The per-step plan of decode attention (b200kv_decode_plan + b200kv_decode_attn_planned): the planned
call must give the bits of the unplanned one (same work split, found another way) and the oracle's
values, a plan that does not belong to the batch must be reported and must write nothing, and the
planned call must keep working when it is chained behind the quantize-on-write kernel."""
import numpy as np
import pytest
import torch

from oracle import oracle as O
from tests import helpers as H
from tests.helpers import D, HKV, HQ

pytestmark = pytest.mark.gpu
SCALE = D ** -0.5
S_BAD_PLAN = 8


@pytest.fixture(scope="module")
def K():
    from inference_engine_b200 import kernels

    return kernels


def make_case(rng, lens, page_size, paged=True, gauss=True):
    B = len(lens)
    if paged:
        num_pages = sum((n + page_size - 1) // page_size for n in lens) + 3
        table = H.random_block_table(rng, lens, page_size, num_pages)
    else:
        num_pages = B + 1
        table = rng.permutation(num_pages)[:B].astype(np.int32)
    cache = H.random_filled_cache(rng, num_pages, page_size, gauss=gauss)
    q = H.randn_bf16(rng, B, HQ, D)
    cached = np.array([n - 1 for n in lens], np.int32)
    return q, cache, cached, table


CASES = {
    "boundaries": [1, 2, 15, 16, 17, 31, 32, 33, 63, 64, 65, 127, 128, 129, 130, 255, 256, 257, 1000],
    "one long": [4096],
    "few long": [2048, 2048, 2048],
    "many short": [128] * 256,
    "ragged": [int(x) for x in np.random.default_rng(5).integers(1, 3000, 37)],
    "more entries than the shared-memory length table": [20] * 700,
}


@pytest.mark.parametrize("name", list(CASES))
@pytest.mark.parametrize("page_size", [16, 64, 0])
def test_planned_equals_unplanned_and_oracle(K, name, page_size):
    """page_size 0 = the reference's layout: one row per sequence, slot_ids 1-D."""
    lens = CASES[name]
    paged = page_size > 0
    if not paged:
        if len(lens) > 64:
            pytest.skip("the one-row-per-sequence layout is covered by the smaller batches")
        page_size = (max(lens) + 24 + 15) // 16 * 16  # rows of any length are fine, the scale rows must stay 16-byte aligned
    rng = np.random.default_rng(list(CASES).index(name) * 1000 + page_size)
    q, cache, cached, table = make_case(rng, lens, page_size, paged)
    B = len(lens)
    for nd in (B, max(B - 3, 0)):
        tq, tc, tcl, ttab, tnd = H.bf16_tensor(q), H.cache_to_torch(cache), H.i32(cached), H.i32(table), H.i32([nd])
        plain = torch.full((B, HQ, D), 7.0, dtype=torch.bfloat16, device="cuda")
        planned = plain.clone()
        K.decode_attention(tq, tc, tcl, ttab, tnd, SCALE, out=plain)
        plan = K.plan_decode_step(tcl, ttab, tnd, tc)
        for _ in range(2):  # the plan serves any number of calls of the step
            K.decode_attention(tq, tc, tcl, ttab, tnd, SCALE, out=planned, plan=plan)
        torch.cuda.synchronize()
        assert K.check_status() == 0
        assert torch.equal(plain, planned), "the plan must reproduce the in-kernel work split bit for bit"
        assert np.all(H.to_f32(planned)[nd:] == 7.0), "rows of non-decoding entries must not be written"
        if nd:
            want = O.decode_attention(q, cache, cached, table, nd, SCALE)
            mx, mean = H.attn_errors(H.to_f32(planned)[:nd], want[:nd])
            assert mx <= 8e-3 and mean <= 4e-4, (mx, mean)


def test_planned_call_with_fewer_query_rows_than_entries(K):
    """A mixed step packs tokens: its decoding entries come first with one row each, and a step with fewer tokens
    than entries passes q / out with fewer rows than cached_lens has entries.  The plan covers all entries; the
    planned call must accept that and give the unplanned result (it once compared q's row count with the plan's
    entry count and refused the plan)."""
    rng = np.random.default_rng(77)
    lens = [300, 17, 2049, 64] + [1] * 9  # 13 entries, the first 4 decoding
    q, cache, cached, table = make_case(rng, lens, 16)
    nd, rows = 4, 6  # six packed token rows, thirteen entries
    tq, tc, tcl, ttab, tnd = H.bf16_tensor(q[:rows]), H.cache_to_torch(cache), H.i32(cached), H.i32(table), H.i32([nd])
    plain = torch.full((rows, HQ, D), 7.0, dtype=torch.bfloat16, device="cuda")
    planned = plain.clone()
    K.decode_attention(tq, tc, tcl, ttab, tnd, SCALE, out=plain)
    plan = K.plan_decode_step(tcl, ttab, tnd, tc)
    K.decode_attention(tq, tc, tcl, ttab, tnd, SCALE, out=planned, plan=plan)
    torch.cuda.synchronize()
    assert K.check_status() == 0
    assert torch.equal(plain, planned)
    assert np.all(H.to_f32(planned)[nd:] == 7.0)
    want = O.decode_attention(q, cache, cached, table, nd, SCALE)
    mx, mean = H.attn_errors(H.to_f32(planned)[:nd], want[:nd])
    assert mx <= 8e-3 and mean <= 4e-4, (mx, mean)


def test_plan_of_another_step_is_reported_and_writes_nothing(K):
    rng = np.random.default_rng(31)
    lens = [700, 33, 1500, 16, 257]
    q, cache, cached, table = make_case(rng, lens, 16)
    B = len(lens)
    tq, tc, ttab, tnd = H.bf16_tensor(q), H.cache_to_torch(cache), H.i32(table), H.i32([B])
    tcl = H.i32(cached)
    plan = K.plan_decode_step(tcl, ttab, tnd, tc)
    good = K.decode_attention(tq, tc, tcl, ttab, tnd, SCALE, plan=plan).clone()
    # the next step: every sequence is one token longer, the plan is stale
    tcl2 = H.i32(cached + 1)
    # (tokens cached+1 exist in the random cache: the table rows have room for them)
    out = torch.full((B, HQ, D), 7.0, dtype=torch.bfloat16, device="cuda")
    K.decode_attention(tq, tc, tcl2, ttab, tnd, SCALE, out=out, plan=plan)
    torch.cuda.synchronize()
    assert K.check_status() & S_BAD_PLAN
    assert np.all(H.to_f32(out) == 7.0), "a warp that saw a stale plan must not write"
    # a plan made for another batch size is refused as a whole
    K.decode_attention(tq[:3], tc, tcl[:3], ttab[:3], H.i32([3]), SCALE, out=out[:3], plan=plan)
    torch.cuda.synchronize()
    assert K.check_status() & S_BAD_PLAN
    assert np.all(H.to_f32(out) == 7.0)
    # nothing was left behind: the right plan still gives the right bits
    again = K.decode_attention(tq, tc, tcl, ttab, tnd, SCALE, plan=K.plan_decode_step(tcl, ttab, tnd, tc))
    assert torch.equal(good, again) and K.check_status() == 0


def test_planned_call_chained_behind_the_write_kernel(K):
    """plan -> (write -> planned attention) x layers on one stream with early start: the attention
    kernel reads its plan before it waits for the write kernel and must still see the new token."""
    rng = np.random.default_rng(19)
    lens = [257, 16, 1000, 64, 3, 4096]
    B, P, layers = len(lens), 16, 4
    pages = sum((n + P - 1) // P for n in lens) + 2
    table = H.random_block_table(rng, lens, P, pages)
    cached = np.array([n - 1 for n in lens], np.int32)
    cos, sin = O.rope_tables(cached)
    w = O.bf16_round((1 + 0.02 * rng.standard_normal(D)).astype(np.float32))
    dev_caches, qkvs, wants = [], [], []
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
            plan = K.plan_decode_step(tcl, ttab, tnd, dev_caches[0])
            outs = []
            for l in range(layers):
                tq, tk, tv = qkvs[l].split([HQ * D, HKV * D, HKV * D], dim=-1)
                qr = K.fused_rope_kv_decode(tq.view(B, HQ, D), tk.view(B, HKV, D), tv.view(B, HKV, D), tw, tw, tcos, tsin,
                                            ttab, dev_caches[l], tcl, tnd, 1e-6)
                outs.append(K.decode_attention(qr, dev_caches[l], tcl, ttab, tnd, SCALE, plan=plan))
            torch.cuda.synchronize()
            for l in range(layers):
                mx, mean = H.attn_errors(H.to_f32(outs[l]), wants[l])
                assert mx <= 8e-3 and mean <= 4e-4, (rep, l, mx, mean)
    finally:
        K.set_early_start(False)
    assert K.check_status() == 0


def test_plan_argument_validation(K):
    from inference_engine_b200 import _lib

    lib = _lib.load()
    rng = np.random.default_rng(2)
    q, cache, cached, table = make_case(rng, [40, 50], 16)
    tq, tc, tcl, ttab, tnd = H.bf16_tensor(q), H.cache_to_torch(cache), H.i32(cached), H.i32(table), H.i32([2])
    small = torch.empty(64, dtype=torch.uint8, device="cuda")
    with pytest.raises(AssertionError):
        K.plan_decode_step(tcl, ttab, tnd, tc, out=small)
    plan = K.plan_decode_step(tcl, ttab, tnd, tc)
    assert plan.numel() == lib.b200kv_decode_plan_bytes(K.num_sms(tq.device))
    with pytest.raises(ValueError):  # the two-kernel reduction needs the unplanned kernel's prefix array
        K.decode_attention(tq, tc, tcl, ttab, tnd, SCALE, variant=2, plan=plan)
