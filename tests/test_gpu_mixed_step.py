"""One chunked-prefill + decode step through the attention ops in the reference's call order
(architecture.py:99-198), against the same composition of the CPU oracle, and a small
random-init decoder run end to end."""
import numpy as np
import pytest
import torch

from oracle import oracle as O
from tests import helpers as H
from tests.helpers import D, HKV, HQ

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def S():
    from inference_engine_b200 import scaffold

    return scaffold


@pytest.mark.parametrize("chained", [False, True])
@pytest.mark.parametrize("block_m", [16, 128])
def test_layer_attention_path_matches_oracle(S, block_m, chained):
    """chained = every kernel of the path launched with programmatic stream serialization (each may be
    brought up while its predecessor still runs and waits for it before touching its data), run three times
    back to back so that kernels of consecutive passes chain as well."""
    from inference_engine_b200 import kernels as K

    rng = np.random.default_rng(77 + block_m)
    page = 16
    plan = S.plan_step([37, 130], [(48, 70), (0, 33)], n_tokens=128, num_entries=6, block_m=block_m)
    table_t, pages = S.assign_pages(plan, page, 16, generator=torch.Generator().manual_seed(5))
    table = table_t.numpy()
    nd, N, E = 2, 128, 6
    cache = H.random_filled_cache(rng, pages, page)
    for b in (0, 1, 2):  # entries with history carry a calibration from their first chunk
        cache.k_calibration[table[b, 0]] = (0.5 + 1.5 * rng.random((HKV, 1, D))).astype(np.float32)
    q, k, v = H.randn_bf16(rng, N, HQ, D), H.randn_bf16(rng, N, HKV, D), H.randn_bf16(rng, N, HKV, D)
    qw = O.bf16_round((1 + 0.02 * rng.standard_normal(D)).astype(np.float32))
    kw = O.bf16_round((1 + 0.02 * rng.standard_normal(D)).astype(np.float32))
    cos, sin = O.rope_tables(np.asarray(plan["positions"], np.int32))
    cu, cached, cu_cached = plan["cu_seqlens"], plan["cached"], plan["cu_cached"]

    dev_cache = H.cache_to_torch(cache)
    inp = S.upload_step(plan, table_t, [0] * N, "cuda", block_m)
    prefix = S.PrefixScratch(torch.zeros(HKV, cu_cached[-1] + 8, D, device="cuda", dtype=torch.bfloat16),
                             torch.zeros(HKV, cu_cached[-1] + 8, D, device="cuda", dtype=torch.bfloat16), inp.cu_cached)
    args = (H.bf16_tensor(q), H.bf16_tensor(k), H.bf16_tensor(v), H.bf16_tensor(qw), H.bf16_tensor(kw),
            H.bf16_tensor(cos)[:, None, :], H.bf16_tensor(sin)[:, None, :])
    K.set_early_start(chained)
    try:
        for _ in range(3 if chained else 1):  # the step is idempotent: same rows, same values
            out = S.attention_ops(*args, dev_cache, inp, inp.cached_lens, inp.block_table, inp.num_decoding, prefix)
        torch.cuda.synchronize()
    finally:
        K.set_early_start(False)
    assert K.check_status() == 0

    q_p, k_p = O.norm_rope_prefill(q, k, qw, kw, cos, sin, 1e-6)
    O.quantize_prefill(k_p, v, cu, table, cached, nd, cache)
    kpre = np.zeros((HKV, cu_cached[-1] + 8, D), np.float32)
    vpre = np.zeros_like(kpre)
    O.dequantize_prefix(cache, cu_cached, table, kpre, vpre)
    want = O.prefill_attention(q_p, k_p, v, cu, kpre, vpre, cu_cached, nd)
    q_d = O.write_decode(q[:E], k[:E], v[:E], qw, kw, cos[:E], sin[:E], table, cache, cached, nd, 1e-6)
    O.decode_attention(q_d, cache, cached, table, nd, D ** -0.5, out=want[:E])

    H.assert_cache_equal(H.cache_to_numpy(dev_cache), cache, "mixed step: ")
    assert np.array_equal(H.to_bits(prefix.k), O.bf16_bits(kpre)) and np.array_equal(H.to_bits(prefix.v), O.bf16_bits(vpre))
    mx, mean = H.attn_errors(H.to_f32(out), want)
    assert mx <= 2e-2 and mean <= 2e-3, (mx, mean)


def test_small_decoder_mixed_then_decode_steps(S):
    """A 2-layer decoder with the real head geometry: a mixed step, then two pure-decode steps
    of every sequence; tokens are valid ids, the status word stays clear and a second run on
    fresh caches reproduces the tokens exactly."""
    from inference_engine_b200 import kernels as K

    dev = torch.device("cuda", 0)
    model = S.DecoderScaffold(dev, hidden=256, ffn=512, vocab=1000, layers=2, seed=3)
    page, entries, n_tokens = 16, 6, 128
    plan = S.plan_step([37, 130], [(48, 70), (0, 33)], n_tokens=n_tokens, num_entries=entries)
    table, pages = S.assign_pages(plan, page, 16, generator=torch.Generator().manual_seed(1))
    ids = torch.randint(0, 1000, (n_tokens,), generator=torch.Generator().manual_seed(2)).tolist()

    def run():
        rng = np.random.default_rng(9)
        caches = [H.cache_to_torch(H.random_filled_cache(rng, pages, page, gauss=True)) for _ in range(2)]
        inp = S.upload_step(plan, table, ids, dev)
        prefix = S.PrefixScratch(torch.zeros(HKV, 64, D, device=dev, dtype=torch.bfloat16),
                                 torch.zeros(HKV, 64, D, device=dev, dtype=torch.bfloat16), inp.cu_cached)
        toks = [model.forward(caches, inp, inp.ids, inp.cached_lens, inp.block_table, inp.num_decoding, prefix)]
        # afterwards all four sequences decode: cached lengths grew by their chunks
        cached = torch.tensor([38, 131, 118, 33], dtype=torch.int32, device=dev)
        nd = torch.tensor([4], dtype=torch.int32, device=dev)
        tab = inp.block_table[:4].contiguous()
        for _ in range(2):
            nxt = model.forward(caches, None, toks[-1][:4].int(), cached, tab, nd)
            toks.append(nxt)
            cached = cached + 1
        torch.cuda.synchronize()
        return [t.cpu() for t in toks]

    a, b = run(), run()
    assert K.check_status() == 0
    for x, y in zip(a, b):
        assert torch.equal(x, y) and int(x[:4].min()) >= 0 and int(x[:4].max()) < 1000
