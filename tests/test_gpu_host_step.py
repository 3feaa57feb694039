"""The host-buffer decode step: the pipelined form (layer groups, three streams) must give exactly what the
plain form gives, which must be what the two ops give when called directly."""
import numpy as np
import pytest
import torch

from oracle import oracle as O
from tests import helpers as H
from tests.helpers import D, HKV, HQ

pytestmark = pytest.mark.gpu


def test_pipelined_host_step_equals_plain_and_direct():
    from inference_engine_b200 import kernels as K
    from inference_engine_b200.host_step import HostDecodeStep

    rng = np.random.default_rng(11)
    L, B, page = 5, 6, 16
    lens = [33, 1, 160, 47, 16, 95]
    table = H.random_block_table(rng, [n + 1 for n in lens], page, 40)
    table[table < 0] = 0

    def fresh():
        r = np.random.default_rng(12)
        return [H.cache_to_torch(H.random_filled_cache(r, 40, page, gauss=True)) for _ in range(L)]

    pin = lambda t: t.pin_memory()
    qkv = pin(torch.from_numpy(O.bf16_bits(H.randn_bf16(rng, L, B, (HQ + 2 * HKV) * D)).view(np.int16)).view(torch.bfloat16))
    cos_np, sin_np = O.rope_tables(np.asarray(lens, np.int32))
    cos = pin(torch.from_numpy(O.bf16_bits(cos_np).view(np.int16)).view(torch.bfloat16).reshape(B, 1, D // 2))
    sin = pin(torch.from_numpy(O.bf16_bits(sin_np).view(np.int16)).view(torch.bfloat16).reshape(B, 1, D // 2))
    cached = pin(torch.tensor(lens, dtype=torch.int32))
    tab = pin(torch.from_numpy(table.astype(np.int32)))
    nd = pin(torch.tensor([B], dtype=torch.int32))

    def run(groups):
        caches = fresh()
        step = HostDecodeStep(caches, B, HQ, HKV, D, tuple(tab.shape))
        out = pin(torch.zeros(L, B, HQ, D, dtype=torch.bfloat16))
        step.run_host(qkv, cos, sin, cached, tab, nd, out)  # plain, eager
        torch.cuda.synchronize()
        if groups:
            step.capture(groups=groups)
            out.zero_()
            for _ in range(2):  # the step is idempotent (same rows, same values)
                step.run_host(qkv, cos, sin, cached, tab, nd, out)
            torch.cuda.synchronize()
        return out.clone(), [H.cache_to_numpy(c) for c in caches]

    out_plain, caches_plain = run(0)
    out_pipe, caches_pipe = run(2)
    assert torch.equal(out_plain, out_pipe)
    for a, b in zip(caches_plain, caches_pipe):
        H.assert_cache_equal(a, b, "pipelined vs plain: ")

    # layer 3 directly through the two ops
    caches = fresh()
    dq = qkv.cuda()
    q, k, v = dq[3].split([HQ * D, HKV * D, HKV * D], dim=-1)
    ones = torch.ones(D, dtype=torch.bfloat16, device="cuda")
    qr = K.fused_rope_kv_decode(q.view(B, HQ, D), k.view(B, HKV, D), v.view(B, HKV, D), ones, ones, cos.cuda(), sin.cuda(),
                                tab.cuda(), caches[3], cached.cuda(), nd.cuda(), 1e-6)
    want = K.decode_attention(qr, caches[3], cached.cuda(), tab.cuda(), nd.cuda(), D ** -0.5)
    assert torch.equal(want.cpu(), out_pipe[3])
    assert K.check_status() == 0
