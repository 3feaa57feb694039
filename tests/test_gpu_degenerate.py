"""Empty and degenerate inputs through every op: nothing to do must mean nothing launched, no fault, and
untouched outputs."""
import numpy as np
import pytest
import torch

from tests import helpers as H
from tests.helpers import D, HKV, HQ

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def K():
    from inference_engine_b200 import kernels

    return kernels


def bf(*shape):
    return torch.zeros(*shape, dtype=torch.bfloat16, device="cuda")


def test_empty_batches(K):
    rng = np.random.default_rng(0)
    cache = H.cache_to_torch(H.random_filled_cache(rng, 4, 16))
    before = [t.clone() for t in (cache.k, cache.v, cache.k_scale, cache.v_scale, cache.k_calibration)]
    i32 = lambda *v: torch.tensor(v, dtype=torch.int32, device="cuda")
    w = torch.ones(D, dtype=torch.bfloat16, device="cuda")
    # decode ops with B = 0
    q = K.fused_rope_kv_decode(bf(0, HQ, D), bf(0, HKV, D), bf(0, HKV, D), w, w, bf(0, 1, D // 2), bf(0, 1, D // 2),
                               torch.zeros(0, 1, dtype=torch.int32, device="cuda"), cache, i32(), i32(0), 1e-6)
    assert q.shape == (0, HQ, D)
    assert K.decode_attention(q, cache, i32(), torch.zeros(0, 1, dtype=torch.int32, device="cuda"), i32(0), 0.1).shape == (0, HQ, D)
    # prefill ops with no rows
    qp, kp = K.fused_norm_rope_prefill(bf(0, HQ, D), bf(0, HKV, D), w, w, bf(0, 1, D // 2), bf(0, 1, D // 2), 1e-6)
    assert qp.shape == (0, HQ, D) and kp.shape == (0, HKV, D)
    table = torch.zeros(2, 2, dtype=torch.int32, device="cuda")
    K.quantize_kv_prefill(kp, bf(0, HKV, D), i32(0, 0, 0), table, i32(0, 0), i32(0), cache)
    pk, pv = bf(HKV, 8, D), bf(HKV, 8, D)
    K.dequantize_kv_prefix(cache, i32(0, 0, 0), table, pk, pv)
    out = K.prefill_attention(bf(0, HQ, D), bf(0, HKV, D), bf(0, HKV, D), i32(), i32(0, 0, 0), i32(-1, -1), pk, pv,
                              i32(0, 0, 0), 128)
    assert out.shape == (0, HQ, D)
    # block ops and sampler with no rows
    assert K.silu_mul(bf(0, 256)).shape == (0, 128)
    r, n = K.add_rms_norm(bf(0, 256), bf(0, 256), torch.ones(256, dtype=torch.bfloat16, device="cuda"), 1e-6)
    assert r.shape == n.shape == (0, 256)
    seed = torch.tensor([3], dtype=torch.int64, device="cuda")
    assert K.sample(bf(0, 1000), 0.0, seed).shape == (0, 1) and int(seed.item()) == 3
    torch.cuda.synchronize()
    assert K.check_status() == 0
    for a, b in zip(before, (cache.k, cache.v, cache.k_scale, cache.v_scale, cache.k_calibration)):
        assert torch.equal(a, b)


def test_step_with_only_idle_tiles_and_no_decoders(K):
    """A step whose entries all have zero tokens (what a graph bucket replays when nothing is scheduled for an
    entry): every kernel runs its grid and writes nothing."""
    rng = np.random.default_rng(1)
    cache = H.cache_to_torch(H.random_filled_cache(rng, 4, 16))
    before = cache.k.clone()
    i32 = lambda *v: torch.tensor(v, dtype=torch.int32, device="cuda")
    N = 16
    q, k, v = bf(N, HQ, D), bf(N, HKV, D), bf(N, HKV, D)
    table = torch.zeros(3, 2, dtype=torch.int32, device="cuda")
    cu = i32(0, 0, 0, 0)  # three entries, none owns a row of the 16 packed rows
    K.quantize_kv_prefill(k, v, cu, table, i32(0, 0, 0), i32(0), cache)
    out = K.prefill_attention(q, k, v, torch.zeros(N, dtype=torch.int32, device="cuda"), cu, i32(-1, -1, -1, -1),
                              bf(HKV, 8, D), bf(HKV, 8, D), i32(0, 0, 0, 0), 128)
    torch.cuda.synchronize()
    assert out.shape == (N, HQ, D) and K.check_status() == 0 and torch.equal(before, cache.k)
