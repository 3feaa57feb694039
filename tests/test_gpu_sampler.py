"""GPU parity of the sampler against the reference kernels' own tokens (golden) and against the CPU oracle on
the real vocabulary size.  Token ids are integers: the comparison is exact."""
import numpy as np
import pytest
import torch

from oracle import oracle as O
from tests import helpers as H
from tests.test_oracle_sampler import CASES, GOLD

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def K():
    from inference_engine_b200 import kernels

    return kernels


@pytest.mark.parametrize("case", CASES)
def test_reference_golden(K, case):
    g = dict(np.load(GOLD))
    seed = torch.tensor([int(g[f"{case}_seed"])], dtype=torch.int64, device="cuda")
    tok = K.sample(H.bits_tensor(g["logits_bf16"]), float(g[f"{case}_tau"]), seed)
    assert tok.shape == (6, 1) and tok.dtype == torch.int64
    assert np.array_equal(tok.view(-1).cpu().numpy(), g[f"{case}_tokens"])
    assert int(seed.item()) == int(g[f"{case}_seed"]) + 1  # the seed advances by one per call


@pytest.mark.parametrize("tau,dtype", [(0.0, torch.bfloat16), (1.0, torch.bfloat16), (0.3, torch.float32)])
def test_vocabulary_size_vs_oracle(K, tau, dtype):
    rng = np.random.default_rng(5)
    B, V = 9, 151936
    x = O.bf16_round((rng.standard_normal((B, V)) * 3).astype(np.float32))
    t = torch.from_numpy(x).to("cuda").to(dtype)
    seed = torch.tensor([2024], dtype=torch.int64, device="cuda")
    a = K.sample(t, tau, seed).view(-1).cpu().numpy()
    b = K.sample(t, tau, seed).view(-1).cpu().numpy()  # seed 2025 now
    assert np.array_equal(a, O.sample(x, tau, 2024)) and np.array_equal(b, O.sample(x, tau, 2025))
    if tau > 0:
        assert not np.array_equal(a, b)


def test_ties_go_to_the_first_index_and_strided_rows(K):
    buf = torch.zeros(3, 4096 + 64, dtype=torch.bfloat16, device="cuda")
    x = buf[:, :4096]  # a strided view
    x[0, 3000] = x[0, 77] = x[0, 2049] = 5.0
    x[1, 4095] = 1.0
    seed = torch.tensor([0], dtype=torch.int64, device="cuda")
    assert K.sample(x, 0.0, seed).view(-1).tolist() == [77, 4095, 0]
