"""Shared helpers of the parity tests: moving data between the numpy oracle and torch/CUDA."""
from __future__ import annotations

import numpy as np
import torch

from oracle import oracle as O

HQ, HKV, D = 16, 8, 128


def bf16_tensor(x: np.ndarray, device="cuda") -> torch.Tensor:
    """float32 array of bf16-representable values -> torch bf16 tensor (exact)."""
    return torch.from_numpy(np.ascontiguousarray(x, dtype=np.float32)).to(torch.bfloat16).to(device)


def bits_tensor(bits: np.ndarray, device="cuda") -> torch.Tensor:
    """uint16 bf16 bit patterns -> torch bf16 tensor."""
    return torch.from_numpy(np.ascontiguousarray(bits).view(np.int16)).view(torch.bfloat16).to(device)


def to_f32(t: torch.Tensor) -> np.ndarray:
    return t.detach().float().cpu().numpy()


def to_bits(t: torch.Tensor) -> np.ndarray:
    return t.detach().contiguous().cpu().view(torch.int16).numpy().view(np.uint16)


def randn_bf16(rng: np.random.Generator, *shape) -> np.ndarray:
    return O.bf16_round(rng.standard_normal(shape).astype(np.float32))


def cache_to_torch(c: O.KVCache, device="cuda"):
    from inference_engine_b200.kernels import LayerKVCache

    return LayerKVCache(*(torch.from_numpy(a.copy()).to(device) for a in (c.k, c.v, c.k_scale, c.v_scale, c.k_calibration)))


def cache_to_numpy(c) -> O.KVCache:
    return O.KVCache(*(t.detach().cpu().numpy() for t in (c.k, c.v, c.k_scale, c.v_scale, c.k_calibration)))


def assert_cache_equal(got: O.KVCache, want: O.KVCache, what=""):
    for name in ("k", "v", "k_scale", "v_scale", "k_calibration"):
        a, b = getattr(got, name), getattr(want, name)
        assert a.dtype == b.dtype and a.shape == b.shape
        same = a.view(np.uint8) == b.view(np.uint8)
        assert same.all(), f"{what}{name}: {np.count_nonzero(~same)} bytes differ from the oracle"


def i32(x, device="cuda") -> torch.Tensor:
    return torch.as_tensor(np.asarray(x, dtype=np.int32)).to(device)


def random_filled_cache(rng, num_pages, page_size, gauss=False) -> O.KVCache:
    """A cache full of plausible contents: random codes, positive scales, calibration of ones."""
    c = O.make_cache(num_pages, HKV, page_size, D)
    if gauss:
        for name, sname in (("k", "k_scale"), ("v", "v_scale")):
            x = O.bf16_round(rng.standard_normal((num_pages, HKV, page_size, D)).astype(np.float32))
            codes, scale = O.quantize_rows(x)
            getattr(c, name)[...] = codes
            getattr(c, sname)[...] = scale
    else:
        c.k[...] = rng.integers(-127, 128, c.k.shape, dtype=np.int8)
        c.v[...] = rng.integers(-127, 128, c.v.shape, dtype=np.int8)
        c.k_scale[...] = (0.01 + 0.03 * rng.random(c.k_scale.shape)).astype(np.float32)
        c.v_scale[...] = (0.01 + 0.03 * rng.random(c.v_scale.shape)).astype(np.float32)
    return c


def random_block_table(rng, lens, page_size, num_pages):
    """Disjoint random pages for sequences of the given token counts -> int32 [B, max_pages]
    (unused entries -1)."""
    need = [(n + page_size - 1) // page_size for n in lens]
    assert sum(need) <= num_pages
    perm = rng.permutation(num_pages)
    table = np.full((len(lens), max(max(need), 1)), -1, np.int32)
    at = 0
    for b, k in enumerate(need):
        table[b, :k] = perm[at : at + k]
        at += k
    return table


def attn_errors(got: np.ndarray, want: np.ndarray):
    err = np.abs(got.astype(np.float32) - want.astype(np.float32)) / np.maximum(1.0, np.abs(want))
    return float(err.max()), float(err.mean())
