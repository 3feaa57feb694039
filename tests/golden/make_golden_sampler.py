"""Golden vectors for the sampler (sample: Gumbel-max, two stages), produced by the UNMODIFIED reference kernels
under Triton's CPU interpreter with the harness shims of make_golden.py.

Run:  python tests/golden/make_golden_sampler.py --reference /path/to/inference-engine
Writes tests/golden/reference_sampler.npz; bf16 arrays are stored as uint16 bit patterns (suffix _bf16)."""
from __future__ import annotations

import argparse
import os
import sys

os.environ["TRITON_INTERPRET"] = "1"

import numpy as np
import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from make_golden import install_shims, to_bits  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="checkout of kbwal/inference-engine (the unmodified reference)")
    ap.add_argument("--out", default=os.path.join(os.path.dirname(os.path.abspath(__file__)), "reference_sampler.npz"))
    args = ap.parse_args()
    sys.path.insert(0, os.path.join(args.reference, "qwen3-1.7b"))
    import kernels

    install_shims(kernels)
    g = torch.Generator().manual_seed(77)
    B, V = 6, 5000  # three blocks of 2048 columns, the last one ragged
    logits = (torch.randn(B, V, generator=g) * 2.0).to(torch.bfloat16)
    logits[1, 4097] = logits[1, 17] = logits[1].max() + 1  # an exact tie across blocks: the first index wins
    out = {"logits_bf16": to_bits(logits)}
    for name, tau, seed0 in (("greedy", 0.0, 5), ("t07", 0.7, 5), ("t07_next", 0.7, 6), ("t15_bigseed", 1.5, (1 << 40) + 12345)):
        seed = torch.tensor([seed0], dtype=torch.int64)
        tok = kernels.sample(logits, tau, seed)
        assert int(seed) == seed0 + 1
        out[f"{name}_tau"] = np.float32(tau)
        out[f"{name}_seed"] = np.int64(seed0)
        out[f"{name}_tokens"] = tok.view(-1).numpy().astype(np.int64)
    np.savez_compressed(args.out, **out)
    print("wrote", args.out, {k: (v.tolist() if v.size < 8 else v.shape) for k, v in out.items()})


if __name__ == "__main__":
    main()
