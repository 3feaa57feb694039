"""Golden vectors for the weight-streaming matmul of the decode step (skinny_matmul, the kernel `linear` picks for
few rows), produced by the UNMODIFIED reference kernel under Triton's CPU interpreter, with the harness shims of
make_golden.py.

Run:  python tests/golden/make_golden_linear.py --reference /path/to/inference-engine
Writes tests/golden/reference_linear.npz; bf16 arrays are stored as uint16 bit patterns (suffix _bf16)."""
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
    ap.add_argument("--out", default=os.path.join(os.path.dirname(os.path.abspath(__file__)), "reference_linear.npz"))
    args = ap.parse_args()
    sys.path.insert(0, os.path.join(args.reference, "qwen3-1.7b"))
    import kernels

    install_shims(kernels)
    kernels.skinny_matmul_kernel.configs = kernels.skinny_matmul_kernel.configs[:1]  # the autotuner needs a GPU
    g = torch.Generator().manual_seed(31)
    out = {}
    for tag, (M, N, K) in {"a": (1, 128, 256), "b": (5, 256, 512), "c": (64, 128, 768)}.items():
        x = torch.randn(M, K, generator=g).to(torch.bfloat16)
        w = (torch.randn(N, K, generator=g) * 0.05).to(torch.bfloat16)
        y = kernels.skinny_matmul(x, w)
        out[f"{tag}_x_bf16"], out[f"{tag}_w_bf16"], out[f"{tag}_y_bf16"] = to_bits(x), to_bits(w), to_bits(y)
    np.savez_compressed(args.out, **out)
    print("wrote", args.out, {k: v.shape for k, v in out.items()})


if __name__ == "__main__":
    main()
