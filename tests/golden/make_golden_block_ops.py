"""Golden vectors for the two element-wise ops of the decoder block (silu_mul, add_rms_norm), produced by
the UNMODIFIED reference kernels under Triton's CPU interpreter, with the harness shims of make_golden.py.

Run:  python tests/golden/make_golden_block_ops.py --reference /path/to/inference-engine
Writes tests/golden/reference_block_ops.npz; bf16 arrays are stored as uint16 bit patterns (suffix _bf16)."""
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
    ap.add_argument("--out", default=os.path.join(os.path.dirname(os.path.abspath(__file__)), "reference_block_ops.npz"))
    args = ap.parse_args()
    sys.path.insert(0, os.path.join(args.reference, "qwen3-1.7b"))
    import kernels

    install_shims(kernels)
    g = torch.Generator().manual_seed(21)
    out = {}
    # silu_mul: [N, 2D] -> [N, D]; D not a multiple of the kernel's 1024-column block, a strided input view
    N, Dm = 5, 1536
    buf = (torch.randn(N, 2 * Dm + 64, generator=g) * 2.0).to(torch.bfloat16)
    gate_up = buf[:, : 2 * Dm]
    y = kernels.silu_mul(gate_up)
    out["sm_in_bf16"], out["sm_out_bf16"] = to_bits(gate_up), to_bits(y)
    # add_rms_norm: residual, delta [N, D] -> (residual + delta, rmsnorm(residual + delta) * w)
    N, Dm = 7, 2048
    res = (torch.randn(N, Dm, generator=g) * 3.0).to(torch.bfloat16)
    delta = torch.randn(N, Dm, generator=g).to(torch.bfloat16)
    w = (1 + 0.1 * torch.randn(Dm, generator=g)).to(torch.bfloat16)
    new_res, normed = kernels.add_rms_norm(res, delta, w, 1e-6)
    out.update(arn_res_bf16=to_bits(res), arn_delta_bf16=to_bits(delta), arn_w_bf16=to_bits(w),
               arn_new_res_bf16=to_bits(new_res), arn_normed_bf16=to_bits(normed))
    np.savez_compressed(args.out, **out)
    print("wrote", args.out, {k: v.shape for k, v in out.items()})


if __name__ == "__main__":
    main()
