"""Builds libb200kv.so (the C-ABI CUDA library) in-tree with nvcc for sm_100a.

    python -m inference_engine_b200.build [--force]

The write-path translation unit is compiled with -fmad=false: its results must be bit-identical
to separately rounded IEEE fp32 arithmetic.  There is no other backend and no fallback: if the
library cannot be built or loaded the package raises.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
INCLUDE = os.path.join(ROOT, "include")
LIB = os.path.join(PKG, "libb200kv.so")
OBJ_DIR = os.path.join(PKG, "build")

ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON = ["-O3", "-lineinfo", "-std=c++17", "-Xcompiler", "-fPIC", "-I", INCLUDE, "-I", CSRC]
UNITS = {
    "abi.cu": [],
    "write_kernels.cu": ["-fmad=false"],
    "decode_attn.cu": [],
    "prefill_attn.cu": [],
    "prefill_attn_tc5.cu": [],
    "block_ops.cu": [],
    "sampler.cu": ["-fmad=false"],
    "skinny_linear_tc5.cu": [],
}
# The same library with per-warp timestamps compiled into the decode-attention kernel (bench.py --phases);
# never loaded by the product path.
STAMPS_LIB = os.path.join(PKG, "libb200kv_stamps.so")


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found: libb200kv.so cannot be built")


def sources() -> list[str]:
    return [os.path.join(CSRC, u) for u in UNITS if os.path.exists(os.path.join(CSRC, u))]


def needs_build() -> bool:
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    deps = sources() + [os.path.join(CSRC, "common.cuh"), os.path.join(INCLUDE, "b200kv.h")]
    return any(os.path.getmtime(d) > t for d in deps if os.path.exists(d))


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and not needs_build():
        return LIB
    nvcc = _nvcc()
    os.makedirs(OBJ_DIR, exist_ok=True)
    objs = []
    for unit, extra in UNITS.items():
        src = os.path.join(CSRC, unit)
        obj = os.path.join(OBJ_DIR, unit.replace(".cu", ".o"))
        cmd = [nvcc, *ARCH, *COMMON, *extra, "-c", src, "-o", obj]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
        subprocess.run(cmd, check=True)
        objs.append(obj)
    tmp = LIB + ".tmp"
    subprocess.run([nvcc, *ARCH, "-shared", "-cudart", "static", "-o", tmp, *objs], check=True)
    os.replace(tmp, LIB)
    build_stamps(nvcc, objs)
    return LIB


def build_stamps(nvcc: str, objs: list[str]) -> str:
    """libb200kv_stamps.so = the library with decode_attn.cu recompiled under -DB200KV_STAMPS."""
    obj = os.path.join(OBJ_DIR, "decode_attn_stamps.o")
    subprocess.run([nvcc, *ARCH, *COMMON, "-DB200KV_STAMPS", "-c", os.path.join(CSRC, "decode_attn.cu"), "-o", obj], check=True)
    rest = [o for o in objs if os.path.basename(o) != "decode_attn.o"]
    tmp = STAMPS_LIB + ".tmp"
    subprocess.run([nvcc, *ARCH, "-shared", "-cudart", "static", "-o", tmp, *rest, obj], check=True)
    os.replace(tmp, STAMPS_LIB)
    return STAMPS_LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
