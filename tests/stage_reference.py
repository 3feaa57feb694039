"""Put an UNMODIFIED copy of the reference engine's Python files where the GPU tests and the Triton
comparison of the benchmark look for them when no checkout is named through B200KV_REFERENCE:
baseline/_ref/qwen3-1.7b/ under the repository root (git-ignored: the copy is never committed).

    python tests/stage_reference.py --reference /path/to/inference-engine

Only tests/test_gpu_reference_caller.py (which imports architecture.py and engine.py with `kernels` resolving to
this repository's module) and `bench.py --vs-triton` (which imports the reference's kernels.py to time its Triton
kernels beside the CUDA ones) read the copy."""
from __future__ import annotations

import argparse
import filecmp
import os
import shutil

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
FILES = ["architecture.py", "engine.py", "kernels.py"]


def stage(reference: str) -> str | None:
    src = os.path.join(reference, "qwen3-1.7b")
    if not all(os.path.exists(os.path.join(src, f)) for f in FILES):
        return None
    dst = os.path.join(ROOT, "baseline", "_ref", "qwen3-1.7b")
    os.makedirs(dst, exist_ok=True)
    for f in FILES:
        a, b = os.path.join(src, f), os.path.join(dst, f)
        if not (os.path.exists(b) and filecmp.cmp(a, b, shallow=False)):
            shutil.copyfile(a, b)
    return dst


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="checkout of kbwal/inference-engine")
    print(stage(ap.parse_args().reference) or "no qwen3-1.7b/ with the expected files under that path")
