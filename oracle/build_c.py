"""Builds the C restatement (oracle/kvattn_oracle.c) into oracle/_build/libkvoracle.so.

    python oracle/build_c.py

Test infrastructure only.  -ffp-contract=off and no fast-math keep every fp32 operation
separately rounded, as the restatement requires."""
import os
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "kvattn_oracle.c")
OUT_DIR = os.path.join(HERE, "_build")
LIB = os.path.join(OUT_DIR, "libkvoracle.so")


def build(force: bool = False) -> str:
    if not force and os.path.exists(LIB) and os.path.getmtime(LIB) >= os.path.getmtime(SRC):
        return LIB
    os.makedirs(OUT_DIR, exist_ok=True)
    tmp = LIB + ".tmp"
    subprocess.run(["gcc", "-O2", "-ffp-contract=off", "-fopenmp", "-shared", "-fPIC", "-o", tmp, SRC, "-lm"], check=True)
    os.replace(tmp, LIB)
    return LIB


if __name__ == "__main__":
    print(build())
