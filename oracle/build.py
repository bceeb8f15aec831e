"""Builds the C oracle (oracle/kvfp4_oracle.c) into oracle/_build/libkvfp4_oracle.so with gcc.

The flags matter for parity: -ffp-contract=off keeps every fp32 step of the quantiser a single IEEE operation and
-fno-fast-math keeps NaN / signed-zero semantics (kv_fp4_ref.py:15-25 in the reference spells out the rule)."""
import os
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "kvfp4_oracle.c")
OUT_DIR = os.path.join(HERE, "_build")
LIB = os.path.join(OUT_DIR, "libkvfp4_oracle.so")


def build(force: bool = False) -> str:
    os.makedirs(OUT_DIR, exist_ok=True)
    if not force and os.path.exists(LIB) and os.path.getmtime(LIB) >= os.path.getmtime(SRC):
        return LIB
    cmd = ["gcc", "-O2", "-fPIC", "-shared", "-std=c11", "-fopenmp", "-ffp-contract=off", "-fno-fast-math",
           "-o", LIB, SRC, "-lm"]
    subprocess.run(cmd, check=True)
    return LIB


if __name__ == "__main__":
    print(build(force=True))
