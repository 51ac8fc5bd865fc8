"""Build recipe for the CPU oracle (test infrastructure; never imported by the product package).

`python oracle/build.py` compiles oracle/qc_oracle.c into oracle/_build/libqc_oracle.so with gcc.
Floating-point contraction and fast-math are disabled so every fp32 operation is a single
correctly-rounded IEEE operation, which the bit-exact comparisons rely on.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "qc_oracle.c")
OUT_DIR = os.path.join(HERE, "_build")
OUT = os.path.join(OUT_DIR, "libqc_oracle.so")


def build(force: bool = False) -> str:
    os.makedirs(OUT_DIR, exist_ok=True)
    if not force and os.path.exists(OUT) and os.path.getmtime(OUT) >= os.path.getmtime(SRC):
        return OUT
    cmd = [
        "gcc", "-O2", "-fopenmp", "-ffp-contract=off", "-fno-fast-math", "-fno-unsafe-math-optimizations",
        "-shared", "-fPIC", "-o", OUT, SRC, "-lm",
    ]
    subprocess.run(cmd, check=True)
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
