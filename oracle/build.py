"""Build recipe for the CPU oracle (test infrastructure; never imported by the product).

    python oracle/build.py            # -> oracle/libsapient_oracle.so

Flags: -O3 -ffp-contract=off keeps every rounding point of the restated Rust code
(Rust never contracts or reassociates float arithmetic); -mavx2 -mfma only makes
the explicit fmaf calls of the restated AVX2 Q8_0 dot single instructions.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "sapient_oracle.cpp")
OUT = os.path.join(HERE, "libsapient_oracle.so")


def build_oracle(force: bool = False) -> str:
    if not force and os.path.exists(OUT) and os.path.getmtime(OUT) >= os.path.getmtime(SRC):
        return OUT
    cmd = [
        "g++", "-std=c++17", "-O3", "-ffp-contract=off", "-fno-fast-math", "-mavx2", "-mfma",
        "-fopenmp", "-shared", "-fPIC", "-Wall", "-Wextra", "-o", OUT, SRC,
    ]
    subprocess.run(cmd, check=True)
    return OUT


if __name__ == "__main__":
    print(build_oracle(force="--force" in sys.argv))
