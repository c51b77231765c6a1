"""Compile the CPU oracle (oracle/lif_oracle.c) into oracle/liblif_oracle.so.

TEST INFRASTRUCTURE ONLY: the shared object built here is the checker used by the tests,
the smoke check and the benchmark's CPU-baseline leg; the shipped package never loads it.

``-ffp-contract=off`` matters: gcc's default would fuse multiply-adds and change the
rounding the oracle is meant to reproduce.

The reference's own native code (snnlib/cuda/snn.cpp, snn_kernel_fp.cu, snn_kernel_bp.cu)
is CUDA against the PyTorch 1.8 C++ API and has no CPU build; it is not compiled here.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "lif_oracle.c")
OUT = os.path.join(HERE, "liblif_oracle.so")


def build(force: bool = False) -> str:
    if (not force and os.path.exists(OUT)
            and os.path.getmtime(OUT) >= os.path.getmtime(SRC)):
        return OUT
    cmd = ["gcc", "-O2", "-std=c11", "-fPIC", "-shared", "-fopenmp", "-ffp-contract=off",
           "-fno-fast-math", "-o", OUT, SRC, "-lm"]
    subprocess.run(cmd, check=True)
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
