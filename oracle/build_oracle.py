"""Compile the CPU oracle (oracle/lif_oracle.c) into oracle/liblif_oracle.so.

TEST INFRASTRUCTURE ONLY: the shared object built here is the checker used by the tests,
the smoke check and the benchmark's CPU-baseline leg; the shipped package never loads it.

``-ffp-contract=off`` matters: gcc's default would fuse multiply-adds and change the
rounding the oracle is meant to reproduce.

The reference's own native code (snnlib/cuda/snn.cpp, snn_kernel_fp.cu, snn_kernel_bp.cu)
is CUDA against the PyTorch 1.8 C++ API and has no CPU build; it is not compiled here.

``install_reference()`` places the reference's own CPU implementation of the path - its
pure-PyTorch twin snnlib/example/gold_op.py - into the git-ignored folder oracle/_ref/ when a
reference checkout is mounted, so that the benchmark's reference arm can time the unmodified
reference code on machines where the checkout itself is absent. Nothing under oracle/_ref/ is
part of the repository's history.
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


REF_DIR = os.path.join(HERE, "_ref")
# the reference checkout: $SNN_REFERENCE_CHECKOUT, else a folder named "reference" beside this repository
REF_CHECKOUT = os.environ.get("SNN_REFERENCE_CHECKOUT",
                              os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference"))


def install_reference() -> str:
    """Copy the reference's gold_op.py (unmodified) into oracle/_ref/. Returns the installed path,
    the path of an earlier install when no checkout is mounted, or '' when there is neither."""
    import shutil
    dst = os.path.join(REF_DIR, "gold_op.py")
    src = os.path.join(REF_CHECKOUT, "snnlib", "example", "gold_op.py")
    if os.path.exists(src):
        os.makedirs(REF_DIR, exist_ok=True)
        shutil.copyfile(src, dst)
    return dst if os.path.exists(dst) else ""


if __name__ == "__main__":
    print(install_reference() or "no reference checkout: oracle/_ref not installed")
    print(build(force="--force" in sys.argv))
