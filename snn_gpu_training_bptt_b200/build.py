"""Build libsnn_b200.so (the C-ABI CUDA library) in-tree with nvcc for sm_100a.

    python -m snn_gpu_training_bptt_b200.build [--force] [--verbose]

The shared object lands next to this file so it travels with the source tree. There is no
other backend: without it the package refuses to run.
"""
import glob
import os
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG, "csrc")
INCLUDE = os.path.join(os.path.dirname(PKG), "include")
LIB = os.path.join(PKG, "libsnn_b200.so")

NVCC_FLAGS = [
    "-O3", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
    "-Xcompiler", "-fPIC", "-shared",
]


def sources():
    return sorted(glob.glob(os.path.join(CSRC, "*.cu")))


def _stale():
    if not os.path.exists(LIB):
        return True
    built = os.path.getmtime(LIB)
    deps = sources() + glob.glob(os.path.join(CSRC, "*.cuh")) + glob.glob(os.path.join(INCLUDE, "*.h"))
    return any(os.path.getmtime(d) > built for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and not _stale():
        return LIB
    nvcc = os.environ.get("NVCC", "nvcc")
    objdir = os.path.join(PKG, "build")
    os.makedirs(objdir, exist_ok=True)
    compile_flags = [f for f in NVCC_FLAGS if f != "-shared"] + (["-Xptxas", "-v"] if verbose else [])

    def compile_one(src):
        obj = os.path.join(objdir, os.path.basename(src)[:-3] + ".o")
        res = subprocess.run([nvcc] + compile_flags + ["-c", "-o", obj, src], capture_output=True, text=True)
        return obj, res

    from concurrent.futures import ThreadPoolExecutor
    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as pool:
        results = list(pool.map(compile_one, sources()))
    for obj, res in results:
        if verbose or res.returncode:
            sys.stderr.write(res.stdout + res.stderr)
        if res.returncode:
            raise subprocess.CalledProcessError(res.returncode, "nvcc -c " + obj)
    subprocess.run([nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", LIB] +
                   [obj for obj, _ in results], check=True)
    return LIB


WAIT_TEST_LIB = os.path.join(PKG, "libsnn_b200_waittest.so")


def build_wait_test(force: bool = False) -> str:
    """Test-only variant of the library (used by one GPU test, never by the package): every bounded
    wait of the tcgen05 kernels limited to ~10 ms and a hook that makes the persistent forward
    kernel's producer skip one K stage, so the expiry path can be exercised."""
    build()                                   # the ordinary objects are reused for everything else
    src = os.path.join(CSRC, "linear_lif_tcgen05.cu")
    if (not force and os.path.exists(WAIT_TEST_LIB)
            and os.path.getmtime(WAIT_TEST_LIB) >= max(os.path.getmtime(src), os.path.getmtime(LIB))):
        return WAIT_TEST_LIB
    nvcc = os.environ.get("NVCC", "nvcc")
    objdir = os.path.join(PKG, "build")
    obj = os.path.join(objdir, "linear_lif_tcgen05_waittest.o")
    flags = [f for f in NVCC_FLAGS if f != "-shared"] + ["-DSNN_TC_WAIT_TEST", "-DSNN_TC_WAIT_CYCLES=20000000LL"]
    subprocess.run([nvcc] + flags + ["-c", "-o", obj, src], check=True)
    others = [os.path.join(objdir, os.path.basename(s)[:-3] + ".o") for s in sources() if s != src]
    subprocess.run([nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", WAIT_TEST_LIB, obj] + others,
                   check=True)
    return WAIT_TEST_LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
