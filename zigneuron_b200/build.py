"""Builds libzn_b200.so in-tree from csrc/*.cu with nvcc for sm_100a.

    python zigneuron_b200/build.py        # incremental (run by path: importing the package needs the built library)
    python zigneuron_b200/build.py -f     # from scratch
"""
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "csrc", "build")
LIB = os.path.join(HERE, "libzn_b200.so")

NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
# ZN_DIAG=1 in the environment of the build adds -DZN_DIAG: the timing-only switches that give wrong results
# (a step without its gradient exchange, overridden descriptor strides) exist in such builds only.
FLAGS = [
    *(["-DZN_DIAG"] if os.environ.get("ZN_DIAG") else []),
    "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
    "-I", os.path.join(ROOT, "include"), "-I", CSRC,
]


def sources():
    return sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))


def _stale(target, deps):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def _compile(src, force):
    obj = os.path.join(OBJ, src[:-3] + ".o")
    # every header of the package is a dependency of every object (an edited activation formula in zn_act.cuh
    # must rebuild both GEMM families and the row-wise kernels)
    headers = [os.path.join(CSRC, f) for f in sorted(os.listdir(CSRC)) if f.endswith((".h", ".cuh"))]
    deps = [os.path.join(CSRC, src), *headers, os.path.join(ROOT, "include", "zn_b200.h")]
    if force or _stale(obj, deps):
        subprocess.check_call([NVCC, *FLAGS, "-c", os.path.join(CSRC, src), "-o", obj])
    return obj


def build(force=False, verbose=False):
    os.makedirs(OBJ, exist_ok=True)
    with ThreadPoolExecutor(max_workers=8) as pool:
        objs = list(pool.map(lambda s: _compile(s, force), sources()))
    if force or _stale(LIB, objs):
        subprocess.check_call([NVCC, "-gencode", "arch=compute_100a,code=sm_100a", "-shared", "-o", LIB, *objs, "-ldl"])
    if verbose:
        print(LIB)
    return LIB


if __name__ == "__main__":
    build(force="-f" in sys.argv[1:], verbose=True)
