"""Builds libstk_b200.so (sm_100a only) next to the Python package with plain nvcc.

Run as ``python -m stk_b200.csrc.build``; ``stk_b200.backend.lib`` loads the result with ctypes.
The library links the CUDA runtime statically and nothing else (the one driver call it needs,
cuTensorMapEncodeTiled, is looked up at run time), so it does not depend on torch's C++ ABI.
"""
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.dirname(HERE)
LIB_PATH = os.path.join(PKG, "libstk_b200.so")
SOURCES = ["stk_b200.cu"]
HEADERS = ["bsmm_sm100.cuh", "bsmm_pair_sm100.cuh", "bsmm_wide_sm100.cuh", "bsmm_row_sm100.cuh", "bsmm_api.cuh", "meta_sm100.cuh", "plan_sm100.cuh", "index.cuh", "dmoe_sm100.cuh", "sm100_ptx.cuh", "status.cuh",
           os.path.join("..", "..", "include", "stk_b200.h")]


def _nvcc():
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found; set NVCC or install the CUDA toolkit")


def is_stale():
    if not os.path.exists(LIB_PATH):
        return True
    built = os.path.getmtime(LIB_PATH)
    deps = [os.path.join(HERE, f) for f in SOURCES + HEADERS]
    return any(os.path.getmtime(d) > built for d in deps)


def build(force=False, verbose=False):
    """Compile the library if it is missing or older than its sources; return its path."""
    if not force and not is_stale():
        return LIB_PATH
    cmd = [
        _nvcc(), "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo",
        "--shared", "-Xcompiler", "-fPIC", "-cudart", "static",
        "-o", LIB_PATH,
    ] + [os.path.join(HERE, s) for s in SOURCES]
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + proc.stdout + proc.stderr)
    if verbose:
        print(proc.stdout + proc.stderr)
    return LIB_PATH


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
