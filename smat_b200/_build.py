"""Builds smat_b200/libsmat_b200.so in-tree with nvcc for sm_100a (cross-compiles without a GPU)."""
import os
import shutil
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.environ.get("SMAT_LIB", os.path.join(HERE, "libsmat_b200.so"))
SOURCES = ["spmm_sm100.cu", "spmm_tall_sm100.cu", "plan.cu", "spmm_static.cu", "bcsr_build.cu", "capi.cu", "mtx_reader.cpp", "reorder.cpp", "knapsack.cpp", "vbr_build.cpp"]
HEADERS = ["ptx_sm100.cuh", "spmm_sched.cuh", "smat_internal.h", os.path.join("..", "..", "include", "smat_b200.h")]


def _nvcc():
    for cand in (shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found")


def needs_build():
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    deps = [os.path.join(CSRC, s) for s in SOURCES + HEADERS]
    return any(os.path.getmtime(d) > t for d in deps)


def build(force=False, verbose=False):
    if not force and not needs_build():
        return LIB
    cmd = [_nvcc(), "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-shared",
           "-Xcompiler", "-fPIC,-pthread", "-ccbin", "g++", "-o", LIB] + [os.path.join(CSRC, s) for s in SOURCES]
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
    if os.environ.get("SMAT_DEFS"):
        for d in os.environ["SMAT_DEFS"].split():
            cmd.insert(1, "-D" + d)
    subprocess.check_call(cmd, cwd=CSRC)
    return LIB


if __name__ == "__main__":
    import sys
    print(build(force=True, verbose="-v" in sys.argv))
