"""Builds libesmm_b200.so (the C-ABI library), libesmm_b200_checked.so (the same sources with their shape- and data-dependent
shared- and global-memory indices bounds-checked), exec_b200 (the driver CLI) and cusparse_bench in-tree with
nvcc for sm_100a.  Usage: `python build.py [--force] [--verbose]`."""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
LIB = os.path.join(HERE, "libesmm_b200.so")
LIB_CHECKED = os.path.join(HERE, "libesmm_b200_checked.so")   # same sources with -DESMM_CHECKED: the sanitizer substitute
EXE = os.path.join(HERE, "exec_b200")
SPARSE_EXE = os.path.join(HERE, "cusparse_bench")
SPARSE_SRC = os.path.join(HERE, "cusparse_bench.cu")
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON = ["-O3", "-std=c++17", "-lineinfo"] + ARCH

LIB_SRCS = [os.path.join(HERE, "csrc", f) for f in
            ("esmm_gemm.cu", "esmm_gemm_packed.cu", "esmm_gemm_skinny.cu", "esmm_preprocess.cu", "esmm_api.cu", "esmm_noalloc.cu",
             "esmm_cusparse.cu", "esmm_gemm_tf32.cu", "esmm_host.cu", "esmm_multi.cu")]
LIB_DEPS = LIB_SRCS + [os.path.join(HERE, "csrc", "esmm_common.cuh"), os.path.join(HERE, "csrc", "esmm_gemm_shared.cuh"), os.path.join(ROOT, "include", "esmm.h")]
EXE_SRCS = [os.path.join(HERE, "driver.cu")]
EXE_DEPS = EXE_SRCS + [os.path.join(ROOT, "include", h) for h in ("runners.cuh", "utils.cuh", "esmm.h")]


def _stale(target: str, deps: list[str]) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.exists(d) and os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    srcs = [s for s in LIB_SRCS if os.path.exists(s)]
    if force or _stale(LIB, LIB_DEPS):
        cmd = [NVCC] + COMMON + (["-Xptxas", "-v"] if verbose else []) + \
              ["-Xcompiler", "-fPIC", "-shared", "-o", LIB] + srcs + ["-lcublas", "-lcusparse", "-ldl"]
        print("+", " ".join(cmd), flush=True)
        subprocess.check_call(cmd)
    if force or _stale(LIB_CHECKED, LIB_DEPS):
        cmd = [NVCC] + COMMON + ["-DESMM_CHECKED", "-Xcompiler", "-fPIC", "-shared", "-o", LIB_CHECKED] + srcs + \
              ["-lcublas", "-lcusparse", "-ldl"]
        print("+", " ".join(cmd), flush=True)
        subprocess.check_call(cmd)
    if os.path.exists(EXE_SRCS[0]) and (force or _stale(EXE, EXE_DEPS + [LIB])):
        cmd = [NVCC] + COMMON + ["-I" + ROOT, "-o", EXE] + EXE_SRCS + \
              ["-L" + HERE, "-lesmm_b200", "-Xlinker", "-rpath", "-Xlinker", "$ORIGIN"]
        print("+", " ".join(cmd), flush=True)
        subprocess.check_call(cmd)
    if os.path.exists(SPARSE_SRC) and (force or _stale(SPARSE_EXE, [SPARSE_SRC, os.path.join(ROOT, "include", "esmm.h"), LIB])):
        cmd = [NVCC] + COMMON + ["-I" + ROOT, "-o", SPARSE_EXE, SPARSE_SRC,
                                 "-L" + HERE, "-lesmm_b200", "-Xlinker", "-rpath", "-Xlinker", "$ORIGIN"]
        print("+", " ".join(cmd), flush=True)
        subprocess.check_call(cmd)
    return LIB


if __name__ == "__main__":
    build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
