"""Ahead-of-time build of libdeepgemm_b200.so (sm_100a only) with nvcc.

The library is built in-tree (deepgemm_b200/lib/) so that it travels with the source
checkout; there is no JIT and nothing is compiled at call time.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG_DIR, "csrc")
LIB_DIR = os.path.join(PKG_DIR, "lib")
LIB_PATH = os.environ.get("DEEPGEMM_B200_LIB") or os.path.join(LIB_DIR, "libdeepgemm_b200.so")
SOURCES = ["lib.cu", "gemm_inst_plain.cu", "gemm_inst_moe.cu", "gemm_inst_mxf4.cu", "gemm_inst_epi.cu",
           "gemm_inst_bf16.cu"]
PUBLIC_HEADER = os.path.join(PKG_DIR, "..", "include", "deepgemm_b200.h")


def dependencies():
    """Every file the library is built from: all sources and headers under csrc/ plus the public header."""
    files = [os.path.join(CSRC, f) for f in sorted(os.listdir(CSRC)) if f.endswith((".cu", ".cuh", ".h"))]
    return files + [PUBLIC_HEADER]


def nvcc_path() -> str:
    cand = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(cand):
        raise RuntimeError("nvcc not found; set NVCC or put it on PATH")
    return cand


def needs_build() -> bool:
    if not os.path.exists(LIB_PATH):
        return True
    t = os.path.getmtime(LIB_PATH)
    return any(os.path.exists(d) and os.path.getmtime(d) > t for d in dependencies())


def build(force: bool = False, verbose: bool = False, trace: bool = False) -> str:
    """Compile every CUDA source for sm_100a (one nvcc per source, in parallel) and link one shared library; returns
    its path.  trace=True builds a second library, lib/libdeepgemm_b200_trace.so, with -DDG_TRACE: the Mega MoE kernel
    then records per-CTA time stamps and wait cycles into a buffer given through dg_debug_set_trace (select it with the
    DEEPGEMM_B200_LIB environment variable; `bench.py --only mega_moe --trace <file>` summarises the stamps)."""
    lib_path = os.path.join(LIB_DIR, "libdeepgemm_b200_trace.so") if trace else LIB_PATH
    if not force and not trace and not needs_build():
        return LIB_PATH
    from concurrent.futures import ThreadPoolExecutor
    os.makedirs(LIB_DIR, exist_ok=True)
    obj_dir = os.path.join(LIB_DIR, "obj_trace" if trace else "obj")
    os.makedirs(obj_dir, exist_ok=True)
    nvcc = nvcc_path()
    flags = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC"]
    if verbose:
        flags += ["-Xptxas", "-v"]
    if trace:
        flags += ["-DDG_TRACE"]

    def compile_one(src):
        obj = os.path.join(obj_dir, os.path.splitext(src)[0] + ".o")
        res = subprocess.run([nvcc, *flags, "-c", os.path.join(CSRC, src), "-o", obj], capture_output=True, text=True)
        return src, obj, res

    with ThreadPoolExecutor(max_workers=len(SOURCES)) as pool:
        results = list(pool.map(compile_one, SOURCES))
    for src, _, res in results:
        if res.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src}:\n" + res.stdout + res.stderr)
        if verbose:
            sys.stderr.write(res.stderr)
    res = subprocess.run([nvcc, "-shared", "-o", lib_path] + [obj for _, obj, _ in results],
                         capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("linking failed:\n" + res.stdout + res.stderr)
    return lib_path


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv, trace="--trace" in sys.argv))
