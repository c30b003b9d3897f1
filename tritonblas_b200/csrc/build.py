"""Builds libtritonblas_b200.so in-tree with nvcc for sm_100a (cross-compiles without a GPU).

Usage: python tritonblas_b200/csrc/build.py [--force] [--verbose]   (run as a script: importing it through the
package would first try to load the library it builds)
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.dirname(HERE)
LIB = os.path.join(PKG, "libtritonblas_b200.so")
# the gemm_inst_* files hold the kernel instantiations (one MMA kind each) and dominate the build: they go first so that
# the parallel compile below starts them before the small files
SOURCES = ["gemm_inst_f16.cu", "gemm_inst_f8.cu", "gemm_inst_mxf4.cu", "gemm_inst_tf32.cu", "gemm_inst_i8.cu", "api.cu",
           "simt_gemm.cu", "quant_mxfp4.cu", "quant_fp8.cu", "moe_ops.cu", "push_tiles.cu", "stream_probe.cu", "selector.cpp"]
HEADERS_DIRS = [HERE, os.path.join(os.path.dirname(PKG), "include")]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
]


def _nvcc():
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.isabs(cand) and os.path.exists(cand) or not os.path.isabs(cand)):
            return cand
    return "nvcc"


def _inputs():
    files = []
    for d in HEADERS_DIRS:
        for f in sorted(os.listdir(d)):
            if f.endswith((".cu", ".cuh", ".cpp", ".h")):
                files.append(os.path.join(d, f))
    return files


def needs_build():
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    return any(os.path.getmtime(f) > t for f in _inputs())


def build(force=False, verbose=False):
    """Compile every source into one shared library; returns its path."""
    if not force and not needs_build():
        return LIB
    from concurrent.futures import ThreadPoolExecutor

    def compile_one(src):
        obj = os.path.join(HERE, os.path.splitext(src)[0] + ".o")
        cmd = [_nvcc(), *NVCC_FLAGS, "-c", os.path.join(HERE, src), "-o", obj]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
            print(" ".join(cmd), flush=True)
        subprocess.run(cmd, check=True)
        return obj

    with ThreadPoolExecutor(max_workers=min(len(SOURCES), os.cpu_count() or 1)) as pool:
        objs = list(pool.map(compile_one, SOURCES))
    cmd = [_nvcc(), "-shared", "-o", LIB, *objs, "-gencode", "arch=compute_100a,code=sm_100a"]
    if verbose:
        print(" ".join(cmd), flush=True)
    subprocess.run(cmd, check=True)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
