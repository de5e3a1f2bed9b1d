"""Builds libmsk_moe.so (the C-ABI library) in-tree with nvcc for sm_100a.

usage: python muse-spark-kernels_b200/build.py [--force] [--verbose]
"""
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OUT = os.path.join(HERE, "muse_moe_w4a16", "libmsk_moe.so")
SOURCES = ["msk_moe.cu"]
HEADERS = ["ptx.cuh", "layout.cuh", "route_sort.cuh", "small_tokens.cuh", "gemm.cuh", "gemm_producer.inl", "gemm_mma.inl",
           "gemm_gather.inl", "gemm_dequant.inl", "gemm_epilogue.inl", os.path.join("..", "..", "include", "msk_moe.h")]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",  # the explicit pair: -arch=sm_100a drops the 'a' features
    "-O3", "-lineinfo", "-std=c++17", "-shared", "-Xcompiler", "-fPIC",
]


def _nvcc():
    return shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"


def _stale():
    if not os.path.exists(OUT):
        return True
    t = os.path.getmtime(OUT)
    deps = [os.path.join(CSRC, f) for f in SOURCES + HEADERS]
    return any(os.path.getmtime(d) > t for d in deps)


def build_library(force=False, verbose=False):
    """Compile csrc/msk_moe.cu -> muse_moe_w4a16/libmsk_moe.so. Returns the .so path."""
    if not force and not _stale():
        return OUT
    cmd = [_nvcc()] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-o", OUT] + [
        os.path.join(CSRC, s) for s in SOURCES
    ]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed building libmsk_moe.so (exit %d)" % res.returncode)
    return OUT


if __name__ == "__main__":
    print(build_library(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
