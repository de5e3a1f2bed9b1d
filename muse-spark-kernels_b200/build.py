"""Builds libmsk_moe.so (the C-ABI library) in-tree with nvcc for sm_100a.

usage: python muse-spark-kernels_b200/build.py [--force] [--verbose]
"""
import ctypes
import hashlib
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OUT = os.path.join(HERE, "muse_moe_w4a16", "libmsk_moe.so")
SOURCES = ["msk_moe.cu"]
HEADERS = ["ptx.cuh", "layout.cuh", "route_sort.cuh", "router_gemm.cuh", "gemm.cuh", "gemm_producer.inl", "gemm_mma.inl",
           "gemm_gather.inl", "gemm_dequant.inl", "gemm_epilogue.inl", os.path.join("..", "..", "include", "msk_moe.h")]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",  # the explicit pair: -arch=sm_100a drops the 'a' features
    "-O3", "-lineinfo", "-std=c++17", "-shared", "-Xcompiler", "-fPIC",
]


def _nvcc():
    return shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"


def source_id():
    """Hash of every source and header the library is built from; compiled into the library
    (msk_build_id) so that a stale binary can be told from the sources beside it."""
    h = hashlib.sha256()
    for f in sorted(SOURCES + HEADERS):
        with open(os.path.join(CSRC, f), "rb") as fh:
            h.update(f.encode() + b"\0" + fh.read() + b"\0")
    return h.hexdigest()[:16]


def built_id(path=OUT):
    """msk_build_id() of a built library, or None when there is none / it cannot be loaded."""
    if not os.path.exists(path):
        return None
    try:
        lib = ctypes.CDLL(path)
        fn = lib.msk_build_id
        fn.restype = ctypes.c_char_p
        return fn().decode()
    except (OSError, AttributeError):
        return None


def _stale():
    return built_id() != source_id()


def build_library(force=False, verbose=False):
    """Compile csrc/msk_moe.cu -> muse_moe_w4a16/libmsk_moe.so. Returns the .so path."""
    if not force and not _stale():
        return OUT
    cmd = [_nvcc()] + NVCC_FLAGS + [f'-DMSK_BUILD_ID="{source_id()}"'] + (["-Xptxas", "-v"] if verbose else []) + ["-o", OUT] + [
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
