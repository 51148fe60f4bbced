"""Compiles swiftrt_b200/csrc into swiftrt_b200/libsrt_b200.so with nvcc for sm_100a.

The library is built in-tree so that it travels with the source checkout; nothing is
installed into site-packages and nothing is JIT-compiled at import time.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
SO = os.path.join(PKG, "libsrt_b200.so")
SOURCES = [os.path.join(PKG, "csrc", "srt_matmul.cu")]
HEADERS = [os.path.join(PKG, "csrc", h) for h in ("ptx.cuh", "gemm_tcgen05.cuh", "gemm_simt.cuh", "gemm_splitk.cuh",
                                                  "dense_backward.cuh", "lstm_cell.cuh")] + [
    os.path.join(ROOT, "include", "srt_matmul_api.h")]

# the explicit -gencode form is required: a bare -arch=sm_100a does not enable tcgen05
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-shared", "-Xcompiler", "-fPIC", "-I" + os.path.join(ROOT, "include")]


def nvcc_path() -> str:
    path = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(path):
        raise RuntimeError("nvcc not found: the CUDA library cannot be built")
    return path


def needs_build() -> bool:
    if not os.path.exists(SO):
        return True
    t = os.path.getmtime(SO)
    return any(os.path.getmtime(f) > t for f in SOURCES + HEADERS)


def build(force: bool = False, verbose: bool = False) -> str:
    """Builds the shared library if a source is newer than it; returns its path."""
    if force or needs_build():
        cmd = [nvcc_path()] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-o", SO] + SOURCES
        env = dict(os.environ)
        env.pop("CC", None)
        env.pop("CXX", None)
        res = subprocess.run(cmd, capture_output=True, text=True, env=env)
        if verbose:
            sys.stderr.write(res.stderr)
        if res.returncode != 0:
            raise RuntimeError("nvcc failed:\n" + res.stdout + res.stderr)
    return SO


HOST_TEST_SRC = os.path.join(ROOT, "tests", "cpp", "test_host_kat.cpp")
HOST_TEST_BIN = os.path.join(ROOT, "tests", "cpp", "test_host_kat")


def build_host_test(force: bool = False) -> str:
    """Compiles the C++ host-mirror test program (tests/cpp) against the built library."""
    deps = [HOST_TEST_SRC, os.path.join(PKG, "host", "srt_host.hpp"), HEADERS[-1]]
    if force or not os.path.exists(HOST_TEST_BIN) or any(os.path.getmtime(f) > os.path.getmtime(HOST_TEST_BIN) for f in deps):
        build()
        cmd = [nvcc_path(), "-std=c++17", "-O1", "-Wno-deprecated-gpu-targets", "-I" + os.path.join(ROOT, "include"),
               "-I" + os.path.join(PKG, "host"), "-o", HOST_TEST_BIN, HOST_TEST_SRC, "-L" + PKG, "-lsrt_b200",
               "-Xlinker", "-rpath", "-Xlinker", "$ORIGIN/../../swiftrt_b200"]
        env = dict(os.environ)
        env.pop("CC", None)
        env.pop("CXX", None)
        res = subprocess.run(cmd, capture_output=True, text=True, env=env)
        if res.returncode != 0:
            raise RuntimeError("nvcc failed on the host test:\n" + res.stdout + res.stderr)
    return HOST_TEST_BIN


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
    print(build_host_test(force="--force" in sys.argv))
