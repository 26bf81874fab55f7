"""Builds ``libkhcuda_gqa.so`` in-tree with nvcc for sm_100a.

A Rust ``inference-backend-cuda`` crate that binds the library would run the same nvcc command from its
``build.rs``; this module is what the Python harness and the tests use.
"""
from __future__ import annotations

import os
import shutil
import subprocess
from pathlib import Path

PACKAGE_DIR = Path(__file__).resolve().parent
CSRC = PACKAGE_DIR / "csrc"
LIBRARY = PACKAGE_DIR / "libkhcuda_gqa.so"
SOURCES = ["host_sdpa.cpp", "sdpa_api.cu", "sdpa_fp8.cu", "kv_page_write.cu"]
HEADERS = ["common.h", "cuda_objects.h", "host_sdpa.h", "map_instance.h", "sdpa_map.cuh", "sdpa_tc.cuh", "../../include/kh_gqa.h"]


def nvcc_path() -> str:
    found = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(found).exists():
        raise RuntimeError("nvcc not found: libkhcuda_gqa.so cannot be built")
    return found


def is_stale() -> bool:
    if not LIBRARY.exists():
        return True
    built = LIBRARY.stat().st_mtime
    return any((CSRC / name).stat().st_mtime > built for name in SOURCES + HEADERS)


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile every CUDA and host source into one shared library. Returns its path."""
    if not force and not is_stale():
        return LIBRARY
    tmp = LIBRARY.with_suffix(f".so.tmp{os.getpid()}")
    cmd = [
        nvcc_path(), "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
        "-Xcompiler", "-fPIC,-fvisibility=hidden,-Wall", "-shared", "-t", "4", "-cudart", "static",
        "-o", str(tmp),
    ] + [str(CSRC / name) for name in SOURCES]
    if verbose:
        cmd.insert(1, "-Xptxas=-v")
    subprocess.run(cmd, check=True)
    os.replace(tmp, LIBRARY)
    return LIBRARY


if __name__ == "__main__":
    print(build(force=True, verbose=True))
