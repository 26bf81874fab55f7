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
# the same sources compiled with -DKH_GQA_MEASURE: the kernels honour KH_GQA_DEBUG (parts switched off so that the
# others can be timed, and the switch the abort-path test uses). Never loaded unless KH_GQA_LIBRARY=measure.
MEASURE_LIBRARY = PACKAGE_DIR / "libkhcuda_gqa_measure.so"
SOURCES = ["host_sdpa.cpp", "sdpa_api.cu", "sdpa_fp8.cu", "kv_page_write.cu", "bidi_block_sdpa.cu", "peer_exchange.cu"]
HEADERS = ["common.h", "cuda_objects.h", "host_sdpa.h", "map_instance.h", "sdpa_map.cuh", "sdpa_tc.cuh", "sdpa_tm.cuh", "../../include/kh_gqa.h"]


def nvcc_path() -> str:
    found = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(found).exists():
        raise RuntimeError("nvcc not found: libkhcuda_gqa.so cannot be built")
    return found


def is_stale(measure: bool = False) -> bool:
    library = MEASURE_LIBRARY if measure else LIBRARY
    if not library.exists():
        return True
    built = library.stat().st_mtime
    return any((CSRC / name).stat().st_mtime > built for name in SOURCES + HEADERS)


def build(force: bool = False, verbose: bool = False, measure: bool = False) -> Path:
    """Compile every CUDA and host source into one shared library. Returns its path. ``measure``: the
    measurement build (``-DKH_GQA_MEASURE``) instead of the product library."""
    library = MEASURE_LIBRARY if measure else LIBRARY
    if not force and not is_stale(measure):
        return library
    tmp = library.with_suffix(f".so.tmp{os.getpid()}")
    cmd = [
        nvcc_path(), "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
        "-Xcompiler", "-fPIC,-fvisibility=hidden,-Wall", "-shared", "-t", "4", "-cudart", "static",
        "-o", str(tmp),
    ] + [str(CSRC / name) for name in SOURCES]
    if measure:
        cmd.insert(1, "-DKH_GQA_MEASURE")
    if verbose:
        cmd.insert(1, "-Xptxas=-v")
    subprocess.run(cmd, check=True)
    os.replace(tmp, library)
    return library


if __name__ == "__main__":
    import sys
    print(build(force=True, verbose="-v" in sys.argv, measure="--measure" in sys.argv))
