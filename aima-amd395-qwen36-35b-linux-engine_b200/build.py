"""Builds libaima_moe_b200.so (sm_100a) in place with nvcc.

The library links the CUDA runtime statically and has no Python or PyTorch
dependency; it is the artefact C++ hosts dlopen and Python loads with ctypes.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
LIB = HERE / "libaima_moe_b200.so"
SOURCES = ["moe_api.cu", "decode_kernel.cu", "decode_noalloc.cu", "pointwise.cu", "prefill.cu",
           "grouped_gemm_simt.cu", "grouped_gemm_tc.cu", "lm_head.cu", "lm_head_api.cu",
           "image_loader.cu"]


def nvcc_path() -> str:
    for candidate in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if candidate and Path(candidate).exists():
            return candidate
    raise RuntimeError("nvcc not found; the CUDA library cannot be built")


def needs_build() -> bool:
    if not LIB.exists():
        return True
    newest = max(p.stat().st_mtime for p in list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh"))
                 + [HERE.parent / "include" / "aima_moe.h", Path(__file__)])
    return newest > LIB.stat().st_mtime


def build(force: bool = False, verbose: bool = False) -> Path:
    if not force and not needs_build():
        return LIB
    command = [
        nvcc_path(), "-std=c++17", "-O3", "-lineinfo", "-shared", "-Xcompiler", "-fPIC",
        "-Xcompiler", "-fvisibility=hidden",
        "-gencode", "arch=compute_100a,code=sm_100a",
        "-ccbin", shutil.which("g++") or "g++",
        "-o", str(LIB),
    ]
    if verbose:
        command += ["-Xptxas", "-v"]
    command += [str(CSRC / name) for name in SOURCES]
    result = subprocess.run(command, capture_output=True, text=True)
    if result.returncode != 0:
        sys.stderr.write(result.stdout + result.stderr)
        raise RuntimeError("nvcc failed building libaima_moe_b200.so")
    if verbose:
        sys.stderr.write(result.stderr)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
