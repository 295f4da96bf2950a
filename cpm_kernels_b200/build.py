"""Builds ``lib/libcpmk_b200.so`` from ``csrc/*.cu`` and the loadable kernel modules ``lib/gemm.fatbin`` /
``lib/gemv.fatbin`` from ``csrc/modules/*_module.cu`` with nvcc for sm_100a (cross-compiles without a GPU).

Usage: ``python -m cpm_kernels_b200.build [--force] [--verbose]``
"""
from __future__ import annotations

import glob
import os
import subprocess
import sys

_PKG = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(_PKG, "csrc")
LIB_DIR = os.path.join(_PKG, "lib")
LIB_PATH = os.path.join(LIB_DIR, "libcpmk_b200.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-shared", "-Xcompiler", "-fPIC",
    "--threads", "0",                      # one compilation per source file in parallel
]


MODULES = {"gemm": "gemm_module.cu", "gemv": "gemv_module.cu", "transpose": "transpose_module.cu"}
MODULE_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-fatbin"]


def module_path(name: str) -> str:
    """Path of the built kernel module ``name`` ("gemm", "gemv" or "transpose"): the file the reference's loader reads as
    ``cuda/<name>.fatbin`` (cpm_kernels/kernels/base.py:59-71)."""
    return os.path.join(LIB_DIR, name + ".fatbin")


def sources() -> list[str]:
    return sorted(glob.glob(os.path.join(CSRC, "*.cu")))


def _inputs() -> list[str]:
    root = os.path.dirname(_PKG)
    return sources() + glob.glob(os.path.join(CSRC, "*.cuh")) + glob.glob(os.path.join(CSRC, "*.h")) + \
        glob.glob(os.path.join(root, "include", "*.h")) + glob.glob(os.path.join(CSRC, "modules", "*"))


def is_stale() -> bool:
    if not os.path.exists(LIB_PATH) or not all(os.path.exists(module_path(n)) for n in MODULES):
        return True
    built = os.path.getmtime(LIB_PATH)
    return any(os.path.getmtime(p) > built for p in _inputs())


def build_library(force: bool = False, verbose: bool = False) -> str:
    """Compile the library if it is missing or older than its sources; return its path."""
    if not force and not is_stale():
        return LIB_PATH
    nvcc = os.environ.get("NVCC", "nvcc")
    os.makedirs(LIB_DIR, exist_ok=True)
    cmd = [nvcc] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-o", LIB_PATH] + sources()
    proc = subprocess.run(cmd, cwd=CSRC, capture_output=True, text=True)
    if verbose:
        sys.stderr.write(proc.stderr)
    if proc.returncode != 0:
        raise RuntimeError("nvcc failed:\n%s\n%s" % (" ".join(cmd), proc.stderr))
    for name, src in MODULES.items():
        cmd = [nvcc] + MODULE_FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-o", module_path(name), os.path.join("modules", src)]
        proc = subprocess.run(cmd, cwd=CSRC, capture_output=True, text=True)
        if verbose:
            sys.stderr.write(proc.stderr)
        if proc.returncode != 0:
            raise RuntimeError("nvcc failed:\n%s\n%s" % (" ".join(cmd), proc.stderr))
    # the library is written first, so a stale check against its time stamp also covers the modules
    os.utime(LIB_PATH, None)
    return LIB_PATH


if __name__ == "__main__":
    print(build_library(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
