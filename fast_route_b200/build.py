"""Builds ``libfastroute_sm100.so`` in-tree with nvcc for sm_100a.

    python -m fast_route_b200.build [--force] [--verbose]

nvcc cross-compiles without a GPU.  The library is one translation unit
(``csrc/fastroute_sm100.cu``) linked against the static CUDA runtime; the driver API entry
point for tensor maps is resolved at run time, so nothing links against libcuda.
"""

from __future__ import annotations

import glob
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OUT = os.path.join(HERE, "libfastroute_sm100.so")
ROOT = os.path.dirname(HERE)

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-std=c++17", "-O3", "-lineinfo",
              "--shared", "-Xcompiler", "-fPIC"]


def sources():
    files = glob.glob(os.path.join(CSRC, "*.cu")) + glob.glob(os.path.join(CSRC, "*.cuh"))
    files += glob.glob(os.path.join(ROOT, "include", "*.h"))
    return files


def up_to_date() -> bool:
    if not os.path.exists(OUT):
        return False
    t = os.path.getmtime(OUT)
    return all(os.path.getmtime(f) <= t for f in sources())


def find_nvcc() -> str:
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found; it is needed to build libfastroute_sm100.so")
    return nvcc


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and up_to_date():
        return OUT
    cmd = [find_nvcc()] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else [])
    cmd += ["-o", OUT, os.path.join(CSRC, "fastroute_sm100.cu")]
    proc = subprocess.run(cmd, cwd=CSRC, capture_output=True, text=True)
    if verbose or proc.returncode != 0:
        sys.stderr.write(proc.stdout + proc.stderr)
    if proc.returncode != 0:
        raise RuntimeError("nvcc failed building libfastroute_sm100.so")
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
