"""Builds the native libraries in-tree with nvcc / g++ (no torch headers, seconds per file).

``liboxb.so``  — sm_100a CUDA kernels (``csrc/oxb.cu``, one translation unit)
``liboxbrt.so`` — host runtime pieces in C++ (``csrc/runtime.cpp``)
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "--shared",
              "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden"]


def _newer(target: str, sources) -> bool:
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(s) <= t for s in sources)


def _sources(exts):
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(exts))


def build_kernels(force: bool = False, verbose: bool = False) -> str:
    out = os.path.join(CSRC, "liboxb.so")
    srcs = _sources((".cu", ".cuh"))
    if not force and _newer(out, srcs):
        return out
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    cmd = [nvcc] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-o", out, os.path.join(CSRC, "oxb.cu")]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + r.stdout + r.stderr)
    if verbose:
        sys.stderr.write(r.stderr)
    return out


def build_runtime(force: bool = False) -> str:
    out = os.path.join(CSRC, "liboxbrt.so")
    srcs = _sources((".cpp", ".hpp", ".h"))
    cpps = [s for s in srcs if s.endswith(".cpp")]
    if not cpps:
        return ""
    if not force and _newer(out, srcs):
        return out
    cxx = shutil.which("g++") or "g++"
    cmd = [cxx, "-O2", "-std=c++17", "-shared", "-fPIC", "-fvisibility=hidden", "-o", out] + cpps
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("g++ failed:\n" + r.stdout + r.stderr)
    return out


def build_all(force: bool = False, verbose: bool = False):
    return build_kernels(force, verbose), build_runtime(force)


if __name__ == "__main__":
    print(build_all(force="--force" in sys.argv, verbose="-v" in sys.argv))
