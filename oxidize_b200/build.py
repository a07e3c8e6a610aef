"""Builds the native libraries in-tree with nvcc / g++ (no torch headers, seconds per file).

``liboxb.so``  — sm_100a CUDA kernels (``csrc/oxb*.cu``: translation units compiled in parallel as relocatable
device code and linked, device link included, into one shared object)
``liboxbrt.so`` — host runtime pieces in C++ (``csrc/runtime.cpp``)
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")

ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ARCH_FLAGS + ["-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC", "-Xcompiler",
                           "-fvisibility=hidden"]


def _newer(target: str, sources) -> bool:
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(s) <= t for s in sources)


def _sources(exts):
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(exts))


def build_kernels(force: bool = False, verbose: bool = False) -> str:
    out = os.path.join(CSRC, "liboxb.so")
    srcs = _sources((".cu", ".cuh", ".h"))
    if not force and _newer(out, srcs):
        return out
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    units = [s for s in srcs if s.endswith(".cu")]
    headers = [s for s in srcs if not s.endswith(".cu")]
    objdir = os.path.join(CSRC, "build")
    os.makedirs(objdir, exist_ok=True)
    hdr_time = max(os.path.getmtime(h) for h in headers)

    def compile_unit(src: str):
        obj = os.path.join(objdir, os.path.basename(src)[:-3] + ".o")
        if not force and os.path.exists(obj) and os.path.getmtime(obj) >= max(os.path.getmtime(src), hdr_time):
            return obj, ""
        cmd = [nvcc] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-c", "-o", obj, src]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed on {os.path.basename(src)}:\n" + r.stdout + r.stderr)
        return obj, r.stderr

    from concurrent.futures import ThreadPoolExecutor

    with ThreadPoolExecutor(max_workers=max(1, min(len(units), os.cpu_count() or 4))) as ex:
        results = list(ex.map(compile_unit, units))
    if verbose:
        for _, err in results:
            sys.stderr.write(err)
    link = [nvcc] + ARCH_FLAGS + ["--shared", "-Xcompiler", "-fPIC", "-o", out] + [o for o, _ in results]
    r = subprocess.run(link, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("nvcc link failed:\n" + r.stdout + r.stderr)
    return out


def build_runtime(force: bool = False) -> str:
    out = os.path.join(CSRC, "liboxbrt.so")
    srcs = _sources((".cpp", ".hpp", ".h"))
    cpps = [s for s in srcs if s.endswith(".cpp") and os.path.basename(s) != "ffi.cpp"]  # ffi.cpp: build_ffi
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


def build_ffi(force: bool = False) -> str:
    """``liboxidize_ffi.so``: the C ABI over the whole engine (``csrc/oxidize_ffi.h``), a shim that embeds this Python
    interpreter.  The interpreter's path and the package's location are compiled in as defaults."""
    import sysconfig

    src = os.path.join(CSRC, "ffi.cpp")
    out = os.path.join(CSRC, "liboxidize_ffi.so")
    inc = sysconfig.get_config_var("INCLUDEPY") or ""
    if not os.path.exists(src) or not os.path.exists(os.path.join(inc, "Python.h")):
        return ""  # no interpreter headers on this machine: the engine itself does not need the shim
    if not force and _newer(out, [src, os.path.join(CSRC, "oxidize_ffi.h")]):
        return out
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    libdir = sysconfig.get_config_var("LIBDIR") or ""
    cxx = shutil.which("g++") or "g++"
    cmd = [cxx, "-O2", "-std=c++17", "-shared", "-fPIC", "-o", out, src, f"-I{inc}", f"-L{libdir}",
           f"-lpython{sysconfig.get_config_var('LDVERSION')}", f"-Wl,-rpath,{libdir}",
           f'-DOXIDIZE_DEFAULT_PYTHON="{sys.executable}"', f'-DOXIDIZE_DEFAULT_ROOT="{root}"']
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("g++ (ffi) failed:\n" + r.stdout + r.stderr)
    return out


def build_all(force: bool = False, verbose: bool = False):
    return build_kernels(force, verbose), build_runtime(force), build_ffi(force)


if __name__ == "__main__":
    print(build_all(force="--force" in sys.argv, verbose="-v" in sys.argv))
