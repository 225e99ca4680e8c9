"""Builds the native libraries in-tree.

* ``gcore_b200/ops/_gk_kernels.so``   - every CUDA kernel, compiled for sm_100a only.
* ``gcore_b200/runtime/_gk_runtime.so`` - host-side C++ runtime (rollout scheduler, KV block manager, bucket
  planner, sequence balancing); needs only g++.

The libraries export a plain C ABI and are loaded with ``ctypes`` (see ``gcore_b200/ops/_lib.py``); nothing is
JIT-compiled at run time, so a box without a compiler can run a tree that was built elsewhere.

Usage: ``python -m gcore_b200.build_native [--force] [--verbose]``
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

ROOT = Path(__file__).resolve().parent
OPS_SRC = ROOT / "ops" / "csrc"
RT_SRC = ROOT / "runtime" / "csrc"
BUILD = ROOT.parent / "build"
KERNEL_LIB = ROOT / "ops" / "_gk_kernels.so"
RUNTIME_LIB = ROOT / "runtime" / "_gk_runtime.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo", "--use_fast_math",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
    "--expt-relaxed-constexpr",
]
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-fvisibility=hidden", "-Wall", "-pthread"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found")


def _digest(paths) -> str:
    h = hashlib.sha256()
    for p in sorted(paths):
        h.update(p.name.encode())
        h.update(p.read_bytes())
    return h.hexdigest()


def _run(cmd, verbose):
    if verbose:
        print(" ".join(map(str, cmd)), flush=True)
    r = subprocess.run(list(map(str, cmd)), capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"command failed: {' '.join(map(str, cmd))}\n{r.stdout}\n{r.stderr}")
    if verbose and (r.stdout or r.stderr):
        print(r.stdout, r.stderr)
    return r


def build_kernels(force=False, verbose=False, ptxas_info=False) -> Path:
    srcs = sorted(OPS_SRC.glob("*.cu"))
    hdrs = sorted(list(OPS_SRC.glob("*.cuh")) + list(OPS_SRC.glob("*.h")))
    stamp = BUILD / "kernels.sha"
    dig = _digest(srcs + hdrs)
    if not force and KERNEL_LIB.exists() and stamp.exists() and stamp.read_text() == dig:
        return KERNEL_LIB
    BUILD.mkdir(exist_ok=True)
    nvcc = _nvcc()
    hdr_dig = _digest(hdrs)

    def compile_one(src: Path) -> Path:
        obj = BUILD / (src.stem + ".o")
        ostamp = BUILD / (src.stem + ".sha")
        d = hashlib.sha256(src.read_bytes() + hdr_dig.encode()).hexdigest()
        if not force and obj.exists() and ostamp.exists() and ostamp.read_text() == d:
            return obj
        flags = list(NVCC_FLAGS)
        if ptxas_info:
            flags += ["-Xptxas", "-v"]
        r = _run([nvcc, *flags, "-I", OPS_SRC, "-c", src, "-o", obj], verbose)
        if ptxas_info:
            (BUILD / (src.stem + ".ptxas.txt")).write_text(r.stderr)
        ostamp.write_text(d)
        return obj

    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 2)) as ex:
        objs = list(ex.map(compile_one, srcs))
    _run([nvcc, "-shared", "-o", KERNEL_LIB, *objs, "-lcudart"], verbose)
    stamp.write_text(dig)
    return KERNEL_LIB


def build_runtime(force=False, verbose=False) -> Path:
    srcs = sorted(RT_SRC.glob("*.cpp"))
    hdrs = sorted(RT_SRC.glob("*.h"))
    stamp = BUILD / "runtime.sha"
    dig = _digest(srcs + hdrs)
    if not force and RUNTIME_LIB.exists() and stamp.exists() and stamp.read_text() == dig:
        return RUNTIME_LIB
    BUILD.mkdir(exist_ok=True)
    cxx = os.environ.get("CXX", "g++")
    _run([cxx, *CXX_FLAGS, "-shared", "-o", RUNTIME_LIB, *srcs], verbose)
    stamp.write_text(dig)
    return RUNTIME_LIB


def build_all(force=False, verbose=False, ptxas_info=False):
    return build_kernels(force, verbose, ptxas_info), build_runtime(force, verbose)


if __name__ == "__main__":
    args = set(sys.argv[1:])
    libs = build_all("--force" in args, "--verbose" in args, "--ptxas" in args)
    for lib in libs:
        print(f"built {lib} ({lib.stat().st_size/1e6:.2f} MB)")
