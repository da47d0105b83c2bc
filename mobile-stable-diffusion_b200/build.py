"""Build libsdfl.so (the CUDA kernels + C ABI) in-tree with nvcc, for sm_100a only.

    python mobile-stable-diffusion_b200/build.py [--force] [--verbose]

Objects go to <package>/build/, the library to <package>/lib/libsdfl.so.  ptxas resource usage
(-Xptxas -v) of every kernel is kept in <package>/build/ptxas.log.
"""
from __future__ import annotations

import concurrent.futures as cf
import os
import shutil
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
BUILD = os.path.join(PKG, "build")
LIBDIR = os.path.join(PKG, "lib")
LIB = os.path.join(LIBDIR, "libsdfl.so")

SOURCES = ["groupnorm.cu", "gn_ring.cu", "gn_multi.cu", "gn_register.cu", "gn_split.cu", "layernorm.cu", "elementwise.cu", "embedding.cu", "permute.cu", "softmax.cu", "resample.cu", "capi.cu"]
HEADERS = [os.path.join(CSRC, "common.cuh"), os.path.join(CSRC, "kernels.h"),
           os.path.join(CSRC, "gn_internal.h"), os.path.join(CSRC, "gn_device.cuh"),
           os.path.join(ROOT, "include", "sdfl.h")]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC,-O2,-Wall",
    "-Xptxas", "-v",
]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found: the CUDA toolkit is required to build libsdfl.so")
    return exe


def _stale(target: str, deps: list[str]) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def _compile(src: str, obj: str) -> str:
    cmd = [_nvcc(), *NVCC_FLAGS, "-c", os.path.join(CSRC, src), "-o", obj]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed on {src}:\n{r.stdout}\n{r.stderr}")
    return f"==== {src}\n{r.stderr}"


def build(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(BUILD, exist_ok=True)
    os.makedirs(LIBDIR, exist_ok=True)
    objs, jobs = [], []
    for src in SOURCES:
        obj = os.path.join(BUILD, src.replace(".cu", ".o"))
        objs.append(obj)
        if force or _stale(obj, [os.path.join(CSRC, src), *HEADERS, os.path.abspath(__file__)]):
            jobs.append((src, obj))
    if jobs:
        with cf.ThreadPoolExecutor(max_workers=len(jobs)) as ex:
            logs = list(ex.map(lambda j: _compile(*j), jobs))
        with open(os.path.join(BUILD, "ptxas.log"), "a" if not force else "w") as f:
            f.write("\n".join(logs))
        if verbose:
            print("\n".join(logs))
    if jobs or force or _stale(LIB, objs):
        cmd = [_nvcc(), "-shared", "-o", LIB, *objs, "-cudart", "static"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
