"""Compile tests/cpp/test_operators.cpp: the C++ operator classes and the C operator handles against the
CPU oracle (oracle/libsdfl_oracle.so is linked as the checker).  Test infrastructure: nothing in the
product package calls this.

    python tests/cpp/build.py
"""
from __future__ import annotations

import os
import shutil
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
PKG = "mobile-stable-diffusion_b200"


def build() -> str:
    src = os.path.join(HERE, "test_operators.cpp")
    exe = os.path.join(HERE, "test_operators")
    deps = [src, os.path.join(ROOT, "include", "sdfl_operators.hpp"), os.path.join(ROOT, "include", "sdfl.h"),
            os.path.join(ROOT, PKG, "lib", "libsdfl.so")]
    if os.path.exists(exe) and all(os.path.getmtime(d) <= os.path.getmtime(exe) for d in deps if os.path.exists(d)):
        return exe
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    cmd = [nvcc, "-O2", "-std=c++17", src, "-o", exe, "-L" + os.path.join(ROOT, PKG, "lib"), "-lsdfl",
           "-L" + os.path.join(ROOT, "oracle"), "-lsdfl_oracle",
           "-Xlinker", "-rpath,$ORIGIN/../../" + PKG + "/lib", "-Xlinker", "-rpath,$ORIGIN/../../oracle"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"C++ test build failed:\n{r.stdout}\n{r.stderr}")
    return exe


if __name__ == "__main__":
    print(build())
