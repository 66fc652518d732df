"""Builds libgometal_host.so: the C++ mirror of go-metal's optimizer host side.

Usage: python go-metal_b200/host/build.py [--force]
Needs only g++; the CUDA library is loaded at run time (dlopen), not linked.
"""
from __future__ import annotations

import glob
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
LIB = os.path.join(os.path.dirname(HERE), "lib", "libgometal_host.so")


def build(force: bool = False) -> str:
    os.makedirs(os.path.dirname(LIB), exist_ok=True)
    sources = sorted(glob.glob(os.path.join(HERE, "*.cpp")))
    deps = sources + glob.glob(os.path.join(HERE, "*.hpp"))
    stale = not os.path.exists(LIB) or any(os.path.getmtime(d) > os.path.getmtime(LIB) for d in deps)
    if force or stale:
        cmd = ["g++", "-std=c++17", "-O2", "-fPIC", "-shared", "-Wall", "-Wextra", "-fvisibility=hidden",
               "-o", LIB] + sources + ["-ldl", "-lpthread"]
        subprocess.run(cmd, check=True)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
