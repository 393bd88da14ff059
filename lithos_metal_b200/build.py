"""Builds the CUDA library in-tree: ``lithos_metal_b200/_lib/liblithos_b200.so`` for sm_100a with nvcc.

``python -m lithos_metal_b200.build`` (or :func:`build`). The shared object has a plain C ABI (include/lithos_b200.h);
it is loaded with ctypes, so no Python headers and no torch headers are involved.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
SRC_DIR = os.path.join(HERE, "csrc")
OUT = os.path.join(HERE, "_lib", "liblithos_b200.so")
SOURCES = ["lithos_b200.cu"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17", "--shared", "-Xcompiler", "-fPIC,-fvisibility=hidden",
              "--fmad=true", "-Xptxas", "-v", "-cudart", "shared"]


def _nvcc() -> str:
    for cand in (shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found: the CUDA library cannot be built")


def _stale() -> bool:
    if not os.path.exists(OUT):
        return True
    t = os.path.getmtime(OUT)
    deps = [os.path.join(SRC_DIR, f) for f in os.listdir(SRC_DIR)] + [os.path.join(ROOT, "include", "lithos_b200.h"), os.path.abspath(__file__)]
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and not _stale():
        return OUT
    os.makedirs(os.path.dirname(OUT), exist_ok=True)
    cmd = [_nvcc(), *NVCC_FLAGS, "-I", os.path.join(ROOT, "include"), "-o", OUT, *[os.path.join(SRC_DIR, s) for s in SOURCES]]
    res = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    log = os.path.join(os.path.dirname(OUT), "build.log")
    with open(log, "w") as f:
        f.write(" ".join(cmd) + "\n" + res.stdout)
    if verbose or res.returncode != 0:
        print(res.stdout)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed (exit {res.returncode}); see {log}")
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose=True))
