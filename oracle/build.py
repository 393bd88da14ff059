"""Builds the CPU oracle (test infrastructure, not product code) into ``oracle/_build/liblm_oracle.so``.

The reference's CPU path for this hot path is Python/numpy, so nothing of the reference is compiled and there is
no ``oracle/_ref``; ``lm_oracle.c`` is a restatement. Run ``python oracle/build.py`` or call :func:`build`.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "lm_oracle.c")
OUT = os.path.join(HERE, "_build", "liblm_oracle.so")
# -ffp-contract=off: the integer-exact draw is specified operation by operation; the compiler must not fuse a*b+c
FLAGS = ["-O2", "-fPIC", "-shared", "-pthread", "-ffp-contract=off", "-fno-fast-math", "-fvisibility=hidden", "-Wall", "-Wextra"]


def build(force: bool = False) -> str:
    if not force and os.path.exists(OUT) and os.path.getmtime(OUT) >= os.path.getmtime(SRC):
        return OUT
    os.makedirs(os.path.dirname(OUT), exist_ok=True)
    subprocess.run(["gcc", *FLAGS, "-o", OUT, SRC, "-lm"], check=True)
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
