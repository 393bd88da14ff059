"""Places the reference's own numpy sampler next to the oracle, so that the benchmark can time the reference's CPU path AS SHIPPED.

    python oracle/make_ref.py /path/to/lithos-metal

Copies ``monolith/nn/sampling_ref.py`` (71 lines of numpy, no other dependency) unchanged into ``oracle/_ref/``. That folder is
not under version control (the reference's sources never enter this repository's history); it travels to the GPU machine with
the working tree like the built libraries do. ``bench.py`` reports ``cpu_baseline_as_shipped`` from it when it is there and
says so when it is not. TEST / BENCHMARK INFRASTRUCTURE ONLY: nothing under ``lithos_metal_b200/`` may import it.
"""
from __future__ import annotations

import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
DEST = os.path.join(HERE, "_ref")


def make(ref_root: str) -> str:
    src = os.path.join(ref_root, "monolith", "nn", "sampling_ref.py")
    if not os.path.exists(src):
        raise FileNotFoundError(src)
    os.makedirs(DEST, exist_ok=True)
    shutil.copyfile(src, os.path.join(DEST, "sampling_ref.py"))
    return os.path.join(DEST, "sampling_ref.py")


def load():
    """The reference module, or None when oracle/_ref has not been made."""
    path = os.path.join(DEST, "sampling_ref.py")
    if not os.path.exists(path):
        return None
    import importlib.util
    spec = importlib.util.spec_from_file_location("lithos_reference_sampling_ref", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


if __name__ == "__main__":
    print(make(sys.argv[1] if len(sys.argv) > 1 else "/root/reference"))
