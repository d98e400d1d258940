"""build.py: compiles libtkd.so (the CUDA kernels and their C-ABI) for sm_100a, in the tree, with nvcc.

    python tensix-kernels_b200/build.py [--verbose]

The library sits beside its sources (csrc/libtkd.so); the Python layer loads it with ctypes and refuses to work
without it. nvcc cross-compiles: no GPU is needed to build.
"""

import subprocess
import sys
from pathlib import Path

CSRC = Path(__file__).resolve().parent / "csrc"
SOURCES = ["tkd_api.cu", "tkd_pack.cu", "tkd_stream.cu", "tkd_topk.cu"]
LIB = CSRC / "libtkd.so"
FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17", "-shared",
    "-Xcompiler", "-fPIC",
]


def stale():
    if not LIB.exists():
        return True
    t = LIB.stat().st_mtime
    deps = list(CSRC.glob("*.cu")) + list(CSRC.glob("*.h")) + [CSRC.parents[1] / "include" / "tkd.h"]
    return any(d.stat().st_mtime > t for d in deps)


def build(verbose=False, force=False):
    if not force and not stale():
        return LIB
    cmd = ["nvcc", *FLAGS, *(["-Xptxas", "-v"] if verbose else []), "-o", str(LIB), *[str(CSRC / s) for s in SOURCES]]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or r.returncode:
        sys.stderr.write(r.stdout + r.stderr)
    if r.returncode:
        raise RuntimeError("nvcc failed building libtkd.so")
    return LIB


if __name__ == "__main__":
    build(verbose="--verbose" in sys.argv, force=True)
    print(LIB)
