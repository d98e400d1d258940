"""build.py: compiles libtkd.so (the CUDA kernels and their C-ABI) for sm_100a, in the tree, with nvcc.

    python tensix-kernels_b200/build.py [--verbose]

The library sits beside its sources (csrc/libtkd.so); the Python layer loads it with ctypes and refuses to work
without it. nvcc cross-compiles: no GPU is needed to build.
"""

import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

CSRC = Path(__file__).resolve().parent / "csrc"
SOURCES = ["tkd_api.cu", "tkd_pack.cu", "tkd_stream.cu", "tkd_stream_bfp8.cu", "tkd_stream_bfp4.cu", "tkd_stream_bf16.cu",
           "tkd_stream_int4.cu", "tkd_hadamard.cu", "tkd_moe.cu",
           "tkd_topk.cu"]
LIB = CSRC / "libtkd.so"
FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17", "-Xcompiler", "-fPIC"]
OBJ = CSRC / "build"


def stale():
    if not LIB.exists():
        return True
    t = LIB.stat().st_mtime
    deps = list(CSRC.glob("*.cu")) + list(CSRC.glob("*.h")) + [CSRC.parents[1] / "include" / "tkd.h"]
    return any(d.stat().st_mtime > t for d in deps)


def _run(cmd, verbose):
    r = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or r.returncode:
        sys.stderr.write(r.stdout + r.stderr)
    if r.returncode:
        raise RuntimeError("nvcc failed building libtkd.so: " + " ".join(cmd))


def build(verbose=False, force=False, defines=(), lib=LIB):
    """Compile the sources (one nvcc per file, side by side) and link them. defines: extra -D flags (experiments)."""
    if not force and not defines and not stale():
        return lib
    OBJ.mkdir(exist_ok=True)
    extra = [*(["-Xptxas", "-v"] if verbose else []), *[f"-D{d}" for d in defines]]
    objs = [OBJ / (Path(s).stem + "".join("_" + d.replace("=", "_") for d in defines) + ".o") for s in SOURCES]
    with ThreadPoolExecutor(len(SOURCES)) as pool:
        list(pool.map(lambda so: _run(["nvcc", *FLAGS, *extra, "-c", "-o", str(so[1]), str(CSRC / so[0])], verbose),
                      zip(SOURCES, objs)))
    _run(["nvcc", "-gencode", "arch=compute_100a,code=sm_100a", "-shared", "-o", str(lib), *map(str, objs)], verbose)
    return lib


if __name__ == "__main__":
    build(verbose="--verbose" in sys.argv, force=True)
    print(LIB)
