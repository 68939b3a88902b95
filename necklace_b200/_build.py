"""Build the native library in-tree with nvcc for sm_100a.

``python -m necklace_b200._build`` compiles every ``csrc/*.cu`` to an object
file under ``build/`` and links ``necklace_b200/_nkb200.so``.  Objects are
rebuilt only when their source (or a header) is newer.  No GPU is needed: nvcc
cross-compiles.  The reference has no build step at all (its only kernels are
numba-JIT, necklace/cuda/quantize.py:16-91); this is the B200 counterpart.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
BUILD = os.path.join(os.path.dirname(HERE), "build", "nkb200")
LIB = os.path.join(HERE, "_nkb200.so")
# the bounds-checked debug variant (-DNKB_DEBUG_BOUNDS): ``--debug-bounds``
BUILD_DBG = os.path.join(os.path.dirname(HERE), "build", "nkb200_dbg")
LIB_DBG = os.path.join(HERE, "_nkb200_dbg.so")

ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "--use_fast_math",
              "-Xptxas", "-v", "-DNDEBUG"]


def _nvcc() -> str:
    cand = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(cand):
        raise RuntimeError("nvcc not found; cannot build necklace_b200 native library")
    return cand


def sources() -> list[str]:
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cu"))


def _headers_mtime() -> float:
    hs = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".h", ".cuh"))]
    return max((os.path.getmtime(h) for h in hs), default=0.0)


def _compile_one(src: str, force: bool, verbose: bool, debug_bounds: bool = False
                 ) -> tuple[str, str]:
    obj = os.path.join(BUILD_DBG if debug_bounds else BUILD, os.path.basename(src)[:-3] + ".o")
    newest = max(os.path.getmtime(src), _headers_mtime())
    if not force and os.path.exists(obj) and os.path.getmtime(obj) >= newest:
        return obj, ""
    extra = ["-DNKB_DEBUG_BOUNDS"] if debug_bounds else []
    cmd = [_nvcc(), *ARCH_FLAGS, *NVCC_FLAGS, *extra, "-I", CSRC, "-c", src, "-o", obj]
    p = subprocess.run(cmd, capture_output=True, text=True)
    log = p.stdout + p.stderr
    if p.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src}:\n{log}")
    with open(obj + ".log", "w") as f:
        f.write(log)
    if verbose:
        print(log)
    return obj, log


def build(force: bool = False, verbose: bool = False, debug_bounds: bool = False) -> str:
    """Compile and link; returns the path of the shared library.  ``debug_bounds`` builds the
    variant whose hand-indexed kernels check every index against the tensor extents."""
    bdir, lib = (BUILD_DBG, LIB_DBG) if debug_bounds else (BUILD, LIB)
    os.makedirs(bdir, exist_ok=True)
    srcs = sources()
    with ThreadPoolExecutor(max_workers=min(8, len(srcs))) as ex:
        results = list(ex.map(lambda s: _compile_one(s, force, verbose, debug_bounds), srcs))
    objs = [o for o, _ in results]
    relink = force or not os.path.exists(lib) or any(
        os.path.getmtime(o) > os.path.getmtime(lib) for o in objs)
    if relink:
        cmd = [_nvcc(), *ARCH_FLAGS, "-shared", "-Xcompiler", "-fPIC", "-o", lib, *objs,
               "-lcudart"]
        p = subprocess.run(cmd, capture_output=True, text=True)
        if p.returncode != 0:
            raise RuntimeError(f"link failed:\n{p.stdout}{p.stderr}")
    return lib


def resource_report() -> str:
    """Registers / spills / shared memory per kernel, from the saved ptxas logs."""
    out = []
    if not os.path.isdir(BUILD):
        return ""
    for f in sorted(os.listdir(BUILD)):
        if f.endswith(".o.log"):
            out.append(f"== {f[:-6]}")
            with open(os.path.join(BUILD, f)) as fh:
                out.append(fh.read())
    return "\n".join(out)


if __name__ == "__main__":
    lib = build(force="--force" in sys.argv, verbose="-v" in sys.argv,
                debug_bounds="--debug-bounds" in sys.argv)
    print(lib)
