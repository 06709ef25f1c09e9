"""Compile the CUDA sources into cula_b200/lib/libcula_kda.so for sm_100a with nvcc.

    python -m cula_b200.build [--force] [--verbose]

The library is built in-tree and loaded with ctypes (cula_b200/_native.py); it has a plain C ABI
(include/cula_kda.h) and links only against the CUDA runtime (the one driver function it needs, the tensor-map encoder
of the dense backward stage, is looked up through the runtime's driver entry point at first use).
"""
from __future__ import annotations

import glob
import os
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG, "csrc")
LIB_DIR = os.path.join(PKG, "lib")
LIB = os.path.join(LIB_DIR, "libcula_kda.so")
OBJ_DIR = os.path.join(PKG, "build")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr",
]


def sources():
    return sorted(glob.glob(os.path.join(CSRC, "*.cu")))


def _deps_mtime():
    files = glob.glob(os.path.join(CSRC, "*")) + glob.glob(os.path.join(PKG, "..", "include", "*.h"))
    return max(os.path.getmtime(f) for f in files)


TIMERS_LIB = os.path.join(LIB_DIR, "libcula_kda_timers.so")


def build(force=False, verbose=False, timers=False):
    """Build the library. ``timers=True`` builds a second library, libcula_kda_timers.so, with -DKDA_PHASE_TIMERS:
    the chunk-parallel forward kernel and the gated backward kernel then count clock64() cycles per phase (see
    cula_b200/phase_timers.py); it is a profiling aid and is never loaded by the package itself."""
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    os.makedirs(LIB_DIR, exist_ok=True)
    obj_dir = OBJ_DIR + ("_timers" if timers else "")
    lib = TIMERS_LIB if timers else LIB
    os.makedirs(obj_dir, exist_ok=True)
    if not force and os.path.exists(lib) and os.path.getmtime(lib) >= _deps_mtime():
        return lib
    extra = (["-Xptxas", "-v"] if verbose else []) + (["-DKDA_PHASE_TIMERS"] if timers else [])
    procs, objs = [], []
    for src in sources():
        obj = os.path.join(obj_dir, os.path.basename(src)[:-3] + ".o")
        objs.append(obj)
        procs.append((src, subprocess.Popen([nvcc, *NVCC_FLAGS, *extra, "-c", src, "-o", obj],
                                            stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    failed = False
    for src, pr in procs:
        out, _ = pr.communicate()
        if pr.returncode != 0 or verbose:
            sys.stderr.write(f"--- {os.path.basename(src)} ---\n{out}\n")
        failed |= pr.returncode != 0
    if failed:
        raise RuntimeError("nvcc failed")
    subprocess.run([nvcc, "-shared", "-o", lib, *objs, "-lcudart"], check=True)
    return lib


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv, timers="--timers" in sys.argv))
