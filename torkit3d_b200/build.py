"""Compile libtk3d_b200.so in-tree with nvcc for sm_100a.

    python -m torkit3d_b200.build [--force] [--verbose] [--bounds]

``--bounds`` builds libtk3d_b200_bounds.so instead: the same sources with -DTK3D_BOUNDS, in which every
coordinate load and index-tensor access is range checked and violations are counted
(tk3d_bounds_violations()).  The tests run a set of shapes through it; it is not what the operators load.

The library has no dependency on torch or Python headers (plain CUDA runtime), so a full rebuild
takes seconds.  Objects are cached under ``torkit3d_b200/csrc/build/`` by source mtime.
"""
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

PKG = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG, "csrc")
INCLUDE = os.path.join(os.path.dirname(PKG), "include")
LIB = os.path.join(PKG, "libtk3d_b200.so")
LIB_BOUNDS = os.path.join(PKG, "libtk3d_b200_bounds.so")  # the range-checked build (-DTK3D_BOUNDS), for tests

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-I" + INCLUDE, "-I" + CSRC,
]


def sources():
    return sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))


def _headers_mtime():
    hs = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    hs.append(os.path.join(INCLUDE, "tk3d.h"))
    return max(os.path.getmtime(h) for h in hs)


def build(force=False, verbose=False, extra_flags=(), bounds=False):
    """Compile the library; ``bounds=True`` builds the range-checked variant next to it."""
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    odir = os.path.join(CSRC, "build", "bounds") if bounds else os.path.join(CSRC, "build")
    lib = LIB_BOUNDS if bounds else LIB
    if bounds:
        extra_flags = tuple(extra_flags) + ("-DTK3D_BOUNDS",)
    os.makedirs(odir, exist_ok=True)
    hm = _headers_mtime()
    jobs = []
    objs = []
    for s in sources():
        src = os.path.join(CSRC, s)
        obj = os.path.join(odir, s[:-3] + ".o")
        objs.append(obj)
        if force or not os.path.exists(obj) or os.path.getmtime(obj) < max(os.path.getmtime(src), hm):
            jobs.append([nvcc, "-c", src, "-o", obj] + NVCC_FLAGS + list(extra_flags)
                        + os.environ.get("TK3D_NVCC_FLAGS", "").split())

    def run(cmd):
        p = subprocess.run(cmd, capture_output=True, text=True)
        if verbose or p.returncode != 0:
            sys.stderr.write(" ".join(cmd) + "\n" + p.stdout + p.stderr)
        return p.returncode

    if jobs:
        with ThreadPoolExecutor(min(8, len(jobs))) as ex:
            rcs = list(ex.map(run, jobs))
        if any(rcs):
            raise RuntimeError("nvcc failed for libtk3d_b200 (see stderr)")
    if jobs or force or not os.path.exists(lib):
        cmd = [nvcc, "-shared", "-o", lib] + objs + ["-gencode", "arch=compute_100a,code=sm_100a", "-lcudart"]
        p = subprocess.run(cmd, capture_output=True, text=True)
        if p.returncode != 0:
            sys.stderr.write(p.stdout + p.stderr)
            raise RuntimeError("link of %s failed" % os.path.basename(lib))
    return lib


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv,
                extra_flags=("-Xptxas", "-v") if "--ptxas" in sys.argv else (), bounds="--bounds" in sys.argv))
