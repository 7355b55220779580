"""Recipe: compile the UNMODIFIED reference CUDA extension for sm_100a into oracle/_ref/.

TEST INFRASTRUCTURE ONLY.  The product never imports anything built here.

The reference (torkit3d v0.1.2) ships one pybind11 module, ``torkit3d._C``, made of
``torkit3d/csrc/torkit3d.cpp`` and the six ``torkit3d/csrc/cuda/*.cu`` files.  They are compiled
where they lie (the path given by ``--ref``), with nvcc directly, against the installed torch
headers -- the reference's own ``setup.py`` is not run and no source file is copied.

Two variants are produced, each a loadable extension module called ``_C``:

  oracle/_ref/nofma/_C.so    nvcc ``-fmad=false``: every multiply/add rounded on its own, i.e. the
                             squared distance is exactly ``(dx*dx + dy*dy) + dz*dz`` as the
                             reference source spells it (``csrc/cuda/chamfer_distance_kernel.cu:65-71``).
                             This is the GPU-side parity checker.
  oracle/_ref/shipped/_C.so  nvcc defaults (what ``setup.py:43-50`` gives a user): timed as
                             "the reference as shipped" next to the new kernels.

Nothing here needs a GPU (nvcc cross-compiles).  Each ``.cu`` takes a few minutes because of the
ATen headers; the files are compiled in parallel.

    python oracle/build_ref.py --ref /path/to/torkit3d-checkout [--jobs 8]
"""
import argparse
import os
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")

CU = [
    "chamfer_distance_kernel.cu",
    "knn_distance_kernel.cu",
    "sample_farthest_points_kernel.cu",
    "ball_query_kernel.cu",
    "group_points_kernel.cu",
    "interpolate_kernel.cu",
]


def _torch_paths():
    import torch  # noqa: F401
    from torch.utils import cpp_extension as ce

    return ce.include_paths(), ce.library_paths()


def build(ref, jobs=8, variants=("nofma", "shipped"), verbose=True):
    csrc = os.path.join(ref, "torkit3d", "csrc")
    if not os.path.isdir(csrc):
        raise FileNotFoundError(csrc)
    inc, libs = _torch_paths()
    pyinc = sysconfig.get_paths()["include"]
    common = ["-DWITH_CUDA", "-DTORCH_EXTENSION_NAME=_C", "-DTORCH_API_INCLUDE_EXTENSION_H",
              "-D_GLIBCXX_USE_CXX11_ABI=1", "-std=c++17", "-O2",
              "-I" + csrc, "-I" + os.path.join(csrc, "include"), "-I" + pyinc]
    for p in inc:
        common += ["-isystem", p]
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    tasks = []
    for var in variants:
        odir = os.path.join(OUT, var, "obj")
        os.makedirs(odir, exist_ok=True)
        extra = ["-fmad=false"] if var == "nofma" else []
        for f in CU:
            obj = os.path.join(odir, f + ".o")
            cmd = [nvcc, "-c", os.path.join(csrc, "cuda", f), "-o", obj,
                   "-gencode", "arch=compute_100a,code=sm_100a", "--expt-relaxed-constexpr",
                   "-Xcompiler", "-fPIC", "-w"] + extra + common
            tasks.append((obj, cmd))
        obj = os.path.join(odir, "torkit3d.cpp.o")
        cmd = ["g++", "-c", os.path.join(csrc, "torkit3d.cpp"), "-o", obj, "-fPIC", "-w",
               "-I/usr/local/cuda/include"] + common
        tasks.append((obj, cmd))

    def run(t):
        obj, cmd = t
        if os.path.exists(obj):
            return obj, 0, ""
        p = subprocess.run(cmd, capture_output=True, text=True)
        if p.returncode != 0 and os.path.exists(obj):
            os.remove(obj)
        if verbose:
            print(("ok   " if p.returncode == 0 else "FAIL ") + obj, flush=True)
        return obj, p.returncode, p.stderr[-2000:]

    with ThreadPoolExecutor(jobs) as ex:
        res = list(ex.map(run, tasks))
    bad = [r for r in res if r[1] != 0]
    if bad:
        raise RuntimeError("reference compile failed:\n" + "\n".join(b[0] + "\n" + b[2] for b in bad))
    for var in variants:
        odir = os.path.join(OUT, var, "obj")
        objs = [os.path.join(odir, f + ".o") for f in CU] + [os.path.join(odir, "torkit3d.cpp.o")]
        so = os.path.join(OUT, var, "_C.so")
        cmd = ["g++", "-shared", "-o", so] + objs + ["-L" + p for p in libs] + \
              ["-Wl,-rpath," + p for p in libs] + \
              ["-L/usr/local/cuda/lib64", "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda",
               "-ltorch", "-ltorch_python", "-lcudart"]
        subprocess.run(cmd, check=True)
        if verbose:
            print("linked", so, flush=True)


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", required=True)
    ap.add_argument("--jobs", type=int, default=8)
    ap.add_argument("--variants", default="nofma,shipped")
    a = ap.parse_args()
    build(a.ref, a.jobs, tuple(a.variants.split(",")))
    sys.exit(0)
