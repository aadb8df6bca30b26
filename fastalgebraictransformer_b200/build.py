"""Build libfat_b200.so (the C-ABI library, nvcc for sm_100a) and libfat_torch_ops.so (the torch.library operators, g++) in-tree.

    python -m fastalgebraictransformer_b200.build [--force] [--verbose]

Every .cu under csrc/ is compiled to an object in csrc/_obj/ (in parallel) and linked into
fastalgebraictransformer_b200/libfat_b200.so.  nvcc cross-compiles, so no GPU is needed.
"""
from __future__ import annotations

import argparse
import concurrent.futures as cf
import glob
import os
import shutil
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG, "csrc")
OBJ = os.path.join(CSRC, "_obj")
LIB = os.path.join(PKG, "libfat_b200.so")
OPS_SRC = os.path.join(CSRC, "torch_ops.cpp")
OPS_LIB = os.path.join(PKG, "libfat_torch_ops.so")

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found: set NVCC or put the CUDA toolkit on PATH")


def _stale(target: str, deps) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile and link the library if any source is newer than it.  Returns the .so path."""
    sources = sorted(glob.glob(os.path.join(CSRC, "*.cu")))
    headers = sorted(glob.glob(os.path.join(CSRC, "*.cuh"))) + \
        sorted(glob.glob(os.path.join(PKG, "..", "include", "*.h")))
    if not sources:
        raise RuntimeError(f"no CUDA sources under {CSRC}")
    os.makedirs(OBJ, exist_ok=True)
    nvcc = _nvcc()
    jobs = []
    for src in sources:
        obj = os.path.join(OBJ, os.path.basename(src)[:-3] + ".o")
        if force or _stale(obj, [src] + headers):
            jobs.append((src, obj))

    def compile_one(job):
        src, obj = job
        cmd = [nvcc, *NVCC_FLAGS, "-Xptxas", "-v", "-c", src, "-o", obj]
        r = subprocess.run(cmd, capture_output=True, text=True)
        return src, r

    if jobs:
        with cf.ThreadPoolExecutor(max_workers=min(len(jobs), os.cpu_count() or 4)) as ex:
            for src, r in ex.map(compile_one, jobs):
                if verbose or r.returncode:
                    sys.stderr.write(r.stdout + r.stderr)
                if r.returncode:
                    raise RuntimeError(f"nvcc failed on {src}")
    objs = [os.path.join(OBJ, os.path.basename(s)[:-3] + ".o") for s in sources]
    if force or jobs or _stale(LIB, objs):
        cmd = [nvcc, "-shared", "-o", LIB, *objs, "-gencode", "arch=compute_100a,code=sm_100a"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode:
            sys.stderr.write(r.stdout + r.stderr)
            raise RuntimeError("link of libfat_b200.so failed")
    build_ops(force or bool(jobs), verbose)
    build_wait_test(force, verbose)
    return LIB


WAIT_TEST_LIB = os.path.join(PKG, "..", "tests", "_build", "libfat_b200_waittest.so")
WAIT_TEST_FLAGS = ["-DFAT_TEST_WITHHOLD_V_TILE=0", "-DFAT_TEST_CE_WITHHOLD_ROW=4", "-DFAT_WAIT_HINT_NS=100000", "-DFAT_WAIT_SPINS=30"]
WAIT_TEST_SOURCES = ("attn_tc_fwd.cu", "loss.cu")


def build_wait_test(force: bool = False, verbose: bool = False) -> str:
    """A TEST-ONLY variant of the library (tests/_build/, never loaded by the package): the attention forward is compiled
    so that its producer leaves out one V tile, the staged loss kernel so that its first block never requests the copy of
    one row, and every bounded wait gives up after ~3 ms.  tests/test_wait_timeout.py uses it to run the give-up paths
    once (status word or NaN losses, teardown, TMEM release).  Only those two sources are recompiled; the other objects
    are the shipped ones."""
    srcs = [os.path.join(CSRC, n) for n in WAIT_TEST_SOURCES]
    headers = sorted(glob.glob(os.path.join(CSRC, "*.cuh"))) + sorted(glob.glob(os.path.join(PKG, "..", "include", "*.h")))
    out_dir = os.path.dirname(WAIT_TEST_LIB)
    os.makedirs(out_dir, exist_ok=True)
    objs = [os.path.join(out_dir, n[:-3] + "_waittest.o") for n in WAIT_TEST_SOURCES]
    others = [os.path.join(OBJ, os.path.basename(s)[:-3] + ".o") for s in sorted(glob.glob(os.path.join(CSRC, "*.cu")))
              if os.path.basename(s) not in WAIT_TEST_SOURCES]
    if not (force or _stale(WAIT_TEST_LIB, srcs + headers + others)):
        return WAIT_TEST_LIB
    nvcc = _nvcc()
    cmds = [[nvcc, *NVCC_FLAGS, *WAIT_TEST_FLAGS, "-c", src, "-o", obj] for src, obj in zip(srcs, objs)]
    cmds.append([nvcc, "-shared", "-o", WAIT_TEST_LIB, *objs, *others, "-gencode", "arch=compute_100a,code=sm_100a"])
    for cmd in cmds:
        r = subprocess.run(cmd, capture_output=True, text=True)
        if verbose or r.returncode:
            sys.stderr.write(r.stdout + r.stderr)
        if r.returncode:
            raise RuntimeError("build of the wait-timeout test library failed")
    return WAIT_TEST_LIB


def build_ops(force: bool = False, verbose: bool = False) -> str:
    """Compile csrc/torch_ops.cpp (the C++ registration of the torch.library operators) against the installed torch
    and link it to libfat_b200.so.  Host code only: g++, no nvcc."""
    header = os.path.join(PKG, "..", "include", "fat_b200.h")
    if not (force or _stale(OPS_LIB, [OPS_SRC, header, LIB])):
        return OPS_LIB
    import torch
    from torch.utils import cpp_extension as ce
    cuda_home = os.environ.get("CUDA_HOME") or os.path.dirname(os.path.dirname(_nvcc()))
    cxx = os.environ.get("CXX") or shutil.which("g++") or "g++"
    cmd = [cxx, "-O2", "-std=c++17", "-fPIC", "-shared", OPS_SRC, "-o", OPS_LIB,
           f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}", "-I" + os.path.join(cuda_home, "include")]
    cmd += ["-I" + p for p in ce.include_paths()]
    cmd += ["-L" + p for p in ce.library_paths()]
    cmd += ["-ltorch", "-ltorch_cpu", "-ltorch_cuda", "-lc10", "-lc10_cuda", "-L" + PKG, "-lfat_b200", "-Wl,-rpath,$ORIGIN"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or r.returncode:
        sys.stderr.write(r.stdout + r.stderr)
    if r.returncode:
        raise RuntimeError("build of libfat_torch_ops.so failed")
    return OPS_LIB


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    a = ap.parse_args()
    print(build(a.force, a.verbose))
