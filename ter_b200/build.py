"""Builds ter_b200/libter_b200.so in-tree with nvcc for sm_100a.

Usage: ``python -m ter_b200.build [--force] [--verbose]``.  nvcc cross-compiles
without a GPU, so this runs anywhere the CUDA toolkit is installed.
"""
from __future__ import annotations

import glob
import os
import shutil
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG, "csrc")
ROOT = os.path.dirname(PKG)
LIB = os.path.join(PKG, "libter_b200.so")
CLI = os.path.join(PKG, "ter_b200_generate")      # command-line front end (csrc/cli/generate_main.cpp)
OBJ_DIR = os.path.join(PKG, "build")

ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
# -fmad=false: no implicit fused multiply-add; every fused operation in the glue kernels is
# an explicit fmaf(), so results are reproducible against the CPU checker bit for bit.
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-fmad=false", "-Xcompiler", "-fPIC",
              "-Xcompiler", "-fno-exceptions", "-Xcompiler", "-fno-rtti", "-Xcompiler", "-Wall"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found: the CUDA toolkit is required to build ter_b200")


def _nccl_flags():
    """Include / link flags for NCCL (headers from the system or the pip wheel)."""
    inc, libdir = None, None
    for d in ("/usr/include",):
        if os.path.exists(os.path.join(d, "nccl.h")):
            inc = d
    try:
        import nvidia.nccl as _n  # type: ignore
        base = os.path.dirname(_n.__file__) if getattr(_n, "__file__", None) else list(_n.__path__)[0]
        if os.path.exists(os.path.join(base, "include", "nccl.h")):
            inc = os.path.join(base, "include")
            libdir = os.path.join(base, "lib")
    except Exception:
        pass
    return inc, libdir


def sources():
    return sorted(glob.glob(os.path.join(CSRC, "*.cu")) + glob.glob(os.path.join(CSRC, "*.cpp")))


def needs_build() -> bool:
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    if not os.path.exists(CLI):
        return True
    deps = sources() + glob.glob(os.path.join(CSRC, "*.h")) + glob.glob(os.path.join(CSRC, "*.cuh")) + \
        glob.glob(os.path.join(CSRC, "cli", "*.cpp")) + \
        [os.path.join(ROOT, "include", "ter_b200.h"), os.path.abspath(__file__)]
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and not needs_build():
        return LIB
    nvcc = _nvcc()
    os.makedirs(OBJ_DIR, exist_ok=True)
    inc, _ = _nccl_flags()
    extra_inc = ["-I", os.path.join(ROOT, "include")] + (["-I", inc] if inc else [])
    objs = []
    procs = []
    for src in sources():
        obj = os.path.join(OBJ_DIR, os.path.basename(src) + ".o")
        objs.append(obj)
        # TER_B200_NVCC_EXTRA: extra compiler flags (diagnostic builds)
        cmd = [nvcc, "-c", src, "-o", obj] + ARCH + NVCC_FLAGS + extra_inc + os.environ.get("TER_B200_NVCC_EXTRA", "").split()
        if verbose:
            cmd += ["-Xptxas", "-v"]
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    failed = False
    for src, p in procs:
        out, _ = p.communicate()
        if p.returncode != 0:
            failed = True
            sys.stderr.write(f"--- nvcc failed on {src}\n{out}\n")
        elif verbose or out.strip():
            sys.stderr.write(f"--- {os.path.basename(src)}\n{out}\n")
    if failed:
        raise RuntimeError("ter_b200 build failed")
    # NCCL is resolved at run time from the process (torch loads it) or the system library.
    link = [nvcc, "-shared", "-o", LIB] + objs + ARCH + ["-Xcompiler", "-fPIC", "-lcudart_static", "-ldl", "-lpthread"]
    subprocess.run(link, check=True)
    # the command-line front end: plain C++ over the C ABI, finds the library next to itself
    subprocess.run([os.environ.get("CXX", "g++"), "-O2", "-std=c++17", "-I", os.path.join(ROOT, "include"),
                    os.path.join(CSRC, "cli", "generate_main.cpp"), "-o", CLI, "-L", PKG, "-lter_b200",
                    "-Wl,-rpath,$ORIGIN"], check=True)
    return LIB


if __name__ == "__main__":
    build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(LIB)
