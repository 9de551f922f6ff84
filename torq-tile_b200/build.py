"""Build recipe of libtorq_tile_b200.so: nvcc for the CUDA translation units, g++ for the C ABI.

Everything is compiled for sm_100a only and linked into one shared library that sits beside this
file (built artefacts are not committed).  Usage: ``python torq-tile_b200/build.py [--force]``.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OUT = os.path.join(HERE, "libtorq_tile_b200.so")
OBJ = os.path.join(HERE, "build")

CU_SOURCES = ["kernels_pack.cu", "kernels_simt.cu", "kernels_umma.cu", "kernels_pair.cu", "kernels_gemv.cu", "kernels_conv.cu", "kernels_float.cu", "static_scratch.cu"]
CXX_SOURCES = ["abi.cpp", "dispatch.cpp"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "--threads", "4"]
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-Wall", "-Wextra", "-fvisibility=default"]


def _nvcc() -> str:
    for cand in (shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found: the CUDA toolkit is required to build libtorq_tile_b200.so")


def _gxx() -> str:
    for cand in ("/usr/bin/g++", shutil.which("g++")):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("g++ not found")


def _stale(target: str, deps) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False, diag: bool = False) -> str:
    """diag: compile the kernels' role timing, traces and GEMV phase stamps in (-DTQT_B200_DIAG; always a full rebuild,
    and the next ordinary build has to be forced too).  They are left out of ordinary builds because the hot loops are
    sensitive to code size."""
    os.makedirs(OBJ, exist_ok=True)
    force = force or diag
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".h", ".cuh", ".inc"))]
    headers += [os.path.join(HERE, "..", "include", f) for f in os.listdir(os.path.join(HERE, "..", "include"))]
    nvcc, gxx = _nvcc(), _gxx()
    objs = []
    procs = []
    for src in CU_SOURCES + CXX_SOURCES:
        path = os.path.join(CSRC, src)
        obj = os.path.join(OBJ, src + ".o")
        objs.append(obj)
        if force or _stale(obj, [path] + headers):
            if src.endswith(".cu"):
                cmd = [nvcc] + NVCC_FLAGS + (["-DTQT_B200_DIAG"] if diag else []) + ["-c", path, "-o", obj]
            else:
                cmd = [gxx] + CXX_FLAGS + ["-c", path, "-o", obj]
            if verbose:
                print(" ".join(cmd))
            procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    for src, p in procs:
        out, _ = p.communicate()
        if p.returncode != 0:
            raise RuntimeError(f"compiling {src} failed:\n{out}")
        if verbose and out.strip():
            print(out)
    if force or procs or not os.path.exists(OUT):
        cmd = [nvcc, "-shared", "-o", OUT] + objs + ["-gencode", "arch=compute_100a,code=sm_100a", "-cudart", "static",
                                                     "-Xcompiler", "-fPIC"]
        if verbose:
            print(" ".join(cmd))
        subprocess.check_call(cmd)
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose=True, diag="--diag" in sys.argv))
