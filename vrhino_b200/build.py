"""Build the CUDA operator library (``libvrb.so``) in-tree with nvcc for sm_100a, and the
multi-GPU host layer (``libvrb_sharded.so``: C++ over NCCL and libvrb.so) with the host compiler.

``python -m vrhino_b200.build`` compiles every ``csrc/*.cu`` to an object file (in parallel)
and links them into ``vrhino_b200/libvrb.so``.  nvcc cross-compiles, so no GPU is needed.
The register / shared-memory report of ``-Xptxas -v`` is kept in ``csrc/build/ptxas.log``.
"""
from __future__ import annotations

import concurrent.futures
import glob
import os
import shutil
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
OBJ = os.path.join(CSRC, "build")
LIB = os.path.join(PKG, "libvrb.so")
SHARDED_SRC = os.path.join(PKG, "host", "sharded_ops.cpp")
SHARDED_LIB = os.path.join(PKG, "libvrb_sharded.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xptxas", "-v", "-I", os.path.join(ROOT, "include"), "-I", CSRC,
]


def _nvcc() -> str:
    found = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(found):
        raise RuntimeError("nvcc not found; the CUDA toolkit is required to build libvrb.so")
    return found


def _sources():
    return sorted(glob.glob(os.path.join(CSRC, "*.cu")))


def _stale(target: str, deps) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(OBJ, exist_ok=True)
    headers = glob.glob(os.path.join(CSRC, "*.cuh")) + glob.glob(os.path.join(ROOT, "include", "*.h"))
    nvcc = _nvcc()
    jobs = []
    for src in _sources():
        obj = os.path.join(OBJ, os.path.basename(src)[:-3] + ".o")
        if force or _stale(obj, [src] + headers):
            jobs.append((src, obj))

    def compile_one(job):
        src, obj = job
        proc = subprocess.run([nvcc, *NVCC_FLAGS, "-c", src, "-o", obj], capture_output=True, text=True)
        return src, proc

    logs = []
    with concurrent.futures.ThreadPoolExecutor(max_workers=max(1, min(8, len(jobs) or 1))) as pool:
        for src, proc in pool.map(compile_one, jobs):
            logs.append(f"==== {os.path.basename(src)}\n{proc.stderr}")
            if proc.returncode != 0:
                sys.stderr.write(proc.stdout + proc.stderr)
                raise RuntimeError(f"nvcc failed on {src}")
            if verbose:
                sys.stderr.write(proc.stderr)
    if logs:
        with open(os.path.join(OBJ, "ptxas.log"), "a") as fh:
            fh.write("\n".join(logs))
    objects = [os.path.join(OBJ, os.path.basename(s)[:-3] + ".o") for s in _sources()]
    if force or jobs or _stale(LIB, objects):
        subprocess.run([nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-shared", "-o", LIB, *objects, "-lcudart"], check=True)
    build_sharded(force)
    return LIB


def build_sharded(force: bool = False) -> str:
    """libvrb_sharded.so: needs nccl.h / libnccl (the system's) next to the CUDA toolkit."""
    headers = glob.glob(os.path.join(ROOT, "include", "*.h"))
    if not (force or _stale(SHARDED_LIB, [SHARDED_SRC, LIB] + headers)):
        return SHARDED_LIB
    cuda_home = os.path.dirname(os.path.dirname(_nvcc()))
    cxx = shutil.which("g++") or "g++"
    subprocess.run([cxx, "-std=c++17", "-O2", "-fPIC", "-shared", "-Wall", "-I", os.path.join(ROOT, "include"),
                    "-I", os.path.join(cuda_home, "include"), "-o", SHARDED_LIB, SHARDED_SRC,
                    "-L", PKG, "-lvrb", "-Wl,-rpath,$ORIGIN", "-L", os.path.join(cuda_home, "lib64"), "-lcudart", "-lnccl",
                    "-lpthread"], check=True)
    return SHARDED_LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
