"""Compile the CUDA sources into tensormark_b200/libtm_cuda.so for sm_100a.

`python -m tensormark_b200.build` (or build()) runs nvcc on every .cu under csrc/
and links one shared library that exports the C ABI declared in include/cuda_shim.h.
The library is kept in-tree next to this file; nothing is installed.
"""
from __future__ import annotations

import concurrent.futures as cf
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
INCLUDE = os.path.join(os.path.dirname(HERE), "include")
OBJ = os.path.join(HERE, "build")
LIB = os.path.join(HERE, "libtm_cuda.so")
CHAIN_LIB = os.path.join(HERE, "libtm_chain.so")

NVCC_FLAGS = [
    "-std=c++20", "-O3", "-lineinfo",
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-Xcompiler", "-fPIC",
    "-I" + INCLUDE, "-I" + CSRC,
    "-DTM_CUDA_BUILD",
]


def _nccl_include() -> list[str]:
    """Header of the NCCL that torch loads (the library itself is resolved at run time)."""
    try:
        import nvidia.nccl  # type: ignore
        inc = os.path.join(os.path.dirname(nvidia.nccl.__file__), "include")
        if os.path.exists(os.path.join(inc, "nccl.h")):
            return ["-I" + inc]
    except Exception:
        pass
    return []


def sources() -> list[str]:
    return sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))


def _stale(target: str, deps: list[str]) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(OBJ, exist_ok=True)
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    headers += [os.path.join(INCLUDE, f) for f in os.listdir(INCLUDE) if f.endswith(".h")]
    flags = NVCC_FLAGS + _nccl_include() + (["-Xptxas", "-v"] if verbose else [])
    jobs = []
    for src in sources():
        obj = os.path.join(OBJ, src[:-3] + ".o")
        if force or _stale(obj, [os.path.join(CSRC, src)] + headers):
            jobs.append((src, ["nvcc"] + flags + ["-c", os.path.join(CSRC, src), "-o", obj]))

    def run(job):
        src, cmd = job
        r = subprocess.run(cmd, capture_output=True, text=True)
        return src, r

    with cf.ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as ex:
        for src, r in ex.map(run, jobs):
            if verbose or r.returncode != 0:
                sys.stderr.write(r.stdout + r.stderr)
            if r.returncode != 0:
                raise RuntimeError(f"nvcc failed on {src}")
    objs = [os.path.join(OBJ, s[:-3] + ".o") for s in sources()]
    if force or jobs or _stale(LIB, objs):
        cmd = ["nvcc", "-shared", "-o", LIB] + objs + ["-ldl"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            sys.stderr.write(r.stdout + r.stderr)
            raise RuntimeError("link failed")
    # the C++ host driver of the decode chain, behind a flat C surface
    chain_src = os.path.join(HERE, "host", "chain_capi.cpp")
    chain_deps = [chain_src, LIB] + [os.path.join(INCLUDE, f) for f in os.listdir(INCLUDE) if f.endswith(".h")]
    if force or _stale(CHAIN_LIB, chain_deps):
        cmd = ["g++", "-std=c++23", "-O2", "-fPIC", "-shared", "-fvisibility=hidden", "-I" + INCLUDE, "-o", CHAIN_LIB,
               chain_src, "-L" + HERE, "-ltm_cuda", "-Wl,-rpath,$ORIGIN"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            sys.stderr.write(r.stdout + r.stderr)
            raise RuntimeError("host driver build failed")
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
