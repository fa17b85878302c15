"""Builds libm40llm_native.so (sm_100a) in-tree from csrc/*.cu with nvcc.

Usage: python build.py [--force] [--verbose]
The shared library lands next to this file so that it travels with the source tree.
"""
from __future__ import annotations

import concurrent.futures as cf
import glob
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "build")
LIB = os.path.join(HERE, "libm40llm_native.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
]


def _newer(src: str, dst: str, deps: list[str]) -> bool:
    if not os.path.exists(dst):
        return True
    t = os.path.getmtime(dst)
    return any(os.path.getmtime(p) > t for p in [src] + deps)


def build(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(OBJ, exist_ok=True)
    sources = sorted(glob.glob(os.path.join(CSRC, "*.cu")))
    headers = sorted(glob.glob(os.path.join(CSRC, "*.cuh"))) + [os.path.join(HERE, "..", "include", "m40llm_native.h")]
    jobs = []
    for src in sources:
        obj = os.path.join(OBJ, os.path.basename(src)[:-3] + ".o")
        if force or _newer(src, obj, headers):
            cmd = ["nvcc", *NVCC_FLAGS, "-c", src, "-o", obj]
            if verbose:
                cmd.insert(1, "-Xptxas=-v")
            jobs.append(cmd)

    def run(cmd):
        r = subprocess.run(cmd, capture_output=True, text=True)
        return cmd, r

    with cf.ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as ex:
        for cmd, r in ex.map(run, jobs):
            if verbose or r.returncode != 0:
                sys.stderr.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
            if r.returncode != 0:
                raise RuntimeError("nvcc failed: " + " ".join(cmd))
    objs = [os.path.join(OBJ, os.path.basename(s)[:-3] + ".o") for s in sources]
    if force or jobs or not os.path.exists(LIB):
        # -lcuda: the tensor-map encoder of the TMA kernels is a driver entry point fetched at run time
        cmd = ["nvcc", "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", LIB, *objs, "-lcudart"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            sys.stderr.write(r.stdout + r.stderr)
            raise RuntimeError("link failed")
    build_host(force or bool(jobs))
    return LIB


HOST_LIB = os.path.join(HERE, "libm40llm_host.so")


def build_host(force: bool = False) -> str:
    """The C++ host mirror (decode layer driver, batch plan, KV compression config); calls the C ABI only."""
    srcs = sorted(glob.glob(os.path.join(HERE, "host", "*.cpp")))
    deps = sorted(glob.glob(os.path.join(HERE, "host", "*.hpp"))) + [os.path.join(HERE, "..", "include", "m40llm_native.h")]
    if force or not os.path.exists(HOST_LIB) or any(os.path.getmtime(p) > os.path.getmtime(HOST_LIB) for p in srcs + deps):
        cxx = "/usr/bin/g++" if os.path.exists("/usr/bin/g++") else "g++"
        cmd = [cxx, "-O2", "-std=c++17", "-fPIC", "-shared", "-o", HOST_LIB, *srcs, "-L" + HERE, "-lm40llm_native",
               "-Wl,-rpath,$ORIGIN"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            sys.stderr.write(r.stdout + r.stderr)
            raise RuntimeError("host library build failed")
    return HOST_LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
