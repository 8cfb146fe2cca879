"""Builds libhiscache_b200.so in-tree with nvcc for sm_100a.

    python history-cache_b200/build_ext.py [--force] [--verbose]

The library has no torch or Python dependency: it is compiled from csrc/*.cu
against include/hiscache_b200.h only and loaded with ctypes.
"""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
INCLUDE = os.path.join(ROOT, "include")
LIB_DIR = os.path.join(HERE, "lib")
OBJ_DIR = os.path.join(LIB_DIR, "obj")
LIB_PATH = os.path.join(LIB_DIR, "libhiscache_b200.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "-I", INCLUDE,
]


def _sources():
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cu"))


def _deps():
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cuh")]
    deps += [os.path.join(INCLUDE, f) for f in os.listdir(INCLUDE) if f.endswith(".h")]
    return deps


def _stale(target, inputs):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(i) > t for i in inputs)


CHECKED_LIB_PATH = os.path.join(LIB_DIR, "libhiscache_b200_checked.so")


def build(force: bool = False, verbose: bool = False) -> str:
    """Compiles every kernel source and links the shared library; returns its path.  Also builds
    libhiscache_b200_checked.so: the same sources with -DHC_CHECK_BOUNDS (index checks in front
    of the aggregation operators, see hc_last_status in the header)."""
    path = _build_one(force, verbose, OBJ_DIR, LIB_PATH, [])
    _build_one(force, False, os.path.join(LIB_DIR, "obj_checked"), CHECKED_LIB_PATH, ["-DHC_CHECK_BOUNDS"])
    return path


def _build_one(force, verbose, obj_dir, lib_path, extra):
    nvcc = os.environ.get("NVCC", "nvcc")
    os.makedirs(obj_dir, exist_ok=True)
    deps = _deps()
    jobs = []
    objs = []
    for src in _sources():
        obj = os.path.join(obj_dir, os.path.basename(src)[:-3] + ".o")
        objs.append(obj)
        if force or _stale(obj, [src] + deps):
            cmd = ([nvcc] + NVCC_FLAGS + extra + (["-Xptxas", "-v"] if verbose else []) +
                   ["-c", src, "-o", obj])
            jobs.append(cmd)

    def run(cmd):
        p = subprocess.run(cmd, capture_output=True, text=True)
        return cmd, p

    with ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as ex:
        for cmd, p in ex.map(run, jobs):
            if verbose or p.returncode != 0:
                sys.stderr.write(" ".join(cmd) + "\n" + p.stdout + p.stderr)
            if p.returncode != 0:
                raise RuntimeError("nvcc failed for " + cmd[-3])
    if force or jobs or _stale(lib_path, objs):
        cmd = [nvcc, "-shared", "-o", lib_path] + objs
        p = subprocess.run(cmd, capture_output=True, text=True)
        if p.returncode != 0:
            sys.stderr.write(p.stdout + p.stderr)
            raise RuntimeError("link failed")
    return lib_path


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
