"""Builds the C-ABI CUDA library in-tree for sm_100a with nvcc, in two variants:

    libet_b200.so        the product: the entry points include/et_b200.h declares
    libet_b200_hooks.so  the same sources with -DET_TEST_HOOKS: also exports the et_debug_*
                         test hooks (forced kernel plans, instruction-rate probes)

Usage: python scpaper-2021_b200/build.py [--force] [--verbose]
No GPU is needed: nvcc cross-compiles.  Objects go to build/ (git-ignored), the shared
libraries next to this file so that they travel with the source tree.
"""
from __future__ import annotations

import concurrent.futures
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
OBJ_DIR = os.path.join(ROOT, "build", "et_b200")
LIB_PATH = os.path.join(HERE, "libet_b200.so")
HOOKS_LIB_PATH = os.path.join(HERE, "libet_b200_hooks.so")

NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
HOST_CXX = "/usr/bin/g++"
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-ccbin", HOST_CXX,
    "-Xcompiler", "-fPIC",
]


def sources() -> list[str]:
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cu"))


def headers() -> list[str]:
    hs = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    hs.append(os.path.join(ROOT, "include", "et_b200.h"))
    return hs


def _stale(target: str, deps: list[str]) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def _has_hooks(src: str) -> bool:
    with open(src) as f:
        return "ET_TEST_HOOKS" in f.read()


def _compile(src: str, verbose: bool, hooks: bool = False) -> str:
    obj = os.path.join(OBJ_DIR, os.path.basename(src)[:-3] + (".hooks.o" if hooks else ".o"))
    if _stale(obj, [src] + headers()):
        cmd = [NVCC] + NVCC_FLAGS + (["-DET_TEST_HOOKS"] if hooks else []) + \
            (["-Xptxas", "-v"] if verbose else []) + ["-c", src, "-o", obj]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if verbose or r.returncode != 0:
            sys.stderr.write(r.stdout + r.stderr)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src}")
    return obj


def build(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(OBJ_DIR, exist_ok=True)
    srcs = sources()
    if force:
        for f in os.listdir(OBJ_DIR):
            if f.endswith(".o"):
                os.remove(os.path.join(OBJ_DIR, f))
    # a source that mentions ET_TEST_HOOKS is compiled twice; the hooks library takes the
    # plain object of every other source
    jobs = [(s, False) for s in srcs] + [(s, True) for s in srcs if _has_hooks(s)]
    with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
        built = list(ex.map(lambda j: _compile(j[0], verbose, j[1]), jobs))
    objs = built[:len(srcs)]
    hooked = {j[0]: o for j, o in zip(jobs[len(srcs):], built[len(srcs):])}
    hook_objs = [hooked.get(s, o) for s, o in zip(srcs, objs)]
    for path, members in ((LIB_PATH, objs), (HOOKS_LIB_PATH, hook_objs)):
        if force or _stale(path, members):
            cmd = [NVCC, "-shared", "-ccbin", HOST_CXX, "-gencode",
                   "arch=compute_100a,code=sm_100a", "-o", path] + members
            r = subprocess.run(cmd, capture_output=True, text=True)
            if r.returncode != 0:
                sys.stderr.write(r.stdout + r.stderr)
                raise RuntimeError("link failed")
    return LIB_PATH


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
