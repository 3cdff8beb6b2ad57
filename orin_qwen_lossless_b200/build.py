"""Builds libbf16n_b200.so (host encoder + policy + sm_100a kernels + C ABI) in-tree with nvcc.

    python -m orin_qwen_lossless_b200.build [--force]

nvcc cross-compiles for sm_100a without a GPU; the .so lands beside this file so it travels with the source tree.
"""
from __future__ import annotations

import concurrent.futures as cf
import os
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(PKG, "csrc")
OBJ = os.path.join(PKG, "build")
LIB = os.path.join(PKG, "libbf16n_b200.so")
INC = os.path.join(os.path.dirname(PKG), "include")

CUDA_SOURCES = ["gemv.cu", "gemv_staged.cu", "gemv_rings.cu", "moe.cu", "moe_decode.cu", "prefill.cu", "expand_tiles.cu", "peer.cu", "fo.cu", "draft.cu", "adapter.cu", "ep_prefill.cu", "capi.cu"]
HOST_SOURCES = ["encode.cpp", "policy.cpp"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC,-pthread",
              "-I", INC]
CXX_FLAGS = ["-O3", "-std=c++17", "-fPIC", "-pthread", "-Wall", "-Wextra", "-I", INC]


def _deps() -> list[str]:
    out = [os.path.join(SRC, f) for f in os.listdir(SRC)]
    out += [os.path.join(INC, f) for f in os.listdir(INC) if f.endswith(".h")]
    return out


def _stale(target: str, sources: list[str]) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in sources)


def _run(cmd: list[str]) -> None:
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("build failed: " + " ".join(cmd) + "\n" + r.stdout + r.stderr)


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile what is out of date and link; returns the library path."""
    os.makedirs(OBJ, exist_ok=True)
    deps = _deps()
    jobs = []
    for s in CUDA_SOURCES:
        o = os.path.join(OBJ, s + ".o")
        if force or _stale(o, deps):
            jobs.append(["nvcc", *NVCC_FLAGS, "-c", os.path.join(SRC, s), "-o", o])
    for s in HOST_SOURCES:
        o = os.path.join(OBJ, s + ".o")
        if force or _stale(o, deps):
            jobs.append(["g++", *CXX_FLAGS, "-c", os.path.join(SRC, s), "-o", o])
    if verbose and jobs:
        print(f"compiling {len(jobs)} translation units", file=sys.stderr)
    with cf.ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as ex:
        list(ex.map(_run, jobs))
    objs = [os.path.join(OBJ, s + ".o") for s in CUDA_SOURCES + HOST_SOURCES]
    if force or jobs or _stale(LIB, objs):
        _run(["nvcc", "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", LIB, *objs, "-lpthread"])
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose=True))
