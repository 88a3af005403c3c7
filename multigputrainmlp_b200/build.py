"""Builds the native library (and the trainer binary) for sm_100a with nvcc, in-tree.

    python -m multigputrainmlp_b200.build            # libmgt_b200.so (+ bin/mgt_native_train when its sources exist)

nvcc cross-compiles without a GPU. The outputs are git-ignored build products.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
OUT_DIR = os.path.join(PKG, "_native")
LIB = os.path.join(OUT_DIR, "libmgt_b200.so")
TRAIN_BIN = os.path.join(ROOT, "bin", "mgt_native_train")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC,-fvisibility=hidden", "--expt-relaxed-constexpr",
]
CUDA_SOURCES = ["walk.cu", "adamw.cu", "engine.cu", "comm.cu"]
HOST_SOURCES = ["plan.cpp", "artifacts.cpp", "host_capi.cpp"]


def _nvcc() -> str:
    path = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(path):
        raise RuntimeError("nvcc not found: the native library cannot be built")
    return path


def _stale(target: str, sources: list[str]) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    deps = list(sources)
    for name in os.listdir(CSRC):
        if name.endswith((".cuh", ".hpp", ".h")):
            deps.append(os.path.join(CSRC, name))
    deps.append(os.path.join(ROOT, "include", "mgt_b200.h"))
    return any(os.path.getmtime(d) > t for d in deps if os.path.exists(d))


def build(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(OUT_DIR, exist_ok=True)
    nvcc = _nvcc()
    objs = []
    sources = [os.path.join(CSRC, s) for s in CUDA_SOURCES + HOST_SOURCES if os.path.exists(os.path.join(CSRC, s))]
    for src in sources:
        obj = os.path.join(OUT_DIR, os.path.basename(src) + ".o")
        objs.append(obj)
        if force or _stale(obj, [src]):
            cmd = [nvcc, *NVCC_FLAGS, "-DMGT_BUILDING_LIBRARY", "-c", src, "-o", obj]
            if verbose:
                cmd.insert(1, "-Xptxas=-v")
            subprocess.run(cmd, check=True)
    if force or _stale(LIB, objs) or any(os.path.getmtime(o) > os.path.getmtime(LIB) for o in objs):
        subprocess.run([nvcc, "-shared", "-o", LIB, *objs, "-gencode", "arch=compute_100a,code=sm_100a"], check=True)
    train_src = os.path.join(CSRC, "train_main.cpp")
    if os.path.exists(train_src):
        os.makedirs(os.path.dirname(TRAIN_BIN), exist_ok=True)
        host = [train_src, os.path.join(CSRC, "plan.cpp"), os.path.join(CSRC, "artifacts.cpp")]
        if force or _stale(TRAIN_BIN, host + [LIB]):
            subprocess.run([nvcc, "-O2", "-std=c++17", "-o", TRAIN_BIN, *host, "-L", OUT_DIR, "-lmgt_b200",
                            "-Xlinker", "-rpath=$ORIGIN/../multigputrainmlp_b200/_native"], check=True)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
