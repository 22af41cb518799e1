"""Builds libmatchattn_b200.so for sm_100a, in-tree, with nvcc alone.

    python -m matchattention_b200.build [--force]

The translation units (C ABI, one per element type, the built-in scratch area) are compiled in
parallel and linked into matchattention_b200/lib/libmatchattn_b200.so.  The
library carries its own static CUDA runtime and has no Python or torch
dependency.
"""
from __future__ import annotations

import concurrent.futures
import os
import shutil
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG, "csrc")
LIB_DIR = os.path.join(PKG, "lib")
OBJ_DIR = os.path.join(PKG, "build")
LIB_PATH = os.path.join(LIB_DIR, "libmatchattn_b200.so")
INCLUDE = os.path.join(os.path.dirname(PKG), "include")

SOURCES = ["matchattn_api.cu", "matchattn_f32.cu", "matchattn_f16.cu", "matchattn_bf16.cu",
           "matchattn_static_scratch.cu", "matchattn_upsample.cu", "matchattn_volume.cu", "matchattn_field_ops.cu", "matchattn_flow_init.cu", "matchattn_backward.cu"]
HEADERS = ["matchattn_kernels.cuh", "matchattn_launch.inl", "matchattn_mma.cuh", "matchattn_binned.cuh",
           "matchattn_staged.cuh"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC,-fvisibility=hidden", "-Xptxas", "-v"]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found: the CUDA extension cannot be built on this machine")
    return exe


def _stale() -> bool:
    if not os.path.exists(LIB_PATH):
        return True
    built = os.path.getmtime(LIB_PATH)
    deps = [os.path.join(CSRC, f) for f in SOURCES + HEADERS] + [os.path.join(INCLUDE, "matchattn.h")]
    return any(os.path.getmtime(d) > built for d in deps)


def _compile(src: str) -> tuple[str, str]:
    obj = os.path.join(OBJ_DIR, src.replace(".cu", ".o"))
    extra = os.environ.get("MATCHATTN_NVCC_EXTRA", "").split()      # e.g. -DMATCHATTN_FAST_EXP=1 for experiments
    cmd = [_nvcc(), *NVCC_FLAGS, *extra, "-I", INCLUDE, "-c", os.path.join(CSRC, src), "-o", obj]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed on {src}:\n{res.stdout}\n{res.stderr}")
    return obj, res.stderr


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and not _stale():
        return LIB_PATH
    os.makedirs(LIB_DIR, exist_ok=True)
    os.makedirs(OBJ_DIR, exist_ok=True)
    with concurrent.futures.ThreadPoolExecutor(max_workers=len(SOURCES)) as pool:
        results = list(pool.map(_compile, SOURCES))
    log = "\n".join(r[1] for r in results)
    with open(os.path.join(OBJ_DIR, "ptxas.log"), "w") as f:
        f.write(log)
    if verbose:
        print(log)
    cmd = [_nvcc(), "-shared", "-o", LIB_PATH, *[r[0] for r in results], "-cudart", "static"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    return LIB_PATH


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print(path)
