"""Ahead-of-time build of ``libdpk_b200.so`` (sm_100a only) with nvcc.

The reference compiles its kernels at run time, per shape, through a JIT loader
(``DynamicPruningKernels/python/utils.py:55-60``); this build compiles a small
fixed set of kernels once.  nvcc cross-compiles without a GPU, so the build also
runs on a CPU-only machine.

    python -m dpk_b200.build [--force] [--verbose]
"""

from __future__ import annotations

import concurrent.futures as cf
import os
import shutil
import subprocess
import sys

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG_DIR)
CSRC = os.path.join(ROOT, "csrc")
LIB_DIR = os.path.join(ROOT, "lib")
OBJ_DIR = os.path.join(LIB_DIR, "obj")
LIB_PATH = os.path.join(LIB_DIR, "libdpk_b200.so")

SOURCES = [
    "dpk_host.cu",
    "dpk_route.cu",
    "dpk_gemm_mn.cu",
    "dpk_gemm_mn_pair.cu",
    "dpk_gemm_k.cu",
    "dpk_gemm_k_pair.cu",
    "dpk_gemv.cu",
    "dpk_ffn.cu",
    "dpk_attn_prefill.cu",
    "dpk_attn_prefill_tc.cu",
    "dpk_attn_prefill_tc2.cu",
    "dpk_attn_decode.cu",
    "dpk_peer.cu",
    "dpk_router_norm.cu",
    "dpk_rope.cu",
    "dpk_ffn_small.cu",
]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
    "-Xptxas", "-v",
]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found; the CUDA toolkit is required to build dpk_b200")
    return exe


def _deps_mtime() -> float:
    newest = 0.0
    for d in (CSRC, os.path.join(os.path.dirname(ROOT), "include")):
        for name in os.listdir(d):
            if name.endswith((".cu", ".cuh", ".h")):
                newest = max(newest, os.path.getmtime(os.path.join(d, name)))
    return newest


def _compile(src: str, verbose: bool) -> str:
    obj = os.path.join(OBJ_DIR, os.path.splitext(src)[0] + ".o")
    cmd = [_nvcc(), *NVCC_FLAGS, "-c", os.path.join(CSRC, src), "-o", obj]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed on {src}:\n{res.stdout}\n{res.stderr}")
    if verbose:
        sys.stderr.write(res.stderr)
    with open(obj + ".ptxas.txt", "w") as f:
        f.write(res.stderr)
    return obj


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile every kernel for sm_100a and link the shared library in-tree."""
    os.makedirs(OBJ_DIR, exist_ok=True)
    if not force and os.path.exists(LIB_PATH) and os.path.getmtime(LIB_PATH) >= _deps_mtime():
        return LIB_PATH
    with cf.ThreadPoolExecutor(max_workers=min(8, len(SOURCES))) as pool:
        objs = list(pool.map(lambda s: _compile(s, verbose), SOURCES))
    cmd = [_nvcc(), "-shared", "-o", LIB_PATH, *objs]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    return LIB_PATH


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(path)
