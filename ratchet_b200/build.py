"""Builds libratchet_b200.so in-tree with nvcc for sm_100a (cross-compiles without a GPU).

    python -m ratchet_b200.build [--force] [--verbose]
"""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
OBJ = os.path.join(CSRC, "build")
LIB = os.path.join(PKG, "libratchet_b200.so")
INCLUDE = os.path.join(ROOT, "include")

SOURCES = [
    "spec.cpp",
    "arena.cpp",
    "quant_host.cpp",
    "gguf_reader.cpp",
    "comm.cpp",
    "api.cu",
    "matmul_simt.cu",
    "gemv_q8_mma.cu",
    "gemv_q8_umma.cu", "gemv_q8_chain.cu",
    "gemv_q4k_mma.cu", "gemv_q4k_umma.cu",
    "dequant.cu",
    "gemm_umma.cu", "gemm_umma_tf32.cu",
    "static_scratch.cu",
]

NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC,-Wall,-Wno-unused-function",
          "-I", INCLUDE, "-I", CSRC]


def _deps_mtime() -> float:
    m = 0.0
    for d in (CSRC, INCLUDE):
        for f in os.listdir(d):
            if f.endswith((".h", ".hpp", ".cuh")):
                m = max(m, os.path.getmtime(os.path.join(d, f)))
    return m


def _compile(src: str, force: bool, verbose: bool, hdr_mtime: float) -> str:
    obj = os.path.join(OBJ, os.path.splitext(src)[0] + ".o")
    path = os.path.join(CSRC, src)
    if (not force and os.path.exists(obj)
            and os.path.getmtime(obj) >= max(os.path.getmtime(path), hdr_mtime)):
        return obj
    cmd = [NVCC, *ARCH, *COMMON, "-c", path, "-o", obj]
    if verbose and src.endswith(".cu"):
        cmd[1:1] = ["-Xptxas", "-v"]
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src}:\n{r.stdout}")
    if verbose and r.stdout.strip():
        print(f"--- {src}\n{r.stdout}")
    return obj


def build(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(OBJ, exist_ok=True)
    hdr = _deps_mtime()
    with ThreadPoolExecutor(max_workers=min(8, len(SOURCES))) as ex:
        objs = list(ex.map(lambda s: _compile(s, force, verbose, hdr), SOURCES))
    if force or not os.path.exists(LIB) or any(os.path.getmtime(o) > os.path.getmtime(LIB) for o in objs):
        cmd = [NVCC, *ARCH, "-shared", "-o", LIB, *objs, "-lcudart", "-ldl"]
        r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}")
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
