"""Builds libframe_b200.so (CUDA kernels + C ABI) for sm_100a with nvcc, in-tree.

    python -m frame_public_b200.build            # incremental
    python -m frame_public_b200.build --force

nvcc cross-compiles without a GPU.  The shared library lands in frame_public_b200/lib/ and is
what the ctypes binding (capi.py) and the C++ adapter load.
"""
from __future__ import annotations

import concurrent.futures
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB_DIR = os.path.join(HERE, "lib")
OBJ_DIR = os.path.join(LIB_DIR, "obj")
LIB_PATH = os.path.join(LIB_DIR, "libframe_b200.so")

NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC,-fvisibility=hidden",
          "-I", os.path.join(HERE, "..", "include")]

# Kernels whose arithmetic must round exactly like the CPU reference (built with
# -ffp-contract=off): no fused multiply-add.
NO_FMA = {"elementwise.cu", "rowops.cu", "scan.cu", "scan_chunked.cu", "conv_pool.cu", "gemm_simt.cu", "shape_ops.cu", "grad_ops.cu"}

SOURCES = ["runtime.cu", "elementwise.cu", "rowops.cu", "scan.cu", "shape_ops.cu", "conv_pool.cu",
           "gemm_simt.cu", "gemm_tcgen05.cu", "conv_tcgen05.cu", "plan.cu", "mamba_scan.cu", "scan_chunked.cu",
           "attention_tcgen05.cu", "conv_halo_tcgen05.cu", "conv_planes_tcgen05.cu", "conv_rows_tcgen05.cu", "index_ops.cu", "grad_ops.cu", "fft_ops.cu"]


def _headers_mtime() -> float:
    paths = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    paths.append(os.path.join(HERE, "..", "include", "frame_b200.h"))
    return max(os.path.getmtime(p) for p in paths)


def _compile(src: str, force: bool, verbose: bool) -> str:
    obj = os.path.join(OBJ_DIR, src.replace(".cu", ".o"))
    path = os.path.join(CSRC, src)
    if (not force and os.path.exists(obj)
            and os.path.getmtime(obj) > max(os.path.getmtime(path), _headers_mtime())):
        return obj
    cmd = [NVCC, *ARCH, *COMMON, "-c", path, "-o", obj]
    if src in NO_FMA:
        cmd.insert(1, "-fmad=false")
    if verbose:
        cmd.insert(1, "-Xptxas=-v")
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src}:\n{res.stdout}\n{res.stderr}")
    if verbose:
        sys.stderr.write(res.stderr)
    return obj


def build(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(OBJ_DIR, exist_ok=True)
    sources = [s for s in SOURCES if os.path.exists(os.path.join(CSRC, s))]
    with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, len(sources))) as pool:
        objs = list(pool.map(lambda s: _compile(s, force, verbose), sources))
    if (force or not os.path.exists(LIB_PATH)
            or any(os.path.getmtime(o) > os.path.getmtime(LIB_PATH) for o in objs)):
        cmd = [NVCC, *ARCH, "-shared", "-o", LIB_PATH, *objs, "-lpthread", "-ldl",
               "-Xlinker", "--version-script=" + os.path.join(CSRC, "exports.map")]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    return LIB_PATH


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
