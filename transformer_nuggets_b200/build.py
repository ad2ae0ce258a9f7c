"""Build ``libtnq.so`` (the C-ABI CUDA library) in-tree for sm_100a.

    python -m transformer_nuggets_b200.build [--force] [--verbose]

nvcc cross-compiles without a GPU.  Objects go to ``build/`` at the repository
root, the library next to the sources.  Nothing here falls back to another
architecture or to a CPU implementation.
"""

from __future__ import annotations

import concurrent.futures
import os
import shutil
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
OBJ_DIR = os.path.join(ROOT, "build", "tnq")
LIB_PATH = os.path.join(CSRC, "libtnq.so")

SOURCES = ["fp8_tensor.cu", "fp8_fused.cu", "fp8_rowwise.cu", "mxfp8.cu", "nvfp4.cu", "to_blocked.cu", "exchange.cu", "gemv.cu", "delayed.cu", "fp8_transpose.cu", "tile_copy.cu", "producer_quant.cu", "fp8_gemm.cu", "mxfp8_gemm.cu", "nvfp4_gemm.cu"]
HEADERS = ["common.cuh", "tile_pipeline.cuh", "mx_scale.cuh", os.path.join(ROOT, "include", "tnq.h")]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-std=c++17", "-O3", "-lineinfo",
    "-Xcompiler", "-fPIC",
    "-Xptxas", "-v",
]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found; libtnq.so cannot be built")
    return exe


def _sources():
    return [s for s in SOURCES if os.path.exists(os.path.join(CSRC, s))]


def _newest_input() -> float:
    paths = [os.path.join(CSRC, s) for s in _sources()]
    paths += [h if os.path.isabs(h) else os.path.join(CSRC, h) for h in HEADERS]
    paths.append(os.path.abspath(__file__))
    return max(os.path.getmtime(p) for p in paths if os.path.exists(p))


def is_current() -> bool:
    return os.path.exists(LIB_PATH) and os.path.getmtime(LIB_PATH) >= _newest_input()


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and is_current():
        return LIB_PATH
    os.makedirs(OBJ_DIR, exist_ok=True)
    nvcc = _nvcc()

    def compile_one(src):
        obj = os.path.join(OBJ_DIR, src.replace(".cu", ".o"))
        cmd = [nvcc, *NVCC_FLAGS, "-c", os.path.join(CSRC, src), "-o", obj]
        r = subprocess.run(cmd, capture_output=True, text=True)
        log = r.stdout + r.stderr
        with open(obj + ".log", "w") as f:
            f.write(" ".join(cmd) + "\n" + log)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src}:\n{log}")
        if verbose:
            print(log)
        return obj

    with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as ex:
        objs = list(ex.map(compile_one, _sources()))
    tmp = LIB_PATH + ".tmp"
    cmd = [nvcc, "-shared", "-o", tmp, *objs, "-gencode", "arch=compute_100a,code=sm_100a"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("link failed:\n" + r.stdout + r.stderr)
    os.replace(tmp, LIB_PATH)
    return LIB_PATH


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(path)
