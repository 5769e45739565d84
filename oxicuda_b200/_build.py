"""Builds libb2q.so (the C-ABI CUDA library) in-tree for sm_100a.

nvcc cross-compiles without a GPU, so this runs on a CPU-only machine too.  The
objects are compiled in parallel and linked with the static CUDA runtime so that
the library loads (and its symbols can be listed) on a box without a driver.
"""
from __future__ import annotations

import os
import shutil
import subprocess
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
LIB = PKG / "libb2q.so"
SOURCES = ["handle.cu", "quant.cu", "kv_cache.cu", "norm_quant.cu", "dnn_quant.cu", "int8.cu", "gemm_fp8_simt.cu", "gemm_tc.cu", "gemv_fp4.cu", "gemv_fp4_mx.cu", "gemv_fp4_mxf4.cu", "gemv_int4.cu", "gemv_fp8.cu", "gemm_fp8_skinny.cu", "moe.cu", "gemm_fp4.cu", "gemm_fp4_bs.cu", "tp.cu", "ggml.cu", "gptq_awq.cu"]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17",
    "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", shutil.which("nvcc")):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found: libb2q.so cannot be built")


def _stale() -> bool:
    if not LIB.exists():
        return True
    t = LIB.stat().st_mtime
    deps = [CSRC / s for s in SOURCES] + [CSRC / "common.cuh", CSRC / "tc_common.cuh", PKG.parent / "include" / "b2q.h"]
    return any(d.stat().st_mtime > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> Path:
    if not force and not _stale():
        return LIB
    nvcc = _nvcc()
    objdir = PKG / "build"
    objdir.mkdir(exist_ok=True)

    def compile_one(src: str) -> str:
        obj = objdir / (src + ".o")
        cmd = [nvcc, *NVCC_FLAGS, "-c", str(CSRC / src), "-o", str(obj)]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src}:\n{r.stderr}")
        if verbose:
            print(r.stderr)
        return str(obj)

    with ThreadPoolExecutor(max_workers=min(8, len(SOURCES))) as ex:
        objs = list(ex.map(compile_one, SOURCES))
    r = subprocess.run([nvcc, "-shared", "-o", str(LIB), *objs, "-cudart", "static", "-ldl"], capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link failed:\n{r.stderr}")
    return LIB


if __name__ == "__main__":
    import sys
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
