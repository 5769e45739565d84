"""oxicuda_b200 — B200-native (sm_100a) quantized linear-layer path behind the OxiCUDA quant/BLAS API.

`quant`  mirrors oxicuda-quant's quantize/dequantize entry points,
`blas`   mirrors oxicuda-blas's INT8 / FP8 / block-scaled FP4 GEMM, GEMV and tile heuristics,
`dist_infer` mirrors oxicuda-dist-infer's column/row-parallel linears over NCCL.
All numeric work happens in libb2q.so (CUDA, C ABI: include/b2q.h); nothing falls back to the CPU.
"""
from . import _lib  # noqa: F401

__all__ = ["quant", "blas", "dist_infer", "_lib"]
