"""Host-side mirror of the oxicuda-blas quantized GEMM/GEMV surface on this path.

Names follow `crates/oxicuda-blas/src/precision/{fp8_ops,fp4_fp6_ops,int_ops}.rs` and
`level3/gemm_api.rs`; every numeric call goes through the C ABI to a CUDA kernel.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from enum import Enum

import torch

from . import _lib as L
from ._lib import TileConfig, default_handle, lib, ptr
from .quant import _back, _dev


class Fp8WorkloadClass(Enum):
    """crates/oxicuda-blas/src/precision/fp8_ops.rs:42-61"""
    SmallSquare = 0
    LargeSquare = 1
    SkinnyM = 2
    SkinnyN = 3
    SkinnyK = 4
    General = 5


def classify_workload(m: int, n: int, k: int) -> Fp8WorkloadClass:
    """fp8_ops.rs:67-87"""
    return Fp8WorkloadClass(lib().b2q_classify_workload(m, n, k))


def _ref_tile(dtype: int, m: int, n: int, k: int) -> TileConfig:
    t = TileConfig()
    st = lib().b2q_ref_tile_config(dtype, m, n, k, C.byref(t))
    if st == L.ERR_INVALID_DIMENSION:
        raise L.InvalidDimension(st, f"GEMM dimensions must be non-zero: m={m}, n={n}, k={k}")
    if st != L.OK:
        raise L.InvalidArgument(st, "b2q_ref_tile_config")
    return t


class Fp8Config:
    """Fp8Config, crates/oxicuda-blas/src/precision/fp8_ops.rs:320-397 (Blackwell arm)."""
    ELEMENT_BYTES = 1

    @staticmethod
    def tile_config(m: int, n: int, k: int) -> TileConfig:
        return _ref_tile(0, m, n, k)

    @staticmethod
    def compute_split_k(m: int, n: int, k: int) -> int:
        return int(lib().b2q_fp8_compute_split_k(m, n, k))


def select_fp4_tile(m: int, n: int, k: int) -> TileConfig:
    """select_fp4_tile, crates/oxicuda-blas/src/precision/fp4_fp6_ops.rs:996-1075 (Sm100 arm)."""
    return _ref_tile(1, m, n, k)


def int8_tile_config(m: int, n: int, k: int) -> TileConfig:
    """Int8GemmConfig::tile_config, crates/oxicuda-blas/src/precision/int_ops.rs:141-176 (Sm100 arm)."""
    return _ref_tile(2, m, n, k)


def select_tile(dtype: str, m: int, n: int, k: int):
    """The static per-shape table the kernels are dispatched with: (TileConfig, kernel_id)."""
    t, kid = TileConfig(), C.c_int()
    st = lib().b2q_select_tile({"fp8": 0, "fp4": 1, "int8": 2}[dtype], m, n, k, C.byref(t), C.byref(kid))
    if st != L.OK:
        raise L.InvalidDimension(st, "b2q_select_tile")
    return t, kid.value


# ---------------------------------------------------------------------------
# FP4 / micro-scaling
# ---------------------------------------------------------------------------
class Fp4Format(Enum):
    """crates/oxicuda-blas/src/precision/fp4_fp6_ops.rs:107-134"""
    E2M1 = 0
    Int4 = 1

    def max_value(self) -> float:
        return 6.0 if self is Fp4Format.E2M1 else 8.0


class ScalingFormat(Enum):
    """fp4_fp6_ops.rs:142-171, plus E8M0 (absent from the reference)."""
    Fp32 = 0
    E8M0 = 1


@dataclass
class MicroScalingConfig:
    """fp4_fp6_ops.rs:190-225"""
    block_size: int = 32
    scaling_format: ScalingFormat = ScalingFormat.Fp32
    VALID_BLOCK_SIZES = (32, 64, 128)

    def validate(self):
        if self.block_size not in self.VALID_BLOCK_SIZES:
            raise L.InvalidArgument(L.ERR_INVALID_ARGUMENT,
                                    f"MicroScaling block_size must be one of [32, 64, 128], got {self.block_size}")

    def num_scales(self, num_elements: int) -> int:
        return -(-num_elements // self.block_size)


class PackedFp4:
    """PackedFp4::{pack,unpack}, fp4_fp6_ops.rs:452-481 (pure byte helpers)."""

    @staticmethod
    def pack(v0: int, v1: int) -> int:
        if v0 > 15 or v1 > 15:
            raise L.InvalidArgument(L.ERR_INVALID_ARGUMENT, f"FP4 raw values must be <= 15: got ({v0}, {v1})")
        return v0 | (v1 << 4)

    @staticmethod
    def unpack(b: int):
        return b & 0x0F, (b >> 4) & 0x0F


class MicroScalingQuantizer:
    """MicroScalingQuantizer, fp4_fp6_ops.rs:746-898: block absmax scale + E2M1/INT4 codes."""

    def __init__(self, config: MicroScalingConfig):
        self.config = config

    def quantize_fp4(self, values: torch.Tensor, format: Fp4Format = Fp4Format.E2M1):
        """fp4_fp6_ops.rs:849-876 -> (packed u8 [n/2], scales f32 or u8 [n/block])."""
        self.config.validate()
        x, was_host = _dev(values.reshape(-1), torch.float32)
        n, blk = x.numel(), self.config.block_size
        e8 = self.config.scaling_format == ScalingFormat.E8M0
        packed = torch.empty((n + 1) // 2, dtype=torch.uint8, device=x.device)
        scales = torch.empty(-(-n // blk), dtype=torch.uint8 if e8 else torch.float32, device=x.device)
        default_handle().call("b2q_fp4_block_quantize_f32", ptr(x), n, blk, format.value,
                              L.SCALE_E8M0 if e8 else L.SCALE_F32, ptr(packed), ptr(scales))
        return _back(packed, was_host), _back(scales, was_host)

    def dequantize_fp4(self, packed: torch.Tensor, scales: torch.Tensor, format: Fp4Format, original_len: int):
        """fp4_fp6_ops.rs:879-897"""
        self.config.validate()
        p, was_host = _dev(packed.reshape(-1), torch.uint8)
        e8 = self.config.scaling_format == ScalingFormat.E8M0
        s, _ = _dev(scales.reshape(-1), torch.uint8 if e8 else torch.float32)
        out = torch.empty(original_len, dtype=torch.float32, device=p.device)
        default_handle().call("b2q_fp4_block_dequantize_f32", ptr(p), original_len, self.config.block_size,
                              format.value, L.SCALE_E8M0 if e8 else L.SCALE_F32, ptr(s), ptr(out))
        return _back(out, was_host)


# ---------------------------------------------------------------------------
# GEMM / GEMV (device tensors in, device tensors out; asynchronous on the current stream)
# ---------------------------------------------------------------------------
def _scale_kind(s: torch.Tensor, n: int) -> int:
    if s.numel() == 1:
        return L.SCALE_SCALAR
    if s.numel() == n:
        return L.SCALE_PER_ROW
    raise L.DimensionMismatch(L.ERR_DIMENSION_MISMATCH, f"scale has {s.numel()} entries, expected 1 or {n}")


def gemm_fp8(a: torch.Tensor, w: torch.Tensor, scale_a: torch.Tensor, scale_w: torch.Tensor, out: torch.Tensor = None,
             out_dtype=torch.bfloat16, fmt: int = L.FP8_E4M3, simt_decode: str = None) -> torch.Tensor:
    """out[M,N] = (A[M,K] . W[N,K]^T) * scale_a * scale_w.  The working replacement of gemm::<E4M3>
    (crates/oxicuda-blas/src/level3/gemm_api.rs:82-231).  `simt_decode` in {"ref","ieee"} runs the
    k-ascending fp32 checker kernel instead of the tensor-core kernel."""
    M, K = a.shape
    N, K2 = w.shape
    if K != K2:
        raise L.DimensionMismatch(L.ERR_DIMENSION_MISMATCH, f"inner dimensions differ: {K} vs {K2}")
    if out is None:
        out = torch.empty(M, N, dtype=out_dtype, device=a.device)
    ot = L.OUT_BF16 if out.dtype == torch.bfloat16 else L.OUT_F32
    h = default_handle()
    args = (ptr(scale_a), _scale_kind(scale_a, M), ptr(scale_w), _scale_kind(scale_w, N), ptr(out), ot)
    if simt_decode is None:
        h.call("b2q_gemm_fp8", ptr(a), ptr(w), M, N, K, fmt, *args)
    else:
        h.call("b2q_gemm_fp8_simt", ptr(a), ptr(w), M, N, K, fmt, 0 if simt_decode == "ref" else 1, *args)
    return out


class EpilogueOp(Enum):
    """EpilogueOp, crates/oxicuda-blas/src/level3/gemm/epilogue.rs:29-45."""
    LinearCombination = 0
    LinearCombinationRelu = 1
    LinearCombinationGelu = 2
    LinearCombinationBias = 3
    LinearCombinationBiasRelu = 4
    # not in the reference: w holds gate and up rows interleaved per 128, out [M x N / 2] = silu(gate) * up
    # (SwiGluExpert::forward, crates/oxicuda-moe/src/expert/ffn.rs:208-243)
    SwiGluPairs = 5

    def needs_bias(self) -> bool:
        return self in (EpilogueOp.LinearCombinationBias, EpilogueOp.LinearCombinationBiasRelu)


def gemm_fp8_ex(a: torch.Tensor, w: torch.Tensor, scale_a: torch.Tensor, scale_w: torch.Tensor, out: torch.Tensor = None,
                alpha: float = 1.0, beta: float = 0.0, bias: torch.Tensor = None, epilogue: EpilogueOp = EpilogueOp.LinearCombination,
                w_is_kn: bool = False, out_dtype=torch.bfloat16, fmt: int = L.FP8_E4M3) -> torch.Tensor:
    """gemm_impl with an EpilogueOp (crates/oxicuda-blas/src/level3/gemm_api.rs:126-231, gemm/epilogue.rs:99-196):
    out = act(alpha * (A . W^T) * scale_a * scale_w + beta * out + bias[col]).  `w` is [N x K], or with w_is_kn the
    reference's row-major [K x N] operand B.  With beta != 0 `out` must hold C on entry.  EpilogueOp.SwiGluPairs: `w`
    holds gate and up rows interleaved per 128 and out is [M x N / 2] = silu(gate) * up."""
    import ctypes as C
    M, K = a.shape
    if w_is_kn:
        K2, N = w.shape
    else:
        N, K2 = w.shape
    if K != K2:
        raise L.DimensionMismatch(L.ERR_DIMENSION_MISMATCH, f"inner dimensions differ: {K} vs {K2}")
    if epilogue.needs_bias() and bias is None:
        raise L.InvalidArgument(L.ERR_INVALID_ARGUMENT, f"{epilogue.name} needs a bias vector")
    if out is None:
        if beta != 0.0:
            raise L.InvalidArgument(L.ERR_INVALID_ARGUMENT, "beta != 0 needs the C operand in `out`")
        out = torch.empty(M, N // 2 if epilogue is EpilogueOp.SwiGluPairs else N, dtype=out_dtype, device=a.device)
    d = L.GemmFp8Desc(a.data_ptr(), w.data_ptr(), M, N, K, fmt, scale_a.data_ptr(), _scale_kind(scale_a, M), scale_w.data_ptr(),
                      _scale_kind(scale_w, N), out.data_ptr(), L.OUT_BF16 if out.dtype == torch.bfloat16 else L.OUT_F32, alpha, beta,
                      bias.data_ptr() if bias is not None else None, epilogue.value, 1 if w_is_kn else 0)
    default_handle().call("b2q_gemm_fp8_ex", C.byref(d))
    return out


def gemm_i8(a: torch.Tensor, b: torch.Tensor, scale_a: torch.Tensor = None, scale_b: torch.Tensor = None,
            want_s32: bool = True, want_f32: bool = False):
    """C[M,N] = A[M,K] . B[N,K]^T with exact s32 accumulation (Int8GemmConfig,
    crates/oxicuda-blas/src/precision/int_ops.rs:78-189).  Returns (c_s32 | None, c_f32 | None)."""
    M, K = a.shape
    N, K2 = b.shape
    if K != K2:
        raise L.DimensionMismatch(L.ERR_DIMENSION_MISMATCH, f"inner dimensions differ: {K} vs {K2}")
    c32 = torch.empty(M, N, dtype=torch.int32, device=a.device) if want_s32 else None
    cf = torch.empty(M, N, dtype=torch.float32, device=a.device) if want_f32 else None
    default_handle().call("b2q_gemm_i8", ptr(a), ptr(b), M, N, K, ptr(c32), ptr(cf), ptr(scale_a), ptr(scale_b))
    return c32, cf


def gemv_fp4_wo(codes: torch.Tensor, scales: torch.Tensor, x: torch.Tensor, N: int, K: int, out: torch.Tensor = None,
                out_dtype=torch.bfloat16, block: int = 32) -> torch.Tensor:
    """out[tokens,N] = x[tokens,K] . dequant(codes[N,K/2], scales[N,K/block])^T  (tokens <= 32).
    Fp4GemmConfig semantics, crates/oxicuda-blas/src/precision/fp4_fp6_ops.rs:337-395 / :879-897."""
    tokens = x.shape[0]
    if out is None:
        out = torch.empty(tokens, N, dtype=out_dtype, device=x.device)
    sf = L.SCALE_E8M0 if scales.dtype == torch.uint8 else L.SCALE_F32
    ot = L.OUT_BF16 if out.dtype == torch.bfloat16 else L.OUT_F32
    default_handle().call("b2q_gemv_fp4_wo", ptr(codes), ptr(scales), sf, block, ptr(x), tokens, N, K, ptr(out), ot)
    return out


def gemm_fp4_wo(codes: torch.Tensor, scales: torch.Tensor, x: torch.Tensor, N: int, K: int, out: torch.Tensor = None,
                out_dtype=torch.bfloat16, block: int = 32, format: Fp4Format = Fp4Format.E2M1) -> torch.Tensor:
    """Weight-only FP4 GEMM for any token count: decode GEMV at 32 tokens or fewer, bf16 expansion + tcgen05 above
    (Fp4GemmConfig, crates/oxicuda-blas/src/precision/fp4_fp6_ops.rs:337-395)."""
    tokens = x.shape[0]
    if out is None:
        out = torch.empty(tokens, N, dtype=out_dtype, device=x.device)
    sf = L.SCALE_E8M0 if scales.dtype == torch.uint8 else L.SCALE_F32
    ot = L.OUT_BF16 if out.dtype == torch.bfloat16 else L.OUT_F32
    default_handle().call("b2q_gemm_fp4_wo", ptr(codes), ptr(scales), sf, block, format.value, ptr(x), tokens, N, K, ptr(out), ot)
    return out


def gemm_fp4_blockscaled(codes: torch.Tensor, scales: torch.Tensor, x: torch.Tensor, N: int, K: int, mxfp8_activations: bool = False,
                         out: torch.Tensor = None, out_dtype=torch.bfloat16) -> torch.Tensor:
    """b2q_gemm_fp4_blockscaled: E2M1 codes + E8M0 block-32 scales on tcgen05 kind::mxf8f6f4.block_scale.  Default: split
    activations (weight-only semantics); mxfp8_activations=True quantizes them to MX E4M3 (W4A8)."""
    tokens = x.shape[0]
    if out is None:
        out = torch.empty(tokens, N, dtype=out_dtype, device=x.device)
    ot = L.OUT_BF16 if out.dtype == torch.bfloat16 else L.OUT_F32
    default_handle().call("b2q_gemm_fp4_blockscaled", ptr(codes), ptr(scales), ptr(x), tokens, N, K, 1 if mxfp8_activations else 0, ptr(out), ot)
    return out


# ---- INT4 group-scaled weight-only linear: crates/oxicuda-blas/src/precision/int_ops.rs:196-429, :602-757 ----
@dataclass
class Int4GemmConfig:
    """int_ops.rs:215-356"""
    m: int
    n: int
    k: int
    layout_a: str = "RowMajor"
    layout_b: str = "RowMajor"
    group_size: int = 128

    PACKED_ELEMENT_BYTES = 4
    VALUES_PER_U32 = 8
    VALID_GROUP_SIZES = (32, 64, 128, 256)

    def validate(self) -> None:
        """int_ops.rs:250-283 (the architecture check always passes on sm_100)."""
        if self.m == 0 or self.n == 0 or self.k == 0:
            raise L.InvalidDimension(L.ERR_INVALID_DIMENSION, f"INT4 GEMM dimensions must be non-zero: m={self.m}, n={self.n}, k={self.k}")
        if self.k % 8 != 0:
            raise L.InvalidDimension(L.ERR_INVALID_DIMENSION, f"INT4 GEMM K dimension must be a multiple of 8 for packing, got k={self.k}")
        if self.group_size == 0 or self.group_size & (self.group_size - 1):
            raise L.InvalidArgument(L.ERR_INVALID_ARGUMENT, f"INT4 group_size must be a positive power of 2, got {self.group_size}")
        if self.k % self.group_size != 0:
            raise L.InvalidArgument(L.ERR_INVALID_ARGUMENT, f"INT4 group_size ({self.group_size}) must divide K ({self.k}) evenly")

    def tile_config(self) -> tuple:
        """int_ops.rs:296-309, the Hopper/Blackwell row: (tile_m, tile_n, tile_k, warp_m, warp_n, stages, tensor core, split_k)."""
        return (128, 128, 128, 64, 64, 4, 1, 1)

    def kernel_name(self) -> str:
        short = {"RowMajor": "r", "ColMajor": "c"}
        return f"int4_gemm_{self.m}x{self.n}x{self.k}_{short[self.layout_a]}{short[self.layout_b]}_f32_gs{self.group_size}"

    def num_groups(self) -> int:
        return self.k // self.group_size

    def packed_k(self) -> int:
        return self.k // self.VALUES_PER_U32


def pack_int4(values: torch.Tensor) -> torch.Tensor:
    """int_ops.rs:375-403: int8 values in [-8, 7], a multiple of 8 of them -> u32 words (as int32 tensors hold them)."""
    n = values.numel()
    if n % 8 != 0:
        raise L.InvalidArgument(L.ERR_INVALID_ARGUMENT, f"pack_int4 requires input length to be a multiple of 8, got {n}")
    v, was_host = _dev(values.reshape(-1), torch.int8)
    packed = torch.empty(n // 8, dtype=torch.int32, device=v.device)
    h = default_handle()
    h.call("b2q_pack_int4", ptr(v), n, ptr(packed))
    h.check()                       # a value outside [-8, 7] is detected on the device
    return _back(packed, was_host)


def unpack_int4(packed) -> torch.Tensor:
    """int_ops.rs:415-429 for one word (an int) or a tensor of words -> int8 values."""
    if isinstance(packed, int):
        packed = torch.tensor([packed if packed < (1 << 31) else packed - (1 << 32)], dtype=torch.int32)
    p, was_host = _dev(packed.reshape(-1), torch.int32)
    out = torch.empty(p.numel() * 8, dtype=torch.int8, device=p.device)
    default_handle().call("b2q_unpack_int4", ptr(p), p.numel(), ptr(out))
    return _back(out, was_host)


def gemm_int4(a_packed: torch.Tensor, scales: torch.Tensor, b: torch.Tensor, config: Int4GemmConfig) -> torch.Tensor:
    """The kernel of generate_int4_gemm_ptx (int_ops.rs:602-757): C[m, n] f32 = dequant(A packed [m, k/8], scales f16
    [m, k/group]) @ B f32 [k, n], summed over k ascending exactly as the reference kernel does."""
    config.validate()
    c = torch.empty(config.m, config.n, dtype=torch.float32, device=a_packed.device)
    default_handle().call("b2q_gemm_int4_f32", ptr(a_packed), ptr(scales), ptr(b.contiguous()), ptr(c), config.m, config.n, config.k,
                          config.group_size)
    return c


def gemv_int4_wo(packed: torch.Tensor, scales: torch.Tensor, group_size: int, x: torch.Tensor, N: int, K: int, out: torch.Tensor = None,
                 out_dtype=torch.bfloat16) -> torch.Tensor:
    """Decode form: out[tokens, N] = x[tokens, K] (bf16) @ dequant(W[N, K])^T; tokens <= 32, K % 128 == 0, group_size >= 32."""
    tokens = x.shape[0]
    if out is None:
        out = torch.empty(tokens, N, dtype=out_dtype, device=x.device)
    ot = L.OUT_BF16 if out.dtype == torch.bfloat16 else L.OUT_F32
    default_handle().call("b2q_gemv_int4_wo", ptr(packed), ptr(scales), group_size, ptr(x.contiguous()), tokens, N, K, ptr(out), ot)
    return out
