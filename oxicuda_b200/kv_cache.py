"""Host-side mirror of the KV-cache quantizers either side of the quantized linear path.

`KvCacheQuantizer` / `KvCacheConfig` / `QuantizedKvCache` follow crates/oxicuda-quant/src/scheme/kv_cache.rs,
`KvQuantConfig` / `QuantizedToken(s)` / `quantize_token` follow crates/oxicuda-infer/src/cache/kv_quant.rs, and
`rms_norm_quantize_fp8` is the RMSNorm of crates/oxicuda-dnn/src/norm/rms_norm.rs fused with the per-token FP8
quantizer that feeds the next linear.  Same names, argument meaning and error behaviour as the reference; the
arithmetic runs in CUDA kernels through the C ABI.  Host tensors are uploaded and results come back on the host.
"""
from __future__ import annotations

from dataclasses import dataclass
from enum import Enum

import torch

from . import _lib as L
from ._lib import default_handle, ptr
from .quant import _back, _dev


class KvAxis(Enum):
    """crates/oxicuda-quant/src/scheme/kv_cache.rs:33-38"""
    PerToken = 0
    PerChannel = 1


@dataclass
class KvCacheConfig:
    """kv_cache.rs:43-86"""
    bits: int
    axis: KvAxis

    @staticmethod
    def new(bits: int, axis: KvAxis) -> "KvCacheConfig":
        if not 2 <= bits <= 8:
            raise L.InvalidBitWidth(L.ERR_INVALID_BIT_WIDTH, f"invalid bit-width {bits}")
        return KvCacheConfig(bits, axis)

    @staticmethod
    def keys_int8() -> "KvCacheConfig":
        return KvCacheConfig(8, KvAxis.PerChannel)

    @staticmethod
    def values_int8() -> "KvCacheConfig":
        return KvCacheConfig(8, KvAxis.PerToken)


@dataclass
class QuantizedKvCache:
    """kv_cache.rs:91-120.  `codes` u8 [n_tokens*head_dim]; `scales`, `zero_points` f32 [n_groups]."""
    codes: torch.Tensor
    scales: torch.Tensor
    zero_points: torch.Tensor
    n_tokens: int
    head_dim: int
    bits: int
    axis: KvAxis

    def n_groups(self) -> int:
        return self.n_tokens if self.axis == KvAxis.PerToken else self.head_dim

    def packed_bytes(self) -> int:
        return (self.codes.numel() * self.bits + 7) // 8


class KvCacheQuantizer:
    """KvCacheQuantizer, kv_cache.rs:125-283."""

    def __init__(self, config: KvCacheConfig):
        self.config = config

    def quantize(self, tensor: torch.Tensor, n_tokens: int, head_dim: int) -> QuantizedKvCache:
        """kv_cache.rs:146-221; bf16 input is quantized from its exact f32 values."""
        if tensor.numel() == 0 or n_tokens == 0 or head_dim == 0:
            raise L.EmptyInput(L.ERR_EMPTY_INPUT, "KvCacheQuantizer::quantize")
        if tensor.numel() != n_tokens * head_dim:
            raise L.DimensionMismatch(L.ERR_DIMENSION_MISMATCH, f"expected {n_tokens * head_dim}, got {tensor.numel()}")
        bf16 = tensor.dtype == torch.bfloat16
        x, was_host = _dev(tensor.reshape(-1), torch.bfloat16 if bf16 else torch.float32)
        groups = n_tokens if self.config.axis == KvAxis.PerToken else head_dim
        codes = torch.empty(n_tokens * head_dim, dtype=torch.uint8, device=x.device)
        scales = torch.empty(groups, dtype=torch.float32, device=x.device)
        zps = torch.empty(groups, dtype=torch.float32, device=x.device)
        default_handle().call("b2q_kv_cache_quantize_bf16" if bf16 else "b2q_kv_cache_quantize_f32", ptr(x), n_tokens, head_dim,
                              self.config.bits, self.config.axis.value, ptr(codes), ptr(scales), ptr(zps))
        return QuantizedKvCache(_back(codes, was_host), _back(scales, was_host), _back(zps, was_host), n_tokens, head_dim,
                                self.config.bits, self.config.axis)

    @staticmethod
    def dequantize(cache: QuantizedKvCache, out_dtype=torch.float32) -> torch.Tensor:
        """kv_cache.rs:224-238"""
        codes, was_host = _dev(cache.codes.reshape(-1), torch.uint8)
        sc, _ = _dev(cache.scales, torch.float32)
        zp, _ = _dev(cache.zero_points, torch.float32)
        out = torch.empty(cache.n_tokens * cache.head_dim, dtype=out_dtype, device=codes.device)
        name = "b2q_kv_cache_dequantize_bf16" if out_dtype == torch.bfloat16 else "b2q_kv_cache_dequantize_f32"
        default_handle().call(name, ptr(codes), cache.n_tokens, cache.head_dim, cache.axis.value, ptr(sc), ptr(zp), ptr(out))
        return _back(out, was_host)

    def append_token(self, cache: QuantizedKvCache, row: torch.Tensor) -> None:
        """kv_cache.rs:254-282: the new row gets a group of its own; the cache grows by one token."""
        if cache.axis != KvAxis.PerToken:
            raise L.InvalidConfig(L.ERR_INVALID_CONFIG, "append_token requires a PerToken cache")
        if row.numel() != cache.head_dim:
            raise L.DimensionMismatch(L.ERR_DIMENSION_MISMATCH, f"expected {cache.head_dim}, got {row.numel()}")
        one = KvCacheQuantizer(KvCacheConfig(cache.bits, KvAxis.PerToken)).quantize(row.to(cache.codes.device), 1, cache.head_dim)
        cache.codes = torch.cat([cache.codes, one.codes.to(cache.codes.device)])
        cache.scales = torch.cat([cache.scales, one.scales.to(cache.scales.device)])
        cache.zero_points = torch.cat([cache.zero_points, one.zero_points.to(cache.zero_points.device)])
        cache.n_tokens += 1


# ---- oxicuda-infer: crates/oxicuda-infer/src/cache/kv_quant.rs ----
@dataclass(frozen=True)
class KvQuantConfig:
    """kv_quant.rs:36-77"""
    bits: int
    symmetric: bool

    @staticmethod
    def new(bits: int, symmetric: bool) -> "KvQuantConfig":
        if bits not in (4, 8):
            raise L.InvalidConfig(L.ERR_INVALID_CONFIG, "KV quant bits must be 4 or 8")
        return KvQuantConfig(bits, symmetric)

    @staticmethod
    def int8() -> "KvQuantConfig":
        return KvQuantConfig(8, False)

    def q_range(self):
        if self.symmetric:
            half = 1 << (self.bits - 1)
            return (-(half - 1), half - 1)
        return (0, (1 << self.bits) - 1)


@dataclass
class QuantizedTokens:
    """A batch of QuantizedToken (kv_quant.rs:82-101): `codes` [n_tokens, d] int8 (symmetric) or uint8, one scale and
    zero point per token."""
    codes: torch.Tensor
    scale: torch.Tensor
    zero_point: torch.Tensor
    symmetric: bool

    def dequantize(self, out_dtype=torch.float32) -> torch.Tensor:
        n, d = self.codes.shape
        codes, was_host = _dev(self.codes.reshape(-1).view(torch.uint8), torch.uint8)
        sc, _ = _dev(self.scale, torch.float32)
        zp, _ = _dev(self.zero_point, torch.float32)
        out = torch.empty(n * d, dtype=out_dtype, device=codes.device)
        name = "b2q_kv_dequantize_tokens_bf16" if out_dtype == torch.bfloat16 else "b2q_kv_dequantize_tokens_f32"
        default_handle().call(name, ptr(codes), n, d, int(self.symmetric), ptr(sc), ptr(zp), ptr(out))
        return _back(out, was_host).view(n, d)


def quantize_tokens(x: torch.Tensor, config: KvQuantConfig) -> QuantizedTokens:
    """quantize_token (kv_quant.rs:112-154) for every row of x [n_tokens, d]."""
    if x.numel() == 0:
        raise L.InvalidConfig(L.ERR_INVALID_CONFIG, "quantize_token: empty vector")
    n, d = x.shape
    bf16 = x.dtype == torch.bfloat16
    xd, was_host = _dev(x.reshape(-1), torch.bfloat16 if bf16 else torch.float32)
    codes = torch.empty(n * d, dtype=torch.uint8, device=xd.device)
    scales = torch.empty(n, dtype=torch.float32, device=xd.device)
    zps = torch.empty(n, dtype=torch.float32, device=xd.device)
    default_handle().call("b2q_kv_quantize_tokens_bf16" if bf16 else "b2q_kv_quantize_tokens_f32", ptr(xd), n, d, config.bits,
                          int(config.symmetric), ptr(codes), ptr(scales), ptr(zps))
    codes = codes.view(torch.int8) if config.symmetric else codes
    return QuantizedTokens(_back(codes, was_host).view(n, d), _back(scales, was_host), _back(zps, was_host), config.symmetric)


@dataclass
class QuantizedToken:
    """kv_quant.rs:82-101 (codes as a list of ints, like the reference's Vec<i32>)."""
    codes: list
    scale: float
    zero_point: float
    _batch: QuantizedTokens = None

    def dequantize(self) -> list:
        return self._batch.dequantize()[0].tolist()


def quantize_token(x, config: KvQuantConfig) -> QuantizedToken:
    """kv_quant.rs:112-154 for one vector (a list or a 1-D tensor)."""
    t = torch.as_tensor(x, dtype=torch.float32).reshape(1, -1)
    b = quantize_tokens(t, config)
    return QuantizedToken([int(c) for c in b.codes[0].tolist()], float(b.scale[0]), float(b.zero_point[0]), b)


def quantize_dequantize_token(x, config: KvQuantConfig) -> list:
    """kv_quant.rs:161-163"""
    return quantize_token(x, config).dequantize()


def quantization_mse(x, config: KvQuantConfig) -> float:
    """kv_quant.rs:169-182 (f64 accumulation of f32 differences)."""
    t = torch.as_tensor(x, dtype=torch.float32).reshape(-1)
    recon = torch.tensor(quantize_dequantize_token(t, config), dtype=torch.float32)
    return float(((t - recon).to(torch.float64) ** 2).sum() / t.numel())


# ---- RMSNorm -> FP8 ----
def rms_norm_quantize_fp8(x: torch.Tensor, gamma: torch.Tensor, eps: float, residual: torch.Tensor = None, fmt: int = L.FP8_E4M3,
                          rounding: int = L.ROUND_RNE, want_y: bool = False):
    """rms_norm / fused_add_rms_norm (crates/oxicuda-dnn/src/norm/rms_norm.rs:49-110, :115-170) followed by the per-token FP8
    quantizer, in one kernel.  x [rows, cols] bf16 on the device; `residual` (bf16, same shape) is updated in place with
    residual + x and normalised instead of x.  Returns (codes u8 [rows, cols], scales f32 [rows]) and y (bf16) when asked."""
    if not x.is_cuda or x.dtype != torch.bfloat16 or gamma.dtype != torch.bfloat16:
        raise L.InvalidArgument(L.ERR_INVALID_ARGUMENT, "rms_norm_quantize_fp8 takes bf16 CUDA tensors")
    rows, cols = x.shape
    if gamma.numel() != cols:
        raise L.DimensionMismatch(L.ERR_DIMENSION_MISMATCH, f"expected {cols}, got {gamma.numel()}")
    if residual is not None and (residual.shape != x.shape or residual.dtype != torch.bfloat16 or not residual.is_contiguous()):
        raise L.InvalidArgument(L.ERR_INVALID_ARGUMENT, "residual must be a contiguous bf16 tensor of x's shape")
    x = x.contiguous()
    codes = torch.empty(rows, cols, dtype=torch.uint8, device=x.device)
    scales = torch.empty(rows, dtype=torch.float32, device=x.device)
    y = torch.empty_like(x) if want_y else None
    default_handle().call("b2q_rms_norm_quantize_fp8_bf16", ptr(x), ptr(residual), ptr(gamma.contiguous()), rows, cols, float(eps), fmt,
                          rounding, ptr(scales), ptr(codes), ptr(y))
    return (codes, scales, y) if want_y else (codes, scales)
