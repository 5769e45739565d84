"""Host-side mirror of the oxicuda-quant entry points on this path.

Same item names, argument meaning and error behaviour as the reference
(`crates/oxicuda-quant/src/scheme/{minmax,fp8,nf4,llm_int8}.rs`), but every call
runs a CUDA kernel through the C ABI on tensors that live in HBM.  A tensor given
on the host is uploaded and the result comes back on the host, which is how the
reference's `&[f32] -> Vec<_>` signatures behave; a CUDA tensor stays on the device.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from enum import Enum

import torch

from . import _lib as L
from ._lib import default_handle, ptr


def _dev(t: torch.Tensor, dtype=None):
    """(device tensor, was_host) — uploads host tensors to the current CUDA device."""
    was_host = not t.is_cuda
    if dtype is not None and t.dtype != dtype:
        t = t.to(dtype)
    t = t.contiguous()
    if was_host:
        t = t.cuda(non_blocking=False)
    return t, was_host


def _back(t: torch.Tensor, was_host: bool):
    return t.cpu() if was_host else t


class QuantScheme(Enum):
    """crates/oxicuda-quant/src/scheme/minmax.rs:26-32"""
    Symmetric = 0
    Asymmetric = 1


@dataclass
class QuantGranularity:
    """crates/oxicuda-quant/src/scheme/minmax.rs:35-44.  kind: 'PerTensor' | 'PerChannel' | 'PerGroup'."""
    kind: str = "PerTensor"
    channel_axis: int = 0
    group_size: int = 0

    @staticmethod
    def PerTensor():
        return QuantGranularity("PerTensor")

    @staticmethod
    def PerChannel(channel_axis: int = 0):
        return QuantGranularity("PerChannel", channel_axis=channel_axis)

    @staticmethod
    def PerGroup(group_size: int):
        return QuantGranularity("PerGroup", group_size=group_size)


@dataclass
class QuantParams:
    """crates/oxicuda-quant/src/scheme/minmax.rs:48-80"""
    scales: torch.Tensor        # f32
    zero_points: torch.Tensor   # i32
    bits: int
    scheme: QuantScheme

    def q_max(self) -> float:
        return float((1 << (self.bits - 1)) - 1) if self.scheme == QuantScheme.Symmetric else float((1 << self.bits) - 1)

    def q_min(self) -> float:
        return -float(1 << (self.bits - 1)) if self.scheme == QuantScheme.Symmetric else 0.0


class MinMaxQuantizer:
    """MinMaxQuantizer, crates/oxicuda-quant/src/scheme/minmax.rs:86-325."""

    def __init__(self, bits: int, scheme: QuantScheme, granularity: QuantGranularity):
        assert 0 < bits <= 16, "bits must be in [1, 16]"
        self.bits, self.scheme, self.granularity = bits, scheme, granularity

    @staticmethod
    def int8_symmetric():
        return MinMaxQuantizer(8, QuantScheme.Symmetric, QuantGranularity.PerTensor())

    @staticmethod
    def int4_per_group(group_size: int):
        return MinMaxQuantizer(4, QuantScheme.Symmetric, QuantGranularity.PerGroup(group_size))

    def _calibrate_rows(self, x: torch.Tensor, rows: int, cols: int, was_host: bool) -> QuantParams:
        h = default_handle()
        scales = torch.empty(rows, dtype=torch.float32, device=x.device)
        zps = torch.empty(rows, dtype=torch.int32, device=x.device)
        h.call("b2q_minmax_calibrate_f32", ptr(x), rows, cols, self.bits, self.scheme.value, ptr(scales), ptr(zps))
        h.check()   # InvalidScale is detected on the device
        return QuantParams(_back(scales, was_host), _back(zps, was_host), self.bits, self.scheme)

    def calibrate(self, tensor: torch.Tensor) -> QuantParams:
        """minmax.rs:134-171 — PerChannel degrades to per-tensor here exactly as in the reference (:140-145)."""
        if tensor.numel() == 0:
            raise L.EmptyInput(L.ERR_EMPTY_INPUT, "MinMaxQuantizer::calibrate")
        x, was_host = _dev(tensor.reshape(-1), torch.float32)
        n = x.numel()
        if self.granularity.kind == "PerGroup":
            g = self.granularity.group_size
            if n % g != 0:
                raise L.GroupSizeMismatch(L.ERR_GROUP_SIZE_MISMATCH, f"len {n} not divisible by group {g}")
            return self._calibrate_rows(x, n // g, g, was_host)
        return self._calibrate_rows(x, 1, n, was_host)

    def calibrate_2d(self, tensor: torch.Tensor, rows: int, cols: int) -> QuantParams:
        """minmax.rs:179-207 — one (scale, zp) per row."""
        if rows == 0:
            raise L.EmptyInput(L.ERR_EMPTY_INPUT, "calibrate_2d: rows == 0")
        if cols == 0:
            raise L.DimensionMismatch(L.ERR_DIMENSION_MISMATCH, "expected 1, got 0")
        x, was_host = _dev(tensor.reshape(-1), torch.float32)
        return self._calibrate_rows(x, rows, cols, was_host)

    def _quantize_rows(self, tensor, params: QuantParams, rows: int, cols: int) -> torch.Tensor:
        x, was_host = _dev(tensor.reshape(-1), torch.float32)
        sc, _ = _dev(params.scales, torch.float32)
        zp, _ = _dev(params.zero_points, torch.int32)
        codes = torch.empty(x.numel(), dtype=torch.int32, device=x.device)
        default_handle().call("b2q_minmax_quantize_f32", ptr(x), rows, cols, ptr(sc), ptr(zp), self.bits,
                              self.scheme.value, ptr(codes))
        return _back(codes, was_host)

    def quantize(self, tensor: torch.Tensor, params: QuantParams) -> torch.Tensor:
        """minmax.rs:252-268 — uses scales[0] / zero_points[0] only."""
        scale = float(params.scales.reshape(-1)[0])
        if not (scale > 0.0) or scale != scale or scale == float("inf"):
            raise L.InvalidScale(L.ERR_INVALID_SCALE, f"scale {scale}")
        p0 = QuantParams(params.scales.reshape(-1)[:1], params.zero_points.reshape(-1)[:1], params.bits, params.scheme)
        return self._quantize_rows(tensor, p0, 1, tensor.numel())

    def quantize_grouped(self, tensor: torch.Tensor, params: QuantParams, group_size: int) -> torch.Tensor:
        """minmax.rs:275-299"""
        n = tensor.numel()
        if n % group_size != 0:
            raise L.GroupSizeMismatch(L.ERR_GROUP_SIZE_MISMATCH, f"len {n} not divisible by group {group_size}")
        return self._quantize_rows(tensor, params, n // group_size, group_size)

    def _dequantize_rows(self, codes, params: QuantParams, rows: int, cols: int) -> torch.Tensor:
        c, was_host = _dev(codes.reshape(-1), torch.int32)
        sc, _ = _dev(params.scales, torch.float32)
        zp, _ = _dev(params.zero_points, torch.int32)
        out = torch.empty(c.numel(), dtype=torch.float32, device=c.device)
        default_handle().call("b2q_minmax_dequantize_f32", ptr(c), rows, cols, ptr(sc), ptr(zp), ptr(out))
        return _back(out, was_host)

    def dequantize(self, codes: torch.Tensor, params: QuantParams) -> torch.Tensor:
        """minmax.rs:302-306"""
        p0 = QuantParams(params.scales.reshape(-1)[:1], params.zero_points.reshape(-1)[:1], params.bits, params.scheme)
        return self._dequantize_rows(codes, p0, 1, codes.numel())

    def dequantize_grouped(self, codes: torch.Tensor, params: QuantParams, group_size: int) -> torch.Tensor:
        """minmax.rs:309-324"""
        return self._dequantize_rows(codes, params, codes.numel() // group_size, group_size)


class Fp8Format(Enum):
    """crates/oxicuda-quant/src/scheme/fp8.rs:32-37"""
    E4M3 = 0
    E5M2 = 1

    def max_val(self) -> float:
        return 448.0 if self is Fp8Format.E4M3 else 57344.0


class Fp8Codec:
    """Fp8Codec, crates/oxicuda-quant/src/scheme/fp8.rs:84-262.

    `rounding="ref"` reproduces the reference codec bit for bit (truncation); `"rne"` is the
    hardware round-to-nearest-even conversion the throughput paths use."""

    def __init__(self, format: Fp8Format, saturate: bool = True, rounding: str = "ref"):
        self.format, self.saturate = format, saturate
        self.rounding = L.ROUND_REF if rounding == "ref" else L.ROUND_RNE

    @staticmethod
    def e4m3(rounding: str = "ref"):
        return Fp8Codec(Fp8Format.E4M3, True, rounding)

    @staticmethod
    def e5m2(rounding: str = "ref"):
        return Fp8Codec(Fp8Format.E5M2, True, rounding)

    def encode(self, data: torch.Tensor) -> torch.Tensor:
        """fp8.rs:135-137; raises NonFiniteFp8 for NaN/Inf input (:116-118)."""
        x, was_host = _dev(data.reshape(-1), torch.float32)
        codes = torch.empty(x.numel(), dtype=torch.uint8, device=x.device)
        h = default_handle()
        h.call("b2q_fp8_encode_f32", ptr(x), x.numel(), self.format.value, self.rounding, ptr(codes))
        h.check()
        return _back(codes, was_host)

    def decode(self, data: torch.Tensor) -> torch.Tensor:
        """fp8.rs:140-142"""
        c, was_host = _dev(data.reshape(-1), torch.uint8)
        out = torch.empty(c.numel(), dtype=torch.float32, device=c.device)
        default_handle().call("b2q_fp8_decode_f32", ptr(c), c.numel(), self.format.value, self.rounding, ptr(out))
        return _back(out, was_host)

    def to_reference_decode_codes(self, codes: torch.Tensor) -> torch.Tensor:
        """Copy of `codes` whose IEEE values equal the reference decoder's reading of `codes`
        (fp8.rs:242-254 reads subnormal codes as 2^(1-bias)*(1+m/2^mb)); feed it to gemm_fp8 to reproduce
        the reference's decode -> f32 matmul composition on the tensor cores."""
        c, was_host = _dev(codes.reshape(-1), torch.uint8)
        c = c.clone()
        default_handle().call("b2q_fp8_remap_ref_subnormals", ptr(c), c.numel(), self.format.value)
        return _back(c, was_host).view(codes.shape)

    def quantization_mse(self, data: torch.Tensor) -> float:
        """fp8.rs:149-159"""
        dec = self.decode(self.encode(data))
        return float(((data.reshape(-1).to(dec.device, torch.float32) - dec) ** 2).sum() / data.numel())

    def quantize_rows(self, x: torch.Tensor, rows: int, cols: int):
        """Absmax-scaled quantization: scale = absmax/max_val per row (rows=1: per tensor).
        Returns (codes u8, scales f32).  Scale rule: crates/oxicuda-dnn/src/quantize/fp8_quantize.rs:28-34."""
        bf16 = x.dtype == torch.bfloat16
        xd, was_host = _dev(x.reshape(-1), torch.bfloat16 if bf16 else torch.float32)
        codes = torch.empty(rows * cols, dtype=torch.uint8, device=xd.device)
        scales = torch.empty(rows, dtype=torch.float32, device=xd.device)
        h = default_handle()
        h.call("b2q_fp8_quantize_rows_bf16" if bf16 else "b2q_fp8_quantize_rows_f32", ptr(xd), rows, cols,
               self.format.value, self.rounding, ptr(scales), ptr(codes))
        return _back(codes, was_host), _back(scales, was_host)


class Nf4Quantizer:
    """Nf4Quantizer, crates/oxicuda-quant/src/scheme/nf4.rs:59-175."""

    def __init__(self, block_size: int = 64):
        assert block_size > 0, "block_size must be > 0"
        self.block_size = block_size

    def encode(self, tensor: torch.Tensor):
        if tensor.numel() == 0:
            raise L.EmptyInput(L.ERR_EMPTY_INPUT, "Nf4Quantizer::encode")
        x, was_host = _dev(tensor.reshape(-1), torch.float32)
        n = x.numel()
        if n % self.block_size != 0:
            raise L.GroupSizeMismatch(L.ERR_GROUP_SIZE_MISMATCH, f"len {n} not divisible by group {self.block_size}")
        packed = torch.empty(n // 2, dtype=torch.uint8, device=x.device)
        absmaxs = torch.empty(n // self.block_size, dtype=torch.float32, device=x.device)
        default_handle().call("b2q_nf4_encode_f32", ptr(x), n, self.block_size, ptr(packed), ptr(absmaxs))
        return _back(packed, was_host), _back(absmaxs, was_host)

    def decode(self, packed: torch.Tensor, absmaxs: torch.Tensor) -> torch.Tensor:
        n_floats = packed.numel() * 2
        expected = n_floats // self.block_size
        if absmaxs.numel() != expected:
            raise L.DimensionMismatch(L.ERR_DIMENSION_MISMATCH, f"expected {expected}, got {absmaxs.numel()}")
        p, was_host = _dev(packed.reshape(-1), torch.uint8)
        a, _ = _dev(absmaxs.reshape(-1), torch.float32)
        out = torch.empty(n_floats, dtype=torch.float32, device=p.device)
        default_handle().call("b2q_nf4_decode_f32", ptr(p), p.numel(), self.block_size, ptr(a), ptr(out))
        return _back(out, was_host)


@dataclass
class LlmInt8Config:
    """crates/oxicuda-quant/src/scheme/llm_int8.rs:45-79"""
    threshold: float = 6.0
    row_wise_activations: bool = True

    @staticmethod
    def new(threshold: float, row_wise_activations: bool):
        if not (threshold == threshold and abs(threshold) != float("inf") and threshold > 0.0):
            raise L.InvalidConfig(L.ERR_INVALID_CONFIG, f"LLM.int8 threshold must be finite and positive, got {threshold}")
        return LlmInt8Config(threshold, row_wise_activations)


@dataclass
class LlmInt8Output:
    """crates/oxicuda-quant/src/scheme/llm_int8.rs:83-92 (+ the integer intermediates, for parity checks)."""
    output: torch.Tensor
    outlier_columns: list
    outlier_fraction: float
    w_q: torch.Tensor = None
    s_w: torch.Tensor = None
    x_q: torch.Tensor = None
    s_x: torch.Tensor = None
    acc: torch.Tensor = None


class LlmInt8Quantizer:
    """LlmInt8Quantizer, crates/oxicuda-quant/src/scheme/llm_int8.rs:99-311."""

    def __init__(self, config: LlmInt8Config = None):
        self.config = config or LlmInt8Config()

    def matmul(self, x: torch.Tensor, w: torch.Tensor, n_samples: int, n_rows: int, n_cols: int,
               dump: bool = False) -> LlmInt8Output:
        """llm_int8.rs:175-288: Y = X . W^T with vector-wise INT8 and fp32 outlier columns."""
        if x.numel() == 0 or w.numel() == 0:
            raise L.EmptyInput(L.ERR_EMPTY_INPUT, "LlmInt8::matmul")
        if x.numel() != n_samples * n_cols:
            raise L.DimensionMismatch(L.ERR_DIMENSION_MISMATCH, f"expected {n_samples * n_cols}, got {x.numel()}")
        if w.numel() != n_rows * n_cols:
            raise L.DimensionMismatch(L.ERR_DIMENSION_MISMATCH, f"expected {n_rows * n_cols}, got {w.numel()}")
        xd, was_host = _dev(x.reshape(-1), torch.float32)
        wd, _ = _dev(w.reshape(-1), torch.float32)
        dev = xd.device
        out = torch.empty(n_samples * n_rows, dtype=torch.float32, device=dev)
        n_out = torch.zeros(1, dtype=torch.int32, device=dev)
        wq = sw = xq = sx = acc = None
        if dump:
            wq = torch.empty(n_rows * n_cols, dtype=torch.int8, device=dev)
            sw = torch.empty(n_rows, dtype=torch.float32, device=dev)
            xq = torch.empty(n_samples * n_cols, dtype=torch.int8, device=dev)
            sx = torch.empty(n_samples, dtype=torch.float32, device=dev)
            acc = torch.empty(n_samples * n_rows, dtype=torch.int32, device=dev)
        default_handle().call("b2q_llm_int8_linear_f32", ptr(xd), ptr(wd), n_samples, n_rows, n_cols,
                              C.c_float(self.config.threshold), int(self.config.row_wise_activations), ptr(out),
                              ptr(wq), ptr(sw), ptr(xq), ptr(sx), ptr(acc), ptr(n_out))
        cols = []
        if int(n_out.item()) > 0:
            col_max = xd.view(n_samples, n_cols).abs().amax(dim=0)
            cols = torch.nonzero(col_max >= self.config.threshold).flatten().tolist()
        b = lambda t: None if t is None else _back(t, was_host)
        return LlmInt8Output(_back(out, was_host), cols, len(cols) / n_cols, b(wq), b(sw), b(xq), b(sx), b(acc))


def fake_quant_inplace(x: torch.Tensor, scale: float, zero_point: float, qmin: float, qmax: float):
    """fake_quant_inplace kernel, crates/oxicuda-quant/src/ptx_kernels.rs:55-121."""
    assert x.is_cuda and x.dtype == torch.float32 and x.is_contiguous()
    default_handle().call("b2q_fake_quant_inplace_f32", ptr(x), x.numel(), C.c_float(scale), C.c_float(zero_point),
                          C.c_float(qmin), C.c_float(qmax))
    return x


def int8_quant(x: torch.Tensor, scale: float) -> torch.Tensor:
    """int8_quant kernel, crates/oxicuda-quant/src/ptx_kernels.rs:129-191."""
    xd, was_host = _dev(x.reshape(-1), torch.float32)
    out = torch.empty(xd.numel(), dtype=torch.int8, device=xd.device)
    default_handle().call("b2q_int8_quant_f32", ptr(xd), xd.numel(), C.c_float(scale), ptr(out))
    return _back(out, was_host)


def int8_dequant(q: torch.Tensor, scale: float) -> torch.Tensor:
    """int8_dequant kernel, crates/oxicuda-quant/src/ptx_kernels.rs:199-252."""
    qd, was_host = _dev(q.reshape(-1), torch.int8)
    out = torch.empty(qd.numel(), dtype=torch.float32, device=qd.device)
    default_handle().call("b2q_int8_dequant_f32", ptr(qd), qd.numel(), C.c_float(scale), ptr(out))
    return _back(out, was_host)
