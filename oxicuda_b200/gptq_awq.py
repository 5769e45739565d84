"""Host-side mirror of oxicuda-dnn's GPTQ / AWQ weight-only quantization (crates/oxicuda-dnn/src/quantize/gptq_awq.rs):
same items, field names, validation messages and error kinds.  Where the reference's `WeightQuantPlan` returns the PTX
text of a kernel (`generate_*_ptx`), the plan here has a method of the kernel's role that runs the CUDA kernel through
the C ABI on device tensors: `gptq_quantize`, `gptq_dequantize`, `awq_scale_search`, `awq_quantize`,
`fused_dequant_gemv`.  Buffers follow `QuantizedWeight`: codes packed 32 / bits to a u32 over the flat row-major matrix,
scales and zero points f32 [rows x cols / group_size].
"""
from __future__ import annotations

from dataclasses import dataclass, field
from enum import Enum
from typing import Optional, Union

import torch

from . import _lib as L
from ._lib import default_handle, ptr
from .quant import _back, _dev

QUANT_BLOCK_SIZE = 256          # gptq_awq.rs:26
MIN_DAMP = 1e-6                 # gptq_awq.rs:29


def _invalid(msg: str) -> L.InvalidArgument:
    return L.InvalidArgument(L.ERR_INVALID_ARGUMENT, msg)


class QuantMethodTag(Enum):
    """gptq_awq.rs:46-52"""
    Gptq = 0
    Awq = 1


@dataclass
class GptqConfig:
    """gptq_awq.rs:64-94 (defaults of `impl Default`)."""
    bits: int = 4
    group_size: int = 128
    block_size: int = 128
    damp_percent: float = 0.01
    symmetric: bool = True
    act_order: bool = False
    true_sequential: bool = True

    def validate(self) -> None:
        """gptq_awq.rs:102-127"""
        if self.bits not in (2, 3, 4, 8):
            raise _invalid(f"GPTQ bits must be 2, 3, 4, or 8; got {self.bits}")
        if self.group_size == 0:
            raise _invalid("GPTQ group_size must be non-zero")
        if self.block_size == 0:
            raise _invalid("GPTQ block_size must be non-zero")
        if self.damp_percent < 0.0:
            raise _invalid(f"GPTQ damp_percent must be non-negative; got {self.damp_percent}")


@dataclass
class AwqConfig:
    """gptq_awq.rs:139-166"""
    bits: int = 4
    group_size: int = 128
    zero_point: bool = True
    search_alpha_min: float = 0.0
    search_alpha_max: float = 1.0
    search_steps: int = 20

    def validate(self) -> None:
        """gptq_awq.rs:174-199"""
        if self.bits not in (4, 8):
            raise _invalid(f"AWQ bits must be 4 or 8; got {self.bits}")
        if self.group_size == 0:
            raise _invalid("AWQ group_size must be non-zero")
        if self.search_alpha_min > self.search_alpha_max:
            raise _invalid(f"AWQ search_alpha_min ({self.search_alpha_min}) must be <= search_alpha_max ({self.search_alpha_max})")
        if self.search_steps == 0:
            raise _invalid("AWQ search_steps must be non-zero")


@dataclass
class WeightQuantMethod:
    """gptq_awq.rs:37-43: `WeightQuantMethod.Gptq(cfg)` / `WeightQuantMethod.Awq(cfg)`."""
    config: Union[GptqConfig, AwqConfig]

    @staticmethod
    def Gptq(config: GptqConfig) -> "WeightQuantMethod":
        return WeightQuantMethod(config)

    @staticmethod
    def Awq(config: AwqConfig) -> "WeightQuantMethod":
        return WeightQuantMethod(config)

    @property
    def is_gptq(self) -> bool:
        return isinstance(self.config, GptqConfig)


@dataclass
class QuantizedWeight:
    """gptq_awq.rs:209-232"""
    method: QuantMethodTag
    bits: int
    group_size: int
    rows: int
    cols: int
    packed_weight_elements: int
    scale_elements: int
    zero_point_elements: int
    has_zero_point: bool


class WeightQuantPlan:
    """gptq_awq.rs:240-1085"""

    def __init__(self, method: WeightQuantMethod, rows: int, cols: int):
        """WeightQuantPlan::new (:254-283)"""
        if rows == 0 or cols == 0:
            raise L.InvalidDimension(L.ERR_INVALID_DIMENSION, "weight dimensions must be non-zero")
        method.config.validate()
        group_size = method.config.group_size
        if cols % group_size != 0:
            raise _invalid(f"cols ({cols}) must be divisible by group_size ({group_size})")
        self.method, self.weight_rows, self.weight_cols = method, rows, cols

    @classmethod
    def new(cls, method: WeightQuantMethod, rows: int, cols: int) -> "WeightQuantPlan":
        return cls(method, rows, cols)

    def _bits(self) -> int:
        return self.method.config.bits

    def _group_size(self) -> int:
        return self.method.config.group_size

    def elements_per_u32(self) -> int:
        return 32 // self._bits()

    def _groups_per_row(self) -> int:
        return self.weight_cols // self._group_size()

    def quantized_weight_info(self) -> QuantizedWeight:
        """:996-1027"""
        cfg = self.method.config
        total, epu = self.weight_rows * self.weight_cols, self.elements_per_u32()
        scale_elements = self.weight_rows * self._groups_per_row()
        has_zp = (not cfg.symmetric) if self.method.is_gptq else cfg.zero_point
        return QuantizedWeight(QuantMethodTag.Gptq if self.method.is_gptq else QuantMethodTag.Awq, cfg.bits, cfg.group_size, self.weight_rows,
                               self.weight_cols, -(-total // epu), scale_elements, scale_elements if has_zp else 0, has_zp)

    def workspace_bytes(self) -> int:
        """:1029-1052"""
        cfg = self.method.config
        if self.method.is_gptq:
            return self.weight_cols * 4 + (self.weight_cols * 4 if cfg.act_order else 0) + self.weight_rows * cfg.block_size * 4
        return self.weight_cols * 4 + self.weight_cols * 4 + cfg.search_steps * 4

    def shared_memory_bytes(self) -> int:
        """:1057-1066"""
        cfg = self.method.config
        return (cfg.block_size if self.method.is_gptq else cfg.group_size) * 4

    def launch_params(self):
        """:1071-1080: (grid, block) of the reference's launches (one thread per row for GPTQ, per element for AWQ)."""
        total = self.weight_rows if self.method.is_gptq else self.weight_rows * self.weight_cols
        return -(-total // QUANT_BLOCK_SIZE), QUANT_BLOCK_SIZE

    # ---- the kernels behind generate_*_ptx ----
    def _require(self, gptq: bool, what: str):
        if self.method.is_gptq != gptq:
            raise _invalid(f"{what} called on {'AWQ' if gptq else 'GPTQ'} plan")

    def gptq_quantize(self, weight: torch.Tensor, hessian_diag: torch.Tensor):
        """dnn_gptq_quantize_f32 (:329-499): weight [rows x cols] f32, hessian_diag [cols] f32 ->
        (packed u32 as int32 tensor, scales f32 [rows x groups])."""
        self._require(True, "generate_gptq_quantize_ptx")
        cfg, info = self.method.config, self.quantized_weight_info()
        w, was_host = _dev(weight.reshape(-1), torch.float32)
        hd, _ = _dev(hessian_diag.reshape(-1), torch.float32)
        if w.numel() != self.weight_rows * self.weight_cols or hd.numel() != self.weight_cols:
            raise L.DimensionMismatch(L.ERR_DIMENSION_MISMATCH, "gptq_quantize: weight / hessian_diag size")
        packed = torch.empty(info.packed_weight_elements, dtype=torch.int32, device=w.device)
        scales = torch.empty(info.scale_elements, dtype=torch.float32, device=w.device)
        default_handle().call("b2q_gptq_quantize_f32", ptr(w), ptr(hd), self.weight_rows, self.weight_cols, cfg.group_size, cfg.bits,
                              int(cfg.symmetric), ptr(packed), ptr(scales))
        return _back(packed, was_host), _back(scales, was_host)

    def gptq_dequantize(self, packed: torch.Tensor, scales: torch.Tensor, zeros: Optional[torch.Tensor] = None, out_dtype=torch.float32):
        """dnn_gptq_dequantize_f32 (:509-616) -> [rows x cols]; zero points are read when the plan is asymmetric."""
        self._require(True, "generate_gptq_dequantize_ptx")
        return _dequantize(self, packed, scales, None if self.method.config.symmetric else zeros, out_dtype)

    def awq_scale_search(self, act_stats: torch.Tensor) -> torch.Tensor:
        """dnn_awq_scale_search_f32 (:626-713): per-channel scale a * rsqrt(a), a = max(|act|, 1e-7)."""
        self._require(False, "generate_awq_scale_search_ptx")
        a, was_host = _dev(act_stats.reshape(-1), torch.float32)
        out = torch.empty_like(a)
        default_handle().call("b2q_awq_scale_search_f32", ptr(a), a.numel(), ptr(out))
        return _back(out, was_host)

    def awq_quantize(self, weight: torch.Tensor, channel_scales: torch.Tensor, group_scales: torch.Tensor):
        """dnn_awq_quantize_f32 (:723-857) -> (packed, zeros or None); group_scales [rows x groups] is an input."""
        self._require(False, "generate_awq_quantize_ptx")
        cfg, info = self.method.config, self.quantized_weight_info()
        w, was_host = _dev(weight.reshape(-1), torch.float32)
        cs, _ = _dev(channel_scales.reshape(-1), torch.float32)
        gs, _ = _dev(group_scales.reshape(-1), torch.float32)
        if w.numel() != self.weight_rows * self.weight_cols or cs.numel() != self.weight_cols or gs.numel() != info.scale_elements:
            raise L.DimensionMismatch(L.ERR_DIMENSION_MISMATCH, "awq_quantize: operand size")
        packed = torch.empty(info.packed_weight_elements, dtype=torch.int32, device=w.device)
        zeros = torch.empty(info.scale_elements, dtype=torch.float32, device=w.device) if cfg.zero_point else None
        default_handle().call("b2q_awq_quantize_f32", ptr(w), ptr(cs), ptr(gs), self.weight_rows, self.weight_cols, cfg.group_size, cfg.bits,
                              ptr(packed), ptr(zeros) if zeros is not None else None)
        return _back(packed, was_host), (None if zeros is None else _back(zeros, was_host))

    def dequantize(self, packed: torch.Tensor, scales: torch.Tensor, zeros: Optional[torch.Tensor] = None, out_dtype=torch.float32):
        """The dequantize kernel for either method ((q - zero) * scale when zeros is given)."""
        return _dequantize(self, packed, scales, zeros, out_dtype)

    def fused_dequant_gemv(self, packed: torch.Tensor, scales: torch.Tensor, x: torch.Tensor, zeros: Optional[torch.Tensor] = None,
                           split_k: int = 1) -> torch.Tensor:
        """dnn_fused_dequant_gemv_f32 (:867-986): y [rows] = dequant(W) x.  split_k = 1 keeps the reference's summation
        order (bit-exact); 0 lets the library split the columns over more threads; zeros is this library's extension."""
        cfg = self.method.config
        p, was_host = _dev(packed.reshape(-1), torch.int32)
        s, _ = _dev(scales.reshape(-1), torch.float32)
        xv, _ = _dev(x.reshape(-1), torch.float32)
        z = None if zeros is None else _dev(zeros.reshape(-1), torch.float32)[0]
        if xv.numel() != self.weight_cols or s.numel() != self.weight_rows * self._groups_per_row():
            raise L.DimensionMismatch(L.ERR_DIMENSION_MISMATCH, "fused_dequant_gemv: operand size")
        y = torch.empty(self.weight_rows, dtype=torch.float32, device=p.device)
        default_handle().call("b2q_fused_dequant_gemv_f32", ptr(p), ptr(s), ptr(z) if z is not None else None, ptr(xv), self.weight_rows,
                              self.weight_cols, cfg.group_size, cfg.bits, split_k, ptr(y))
        return _back(y, was_host)


def _dequantize(plan: WeightQuantPlan, packed, scales, zeros, out_dtype):
    cfg = plan.method.config
    p, was_host = _dev(packed.reshape(-1), torch.int32)
    s, _ = _dev(scales.reshape(-1), torch.float32)
    z = None if zeros is None else _dev(zeros.reshape(-1), torch.float32)[0]
    info = plan.quantized_weight_info()
    if p.numel() < info.packed_weight_elements or s.numel() < info.scale_elements:
        raise L.BufferTooSmall(L.ERR_BUFFER_TOO_SMALL, "dequantize: packed / scales shorter than QuantizedWeight says")
    assert out_dtype in (torch.float32, torch.bfloat16)
    out = torch.empty(plan.weight_rows, plan.weight_cols, dtype=out_dtype, device=p.device)
    default_handle().call("b2q_wq_dequantize", ptr(p), ptr(s), ptr(z) if z is not None else None, plan.weight_rows, plan.weight_cols,
                          cfg.group_size, cfg.bits, ptr(out), L.OUT_BF16 if out_dtype == torch.bfloat16 else L.OUT_F32)
    return _back(out, was_host)


@dataclass
class GptqState:
    """gptq_awq.rs:1090-1141"""
    rows: int
    cols: int
    group_size: int
    bits: int
    columns_processed: int = 0
    quantization_error: float = 0.0

    @staticmethod
    def new(rows: int, cols: int, config: GptqConfig) -> "GptqState":
        return GptqState(rows, cols, config.group_size, config.bits)

    def num_groups(self) -> int:
        return -(-self.cols // self.group_size)

    def num_column_blocks(self) -> int:
        return -(-self.cols // self.group_size)

    def elements_per_packed_word(self) -> int:
        return 32 // self.bits

    def is_complete(self) -> bool:
        return self.columns_processed >= self.cols


@dataclass
class AwqChannelScales:
    """gptq_awq.rs:1149-1197"""
    num_channels: int
    scales: list = field(default_factory=list)
    best_alpha: float = 0.5

    @staticmethod
    def new(num_channels: int) -> "AwqChannelScales":
        return AwqChannelScales(num_channels, [1.0] * num_channels, 0.5)

    def set_scale(self, channel: int, scale: float) -> None:
        if channel >= self.num_channels:
            raise _invalid(f"channel index {channel} out of range (num_channels = {self.num_channels})")
        self.scales[channel] = scale

    def apply_alpha(self, alpha: float) -> None:
        self.best_alpha = alpha
        self.scales = [float(torch.tensor(s, dtype=torch.float32).pow(alpha)) for s in self.scales]
