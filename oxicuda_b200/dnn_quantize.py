"""Host-side mirror of oxicuda-dnn's quantize entry points (crates/oxicuda-dnn/src/quantize/{fp8_quantize,int8_quantize,
block_scale}.rs): same names, argument meaning and error behaviour; the arithmetic runs in CUDA kernels through the C
ABI.  The GPU functions of the reference write into caller-provided device buffers and keep the scale on the device;
here they return new tensors (on the device for device input, on the host for host input).
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from . import _lib as L
from ._lib import default_handle, ptr
from .quant import _back, _dev


def quantize_to_fp8(input: torch.Tensor):
    """fp8_quantize.rs:45-122 -> (E4M3 bytes u8 [n], scale f32 [1]); scale = max(absmax / 448, 1e-12)."""
    x, was_host = _dev(input.reshape(-1), torch.float32)
    codes = torch.empty(x.numel(), dtype=torch.uint8, device=x.device)
    scale = torch.zeros(1, dtype=torch.float32, device=x.device)
    default_handle().call("b2q_dnn_quantize_to_fp8_f32", ptr(x), x.numel(), ptr(codes), ptr(scale))
    return _back(codes, was_host), _back(scale, was_host)


def dequantize_from_fp8(input: torch.Tensor, scale: torch.Tensor, n: int = None) -> torch.Tensor:
    """fp8_quantize.rs:125-170: out[i] = e4m3(input[i]) * scale[0] for the first n elements."""
    n = input.numel() if n is None else n
    if input.numel() < n:
        raise L.BufferTooSmall(L.ERR_BUFFER_TOO_SMALL, f"expected {n}, actual {input.numel()}")
    if scale.numel() == 0:
        raise L.BufferTooSmall(L.ERR_BUFFER_TOO_SMALL, "expected 1, actual 0")
    c, was_host = _dev(input.reshape(-1), torch.uint8)
    s, _ = _dev(scale.reshape(-1), torch.float32)
    out = torch.empty(n, dtype=torch.float32, device=c.device)
    default_handle().call("b2q_dnn_dequantize_from_fp8_f32", ptr(c), ptr(s), n, ptr(out))
    return _back(out, was_host)


def quantize_to_int8(input: torch.Tensor):
    """int8_quantize.rs:31-102 -> (int8 [n], scale f32 [1]); scale = max(absmax / 127, 1e-12), ties to even."""
    x, was_host = _dev(input.reshape(-1), torch.float32)
    q = torch.empty(x.numel(), dtype=torch.int8, device=x.device)
    scale = torch.zeros(1, dtype=torch.float32, device=x.device)
    default_handle().call("b2q_dnn_quantize_to_int8_f32", ptr(x), x.numel(), ptr(q), ptr(scale))
    return _back(q, was_host), _back(scale, was_host)


def dequantize_from_int8(input: torch.Tensor, scale: torch.Tensor, n: int = None) -> torch.Tensor:
    """int8_quantize.rs:105-160: out[i] = input[i] * scale[0]."""
    n = input.numel() if n is None else n
    if input.numel() < n:
        raise L.BufferTooSmall(L.ERR_BUFFER_TOO_SMALL, f"expected {n}, actual {input.numel()}")
    if scale.numel() == 0:
        raise L.BufferTooSmall(L.ERR_BUFFER_TOO_SMALL, "expected 1, actual 0")
    q, was_host = _dev(input.reshape(-1), torch.int8)
    s, _ = _dev(scale.reshape(-1), torch.float32)
    out = torch.empty(n, dtype=torch.float32, device=q.device)
    default_handle().call("b2q_dnn_dequantize_from_int8_f32", ptr(q), ptr(s), n, ptr(out))
    return _back(out, was_host)


def quantize_block_scaled(input: torch.Tensor, block_size: int):
    """block_scale.rs:51-150 -> (bytes u8 [n] = rne(clamp(x / scale, +-6)) + 6, scales f32 [ceil(n / block_size)])."""
    n = input.numel()
    if n == 0:
        return torch.empty(0, dtype=torch.uint8), torch.empty(0)
    if block_size == 0 or block_size & (block_size - 1):
        raise L.InvalidArgument(L.ERR_INVALID_ARGUMENT, f"block_size must be a non-zero power of 2, got {block_size}")
    if block_size < 16:
        raise L.InvalidArgument(L.ERR_INVALID_ARGUMENT, f"block_size must be >= 16, got {block_size}")
    x, was_host = _dev(input.reshape(-1), torch.float32)
    out = torch.empty(n, dtype=torch.uint8, device=x.device)
    scales = torch.empty(-(-n // block_size), dtype=torch.float32, device=x.device)
    default_handle().call("b2q_dnn_quantize_block_scaled_f32", ptr(x), n, block_size, ptr(out), ptr(scales))
    return _back(out, was_host), _back(scales, was_host)


@dataclass
class BlockQuantizedInt8:
    """int8_quantize.rs:406-490"""
    data: torch.Tensor
    scales: torch.Tensor
    block_size: int
    orig_len: int

    @staticmethod
    def quantize(input: torch.Tensor, block_size: int) -> "BlockQuantizedInt8":
        assert block_size > 0, "block_size must be > 0"
        x, was_host = _dev(input.reshape(-1), torch.float32)
        n = x.numel()
        q = torch.empty(n, dtype=torch.int8, device=x.device)
        scales = torch.empty(-(-n // block_size), dtype=torch.float32, device=x.device)
        default_handle().call("b2q_block_int8_quantize_f32", ptr(x), n, block_size, ptr(q), ptr(scales))
        return BlockQuantizedInt8(_back(q, was_host), _back(scales, was_host), block_size, n)

    def dequantize(self) -> torch.Tensor:
        q, was_host = _dev(self.data.reshape(-1), torch.int8)
        s, _ = _dev(self.scales, torch.float32)
        n = min(self.orig_len, q.numel(), s.numel() * self.block_size)
        out = torch.empty(n, dtype=torch.float32, device=q.device)
        default_handle().call("b2q_block_int8_dequantize_f32", ptr(q), ptr(s), n, self.block_size, ptr(out))
        return _back(out, was_host)

    def compression_ratio(self) -> float:
        quantized = self.data.numel() + self.scales.numel() * 4
        return 1.0 if quantized == 0 else self.orig_len * 4 / quantized

    def num_blocks(self) -> int:
        return self.scales.numel()


class Fp4BlockQuantizer:
    """block_scale.rs:394-454"""
    MAX_VALUE = 6.0
    REQUIRED_BLOCK_SIZE = 32

    def __init__(self, block_size: int):
        if block_size != self.REQUIRED_BLOCK_SIZE:
            raise L.InvalidArgument(L.ERR_INVALID_ARGUMENT, f"NVFP4/OCP MXFP4 block size must be 32, got {block_size}")
        self.block_size = block_size

    @staticmethod
    def new(block_size: int) -> "Fp4BlockQuantizer":
        return Fp4BlockQuantizer(block_size)

    def compute_scales(self, input: torch.Tensor) -> torch.Tensor:
        """compute_scale (block_scale.rs:437-444) for every block of the tensor."""
        x, was_host = _dev(input.reshape(-1), torch.float32)
        scales = torch.empty(self.num_scales(x.numel()), dtype=torch.float32, device=x.device)
        default_handle().call("b2q_block_absmax_scale_f32", ptr(x), x.numel(), self.block_size, self.MAX_VALUE, ptr(scales))
        return _back(scales, was_host)

    def compute_scale(self, block) -> float:
        return float(self.compute_scales(torch.as_tensor(block, dtype=torch.float32))[0])

    def num_scales(self, n: int) -> int:
        return -(-n // self.block_size)
