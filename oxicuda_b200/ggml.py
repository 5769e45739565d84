"""GGML block codecs and the GGUF v3 container: the on-disk weight formats that feed the quantized linear path.

Codecs (crates/oxicuda-quant/src/scheme/ggml.rs): GgmlType, quantize / dequantize for Q8_0, Q4_0, Q4_1 and Q4_K on the
GPU (b2q_ggml_quantize_f32, b2q_ggml_dequantize), bit-exact with the reference's arithmetic.  Blocks are packed
little-endian records in the field order of the reference's structs (see include/b2q.h).

Container (crates/oxicuda-quant/src/scheme/gguf.rs): read_gguf / write_gguf, GgufFile, GgufTensorInfo and the typed
metadata values: host-side parsing of a byte buffer (never panics on malformed input: InvalidConfig), the tensor-data
region kept verbatim.  `tensor_to_device` hands a stored tensor's records to the GPU dequantizer."""
from __future__ import annotations

import struct
from dataclasses import dataclass, field
from enum import Enum
from typing import List, Optional

import torch

from . import _lib as L
from ._lib import default_handle, ptr


class GgmlType(Enum):
    """GgmlType, ggml.rs:147-185 (the values are this library's codec ids, not GGUF's tensor-type tags)."""
    Q8_0 = 0
    Q4_0 = 1
    Q4_1 = 2
    Q4_K = 3

    def block_size(self) -> int:
        return 256 if self is GgmlType.Q4_K else 32

    def block_bytes(self) -> int:
        return {GgmlType.Q8_0: 34, GgmlType.Q4_0: 18, GgmlType.Q4_1: 20, GgmlType.Q4_K: 148}[self]

    def bits_per_weight(self) -> float:
        """ggml.rs:170-185: the reference counts 6 + 6 bits per Q4_K sub-block (its in-memory struct spends 8 + 8)."""
        return {GgmlType.Q8_0: (256.0 + 16.0) / 32.0, GgmlType.Q4_0: (128.0 + 16.0) / 32.0, GgmlType.Q4_1: (128.0 + 32.0) / 32.0,
                GgmlType.Q4_K: (1024.0 + 96.0 + 32.0) / 256.0}[self]


# tensor-type tags of the GGUF directory (ggml's table) for the codecs above
GGUF_TENSOR_TAGS = {2: GgmlType.Q4_0, 3: GgmlType.Q4_1, 8: GgmlType.Q8_0}


def quantize(weights: torch.Tensor, ty: GgmlType) -> torch.Tensor:
    """quantize_q8_0 / q4_0 / q4_1 / q4_k (ggml.rs:243-472): flat f32 weights on the GPU -> packed records (uint8)."""
    w = weights.reshape(-1).float().contiguous()
    n = w.numel()
    out = torch.empty(max(1, n // ty.block_size()) * ty.block_bytes(), dtype=torch.uint8, device=w.device)
    default_handle().call("b2q_ggml_quantize_f32", ty.value, ptr(w), n, ptr(out))
    return out[:(n // ty.block_size()) * ty.block_bytes()]


def dequantize(blocks: torch.Tensor, ty: GgmlType, out_dtype=torch.float32) -> torch.Tensor:
    """dequantize_* (ggml.rs:265-506): packed records -> flat f32 (or bf16) weights."""
    b = blocks.reshape(-1).contiguous()
    if b.numel() % ty.block_bytes() != 0:
        raise L.DimensionMismatch(L.ERR_DIMENSION_MISMATCH, f"{b.numel()} bytes are not whole {ty.name} records of {ty.block_bytes()} bytes")
    n = b.numel() // ty.block_bytes() * ty.block_size()
    out = torch.empty(n, dtype=out_dtype, device=b.device)
    default_handle().call("b2q_ggml_dequantize", ty.value, ptr(b), n, ptr(out), L.OUT_BF16 if out_dtype == torch.bfloat16 else L.OUT_F32)
    return out


def fake_quantize(weights: torch.Tensor, ty: GgmlType) -> torch.Tensor:
    """fake_quantize, ggml.rs:511-518."""
    return dequantize(quantize(weights, ty), ty)


# ---- GGUF v3 container: crates/oxicuda-quant/src/scheme/gguf.rs ----
GGUF_MAGIC = 0x46554747
GGUF_VERSION = 3
GGUF_DEFAULT_ALIGNMENT = 32
ALIGNMENT_KEY = "general.alignment"


class GgufValueType(Enum):
    """gguf.rs:84-152."""
    U8 = 0
    I8 = 1
    U16 = 2
    I16 = 3
    U32 = 4
    I32 = 5
    F32 = 6
    Bool = 7
    String = 8
    Array = 9
    U64 = 10
    I64 = 11
    F64 = 12

    @staticmethod
    def from_tag(tag: int) -> "GgufValueType":
        try:
            return GgufValueType(tag)
        except ValueError:
            raise L.InvalidConfig(L.ERR_INVALID_CONFIG, f"unknown GGUF value type tag {tag}") from None


_SCALAR_FMT = {GgufValueType.U8: "<B", GgufValueType.I8: "<b", GgufValueType.U16: "<H", GgufValueType.I16: "<h", GgufValueType.U32: "<I",
               GgufValueType.I32: "<i", GgufValueType.F32: "<f", GgufValueType.U64: "<Q", GgufValueType.I64: "<q", GgufValueType.F64: "<d"}


@dataclass
class GgufValue:
    """GgufMetadataValue / GgufArray (gguf.rs:155-295): a typed scalar, string, or homogeneous array (elem_type set)."""
    ty: GgufValueType
    value: object
    elem_type: Optional[GgufValueType] = None

    def as_u32(self) -> Optional[int]:
        return int(self.value) if self.ty in (GgufValueType.U8, GgufValueType.U16, GgufValueType.U32) else None


@dataclass
class GgufMetadataKv:
    key: str
    value: GgufValue


@dataclass
class GgufTensorInfo:
    """gguf.rs:319-330: offset is relative to the start of the tensor-data region."""
    name: str
    dims: List[int]
    ggml_type: int
    offset: int


@dataclass
class GgufFile:
    """gguf.rs:333-381."""
    metadata: List[GgufMetadataKv] = field(default_factory=list)
    tensors: List[GgufTensorInfo] = field(default_factory=list)
    tensor_data: bytes = b""
    alignment: int = GGUF_DEFAULT_ALIGNMENT

    def metadata_get(self, key: str) -> Optional[GgufValue]:
        for kv in self.metadata:
            if kv.key == key:
                return kv.value
        return None

    def tensor_bytes(self, info: GgufTensorInfo) -> bytes:
        """The stored records of one tensor whose type is one of the codecs above."""
        ty = GGUF_TENSOR_TAGS.get(info.ggml_type)
        if ty is None:
            raise L.InvalidConfig(L.ERR_INVALID_CONFIG, f"tensor {info.name!r}: ggml type {info.ggml_type} has no codec here")
        n = 1
        for d in info.dims:
            n *= d
        if n % ty.block_size() != 0:
            raise L.InvalidConfig(L.ERR_INVALID_CONFIG, f"tensor {info.name!r}: {n} weights are not whole {ty.name} blocks")
        size = n // ty.block_size() * ty.block_bytes()
        if info.offset + size > len(self.tensor_data):
            raise L.InvalidConfig(L.ERR_INVALID_CONFIG, f"tensor {info.name!r} runs past the tensor-data region")
        return self.tensor_data[info.offset:info.offset + size]

    def tensor_to_device(self, info: GgufTensorInfo, device, out_dtype=torch.bfloat16) -> torch.Tensor:
        """Upload one tensor's records and dequantize them on the GPU; returns the weights shaped dims[::-1]
        (GGUF lists the fastest-varying dimension first)."""
        ty = GGUF_TENSOR_TAGS[info.ggml_type] if info.ggml_type in GGUF_TENSOR_TAGS else None
        raw = torch.frombuffer(bytearray(self.tensor_bytes(info)), dtype=torch.uint8).to(device)
        return dequantize(raw, ty, out_dtype).reshape(*reversed(info.dims))


class _Reader:
    """Bounds-checked little-endian cursor (gguf.rs:383-470): a short read is InvalidConfig, never an exception of its own."""

    def __init__(self, data: bytes):
        self.b, self.pos = data, 0

    def take(self, n: int) -> bytes:
        if n < 0 or self.pos + n > len(self.b):
            raise L.InvalidConfig(L.ERR_INVALID_CONFIG, f"truncated GGUF: need {n} bytes at offset {self.pos}, {len(self.b) - self.pos} remain")
        out = self.b[self.pos:self.pos + n]
        self.pos += n
        return out

    def scalar(self, ty: GgufValueType):
        fmt = _SCALAR_FMT[ty]
        return struct.unpack(fmt, self.take(struct.calcsize(fmt)))[0]

    def string(self) -> str:
        n = self.scalar(GgufValueType.U64)
        try:
            return self.take(n).decode("utf-8")
        except UnicodeDecodeError:
            raise L.InvalidConfig(L.ERR_INVALID_CONFIG, "GGUF string is not valid UTF-8") from None


def _read_value(r: _Reader, ty: GgufValueType) -> GgufValue:
    if ty == GgufValueType.String:
        return GgufValue(ty, r.string())
    if ty == GgufValueType.Bool:
        return GgufValue(ty, r.scalar(GgufValueType.U8) != 0)
    if ty == GgufValueType.Array:
        et = GgufValueType.from_tag(r.scalar(GgufValueType.U32))
        if et == GgufValueType.Array:
            raise L.InvalidConfig(L.ERR_INVALID_CONFIG, "nested GGUF arrays are not supported")
        n = r.scalar(GgufValueType.U64)
        if n > len(r.b):                                    # every element takes at least one byte
            raise L.InvalidConfig(L.ERR_INVALID_CONFIG, f"GGUF array of {n} elements in a {len(r.b)}-byte file")
        return GgufValue(ty, [_read_value(r, et).value for _ in range(n)], et)
    return GgufValue(ty, r.scalar(ty))


def read_gguf(data: bytes) -> GgufFile:
    """read_gguf, gguf.rs:690-775."""
    r = _Reader(bytes(data))
    magic = r.scalar(GgufValueType.U32)
    if magic != GGUF_MAGIC:
        raise L.InvalidConfig(L.ERR_INVALID_CONFIG, f"bad GGUF magic: expected {GGUF_MAGIC:#010x}, got {magic:#010x}")
    version = r.scalar(GgufValueType.U32)
    if version != GGUF_VERSION:
        raise L.InvalidConfig(L.ERR_INVALID_CONFIG, f"unsupported GGUF version {version} (this reader supports v{GGUF_VERSION})")
    tensor_count, kv_count = r.scalar(GgufValueType.U64), r.scalar(GgufValueType.U64)
    f = GgufFile()
    for _ in range(kv_count):
        key = r.string()
        value = _read_value(r, GgufValueType.from_tag(r.scalar(GgufValueType.U32)))
        if key == ALIGNMENT_KEY and value.as_u32() is not None:
            if value.as_u32() == 0:
                raise L.InvalidConfig(L.ERR_INVALID_CONFIG, "GGUF general.alignment must be non-zero")
            f.alignment = value.as_u32()
        f.metadata.append(GgufMetadataKv(key, value))
    for _ in range(tensor_count):
        name = r.string()
        n_dims = r.scalar(GgufValueType.U32)
        dims = [r.scalar(GgufValueType.U64) for _ in range(n_dims)]
        f.tensors.append(GgufTensorInfo(name, dims, r.scalar(GgufValueType.U32), r.scalar(GgufValueType.U64)))
    start = (r.pos + f.alignment - 1) // f.alignment * f.alignment
    if start > len(r.b):
        raise L.InvalidConfig(L.ERR_INVALID_CONFIG, f"GGUF tensor-data start {start} past end of {len(r.b)}-byte file")
    f.tensor_data = r.b[start:]
    return f


def _write_value(out: bytearray, v: GgufValue):
    def string(s: str):
        raw = s.encode("utf-8")
        out.extend(struct.pack("<Q", len(raw)))
        out.extend(raw)

    def one(ty: GgufValueType, x):
        if ty == GgufValueType.String:
            string(x)
        elif ty == GgufValueType.Bool:
            out.append(1 if x else 0)
        else:
            out.extend(struct.pack(_SCALAR_FMT[ty], x))
    if v.ty == GgufValueType.Array:
        out.extend(struct.pack("<I", v.elem_type.value))
        out.extend(struct.pack("<Q", len(v.value)))
        for x in v.value:
            one(v.elem_type, x)
    else:
        one(v.ty, v.value)


def write_gguf(f: GgufFile) -> bytes:
    """write_gguf, gguf.rs:789-826: counts from the lists, directory in order, padding to the alignment, data verbatim."""
    out = bytearray()
    out.extend(struct.pack("<IIQQ", GGUF_MAGIC, GGUF_VERSION, len(f.tensors), len(f.metadata)))
    for kv in f.metadata:
        raw = kv.key.encode("utf-8")
        out.extend(struct.pack("<Q", len(raw)))
        out.extend(raw)
        out.extend(struct.pack("<I", kv.value.ty.value))
        _write_value(out, kv.value)
    for t in f.tensors:
        raw = t.name.encode("utf-8")
        out.extend(struct.pack("<Q", len(raw)))
        out.extend(raw)
        out.extend(struct.pack("<I", len(t.dims)))
        for d in t.dims:
            out.extend(struct.pack("<Q", d))
        out.extend(struct.pack("<IQ", t.ggml_type, t.offset))
    out.extend(b"\0" * ((-len(out)) % f.alignment))
    out.extend(f.tensor_data)
    return bytes(out)
