"""GGML block codecs and the GGUF container.

CPU: the oracle's restatement of crates/oxicuda-quant/src/scheme/ggml.rs against the properties the reference's own
tests assert on the same LCG inputs (ggml.rs:540-808), and the GGUF reader / writer (gguf.rs:690-826) round trip and
error cases (gguf.rs tests :830-1413).  GPU: quantized records and dequantized values bit-exact against the oracle."""
import struct

import numpy as np
import pytest
import torch


def lcg(n, seed, scale):
    """The reference tests' generator (ggml.rs:541-555): 64-bit LCG, top 32 bits / u32::MAX mapped to [-scale, scale]."""
    state, out = seed, np.empty(n, np.float32)
    for i in range(n):
        state = (state * 6364136223846793005 + 1442695040888963407) & ((1 << 64) - 1)
        f = np.float32(np.float32(state >> 32) / np.float32(4294967295.0))
        out[i] = np.float32((f * np.float32(2.0) - np.float32(1.0)) * np.float32(scale))
    return out


def rel_err(a, b):
    """ggml.rs:557-566"""
    return float(np.abs(a - b).sum(dtype=np.float32) / max(float(np.abs(a).sum(dtype=np.float32)), 1e-8))


def test_oracle_f16_pins(oracle):
    """ggml.rs:569-617: exact values, closeness, overflow to infinity, flush of tiny values, subnormals, bit inverse."""
    rt = lambda v: oracle.ggml_f16_to_f32(oracle.ggml_f32_to_f16_bits(v))
    for v in (0.0, 1.0, -1.0, 0.5, 2.0, 0.25, 1024.0, -0.125):
        assert abs(rt(v) - v) < 1e-6
    for v in (0.1, 3.1457, -2.7188, 100.0, 0.003):
        assert abs(rt(v) - v) / abs(v) < 1e-3
    assert rt(1.0e30) == float("inf") and rt(1.0e-20) == 0.0
    assert abs(rt(1.0e-6) - 1.0e-6) / 1.0e-6 < 0.05
    for v in (1.0, -2.5, 0.333, 65504.0):
        assert abs(oracle.ggml_f16_to_f32(oracle.ggml_f32_to_f16_bits(v)) - np.float32(v)) <= abs(v) * 2.0 ** -11
    # the conversion is numpy's / the hardware's round-to-nearest-even on every finite half and on the midpoints
    vals = np.concatenate([np.arange(0, 0x7C00, 7, dtype=np.uint16).view(np.float16).astype(np.float32),
                           lcg(4000, 9, 70000.0), lcg(2000, 10, 1e-4), lcg(2000, 11, 1e-7)])
    with np.errstate(over="ignore"):
        expect = vals.astype(np.float16).view(np.uint16)
    for v, e in zip(vals, expect):
        assert oracle.ggml_f32_to_f16_bits(float(v)) == int(e), v


def test_oracle_codecs_meet_the_reference_tests(oracle):
    """ggml.rs:636-795 restated on the oracle: round-trip error bounds, code ranges, zero block, six-bit sub-block
    parameters, Q4_1 on one-sided data, Q4_K on blocky data, errors."""
    w = lcg(320, 1, 4.0)
    q = oracle.ggml_quantize(w, oracle.GGML_Q8_0)
    assert q.size == 10 * 34 and rel_err(w, oracle.ggml_dequantize(q, 0)) < 0.01
    codes = oracle.ggml_quantize(lcg(32, 7, 2.0), 0)[2:].view(np.int8)
    assert codes.min() >= -127 and codes.max() <= 127
    assert not oracle.ggml_dequantize(oracle.ggml_quantize(np.zeros(32, np.float32), 0), 0).any()
    w = lcg(256, 2, 3.0)
    assert rel_err(w, oracle.ggml_dequantize(oracle.ggml_quantize(w, 1), 1)) < 0.12
    ramp = (np.arange(32, dtype=np.float32) / np.float32(31.0)) * np.float32(2.0) - np.float32(1.0)
    deq = oracle.ggml_dequantize(oracle.ggml_quantize(ramp, 1), 1)
    amax = np.abs(ramp).max()
    assert ((ramp - deq) ** 2).sum() < ((ramp - np.sign(ramp) * amax) ** 2).sum()
    w = lcg(256, 3, 3.0)
    assert rel_err(w, oracle.ggml_dequantize(oracle.ggml_quantize(w, 2), 2)) < 0.12
    pos = np.float32(1.0) + np.arange(32, dtype=np.float32) / np.float32(31.0)   # one-sided data: the affine codec wins
    assert rel_err(pos, oracle.ggml_dequantize(oracle.ggml_quantize(pos, 2), 2)) <= rel_err(pos, oracle.ggml_dequantize(oracle.ggml_quantize(pos, 1), 1))
    w = lcg(768, 4, 5.0)
    q = oracle.ggml_quantize(w, 3)
    assert q.size == 3 * 148 and rel_err(w, oracle.ggml_dequantize(q, 3)) < 0.12
    assert oracle.ggml_quantize(lcg(256, 9, 4.0), 3)[4:20].max() <= 63
    blocky = np.concatenate([ramp * np.float32((sb + 1.0) * 0.5) for sb in range(8)])
    assert rel_err(blocky, oracle.ggml_dequantize(oracle.ggml_quantize(blocky, 3), 3)) <= 1.05 * rel_err(blocky, oracle.ggml_dequantize(oracle.ggml_quantize(blocky, 1), 1))
    with pytest.raises(ValueError, match="EmptyInput"):
        oracle.ggml_quantize(np.zeros(0, np.float32), 0)
    with pytest.raises(ValueError, match="GroupSizeMismatch"):
        oracle.ggml_quantize(np.zeros(33, np.float32), 0)
    with pytest.raises(ValueError, match="GroupSizeMismatch"):
        oracle.ggml_quantize(np.zeros(255, np.float32), 3)
    # Q4_0 keeps the sign of the FIRST largest magnitude: d = max / -8
    blk = np.zeros(32, np.float32)
    blk[3], blk[9] = -2.0, 2.0
    assert oracle.ggml_f16_to_f32(int(oracle.ggml_quantize(blk, 1)[:2].view(np.uint16)[0])) == 0.25
    blk[3], blk[9] = 2.0, -2.0
    assert oracle.ggml_f16_to_f32(int(oracle.ggml_quantize(blk, 1)[:2].view(np.uint16)[0])) == -0.25


def _sample_file(G):
    """The representative container of the reference's tests (gguf.rs:837-900)."""
    V, T = G.GgufValue, G.GgufValueType
    md = [G.GgufMetadataKv("general.architecture", V(T.String, "llama")), G.GgufMetadataKv("llama.block_count", V(T.U32, 32)),
          G.GgufMetadataKv("llama.attention.head_count", V(T.I32, -1)),
          G.GgufMetadataKv("tokenizer.ggml.tokens", V(T.Array, ["<s>", "</s>", "hello"], T.String)),
          G.GgufMetadataKv("llama.rope.freqs", V(T.Array, [1.0, 0.5, 0.25], T.F32)), G.GgufMetadataKv(G.ALIGNMENT_KEY, V(T.U32, 32)),
          G.GgufMetadataKv("flag", V(T.Bool, True)), G.GgufMetadataKv("big", V(T.U64, 1 << 40)), G.GgufMetadataKv("pi", V(T.F64, 3.141592653589793))]
    tensors = [G.GgufTensorInfo("blk.0.attn_q.weight", [64, 2], 8, 0), G.GgufTensorInfo("blk.0.ffn.weight", [32], 2, 160)]
    data = bytes(range(256)) * 1
    return G.GgufFile(md, tensors, data[:160 + 18], 32)


def test_gguf_round_trip_and_errors():
    from oxicuda_b200 import _lib as L
    from oxicuda_b200 import ggml as G
    f = _sample_file(G)
    raw = G.write_gguf(f)
    assert raw[:4] == b"GGUF" and struct.unpack("<I", raw[4:8])[0] == 3
    assert struct.unpack("<QQ", raw[8:24]) == (2, 9)
    g = G.read_gguf(raw)
    assert g == f and G.write_gguf(g) == raw
    assert g.metadata_get("llama.block_count").value == 32 and g.metadata_get("missing") is None
    assert (len(raw) - len(f.tensor_data)) % 32 == 0                         # the data region starts on the alignment
    assert g.tensor_bytes(g.tensors[1]) == f.tensor_data[160:178]
    # a different alignment moves the data region
    f64 = _sample_file(G)
    f64.alignment = 64
    f64.metadata[5].value.value = 64
    r64 = G.write_gguf(f64)
    assert (len(r64) - len(f64.tensor_data)) % 64 == 0 and G.read_gguf(r64).alignment == 64
    bad = bytearray(raw)
    bad[0] = 0x58
    with pytest.raises(L.InvalidConfig, match="bad GGUF magic"):
        G.read_gguf(bytes(bad))
    bad = bytearray(raw)
    bad[4] = 2
    with pytest.raises(L.InvalidConfig, match="unsupported GGUF version"):
        G.read_gguf(bytes(bad))
    for cut in (3, 10, 30, 60, 100, 200):                                    # truncated anywhere in the header or the directory
        with pytest.raises(L.InvalidConfig):
            G.read_gguf(raw[:cut])
    # an unknown value-type tag
    key = b"k"
    blob = struct.pack("<IIQQ", G.GGUF_MAGIC, 3, 0, 1) + struct.pack("<Q", 1) + key + struct.pack("<I", 99)
    with pytest.raises(L.InvalidConfig, match="unknown GGUF value type"):
        G.read_gguf(blob)
    blob = struct.pack("<IIQQ", G.GGUF_MAGIC, 3, 0, 1) + struct.pack("<Q", len(G.ALIGNMENT_KEY)) + G.ALIGNMENT_KEY.encode() + struct.pack("<II", 4, 0)
    with pytest.raises(L.InvalidConfig, match="non-zero"):
        G.read_gguf(blob)
    blob = struct.pack("<IIQQ", G.GGUF_MAGIC, 3, 0, 1) + struct.pack("<Q", 2) + b"\xff\xfe" + struct.pack("<II", 4, 0)
    with pytest.raises(L.InvalidConfig, match="UTF-8"):
        G.read_gguf(blob)
    assert G.GgmlType.Q8_0.bits_per_weight() == 8.5 and G.GgmlType.Q4_K.block_size() == 256
    assert G.GgmlType.Q4_0.bits_per_weight() < G.GgmlType.Q4_1.bits_per_weight() < G.GgmlType.Q8_0.bits_per_weight()


@pytest.mark.gpu
@pytest.mark.parametrize("ty", [0, 1, 2, 3])
def test_gpu_codecs_bit_exact(cuda, oracle, ty):
    """Records and dequantized values equal the oracle's, on the reference tests' LCG data, on normal data with a wide
    range of block scales (down to binary16 subnormal scales), all-zero and one-sided blocks, and ties of the rounding."""
    from oxicuda_b200 import ggml as G
    from oxicuda_b200._lib import default_handle
    t = G.GgmlType(ty)
    bs = t.block_size()
    rng = np.random.default_rng(40 + ty)
    mag = np.exp2(rng.integers(-22, 12, 4096 // 32)).astype(np.float32).repeat(32)
    parts = [lcg(bs * 10, 1 + ty, 4.0), (rng.standard_normal(4096) * mag).astype(np.float32), np.zeros(bs, np.float32),
             np.abs(rng.standard_normal(bs * 4)).astype(np.float32) + 1.0, -np.abs(rng.standard_normal(bs * 2)).astype(np.float32),
             (rng.integers(-16, 17, bs * 8) * 0.5).astype(np.float32), (rng.standard_normal(1 << 18) * 0.02).astype(np.float32)]
    w = np.concatenate(parts)
    ref_q = oracle.ggml_quantize(w, ty)
    got_q = G.quantize(torch.from_numpy(w).to(cuda), t)
    default_handle().check()
    got_qn = got_q.cpu().numpy()
    assert got_qn.size == ref_q.size == w.size // bs * t.block_bytes()
    if not np.array_equal(got_qn, ref_q):
        bad = np.nonzero(got_qn != ref_q)[0]
        raise AssertionError(f"{bad.size} bytes differ, first at record {bad[0] // t.block_bytes()} byte {bad[0] % t.block_bytes()}")
    ref_d = oracle.ggml_dequantize(ref_q, ty)
    got_d = G.dequantize(got_q, t).cpu().numpy()
    assert np.array_equal(got_d.view(np.uint32), ref_d.view(np.uint32))
    got_b = G.dequantize(got_q, t, torch.bfloat16)
    assert torch.equal(got_b.cpu(), torch.from_numpy(ref_d).to(torch.bfloat16))
    assert torch.equal(G.fake_quantize(torch.from_numpy(w).to(cuda), t).cpu(), torch.from_numpy(ref_d))
    from oxicuda_b200 import _lib as L
    with pytest.raises(L.EmptyInput):
        G.quantize(torch.zeros(0, device=cuda), t)
    with pytest.raises(L.GroupSizeMismatch):
        G.quantize(torch.zeros(bs + 1, device=cuda), t)


@pytest.mark.gpu
def test_gguf_tensor_to_device(cuda, oracle):
    """The reference's end-to-end case (gguf.rs:1350-1412): quantize with Q8_0, store in a container, read it back,
    dequantize -- here the dequantization runs on the GPU from the container's bytes."""
    from oxicuda_b200 import ggml as G
    w = lcg(64 * 4, 21, 2.0)
    rec = oracle.ggml_quantize(w, 0)
    q4 = oracle.ggml_quantize(w, 1)
    pad = (-rec.size) % 32
    data = rec.tobytes() + b"\0" * pad + q4.tobytes()
    f = G.GgufFile([G.GgufMetadataKv("general.name", G.GgufValue(G.GgufValueType.String, "t"))],
                   [G.GgufTensorInfo("w8", [64, 4], 8, 0), G.GgufTensorInfo("w4", [64, 4], 2, rec.size + pad)], data, 32)
    g = G.read_gguf(G.write_gguf(f))
    for info, ty in ((g.tensors[0], 0), (g.tensors[1], 1)):
        got = g.tensor_to_device(info, cuda, torch.float32)
        assert got.shape == (4, 64)
        assert np.array_equal(got.cpu().numpy().reshape(-1), oracle.ggml_dequantize(oracle.ggml_quantize(w, ty), ty))
