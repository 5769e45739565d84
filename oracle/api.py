"""numpy front end of the CPU oracle (oracle/oracle.cpp -> oracle/liboracle.so).

TEST INFRASTRUCTURE ONLY: imported by tests/, by __graft_entry__.smoke() and by the
cpu_baseline / reference legs of bench.py — never by the oxicuda_b200 package.
"""
from __future__ import annotations

import ctypes as C
import subprocess
from pathlib import Path

import numpy as np

_DIR = Path(__file__).resolve().parent
_LIB = _DIR / "liboracle.so"
_lib = None


def build(force: bool = False) -> Path:
    src = _DIR / "oracle.cpp"
    if force or not _LIB.exists() or _LIB.stat().st_mtime < src.stat().st_mtime:
        r = subprocess.run(["make", "-C", str(_DIR), "-B" if force else "-s", "liboracle.so"], capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("building the oracle failed:\n" + r.stdout + r.stderr)
    return _LIB


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        build()
        L = C.CDLL(str(_LIB))
        L.orc_fp8_encode.restype = C.c_int64
        L.orc_fp8_quantize_rows.restype = C.c_int64
        L.orc_llm_int8_matmul.restype = C.c_int64
        L.orc_fp4_quantize_one.restype = C.c_uint8
        L.orc_fp4_quantize_one.argtypes = [C.c_float, C.c_int]
        L.orc_fp4_dequantize_one.restype = C.c_float
        L.orc_fp4_dequantize_one.argtypes = [C.c_uint8, C.c_int]
        L.orc_e8m0_from_absmax.restype = C.c_uint8
        L.orc_e8m0_from_absmax.argtypes = [C.c_float]
        L.orc_fp8_split_k.restype = C.c_uint32
        _lib = L
    return _lib


def _p(a):
    return C.c_void_p(0) if a is None else C.c_void_p(a.ctypes.data)


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def _i64(v):
    return C.c_int64(int(v))


def num_threads() -> int:
    return lib().orc_num_threads()


def set_threads(n: int):
    lib().orc_set_threads(int(n))


# ---- MinMax ----
def minmax_calibrate(x, rows, cols, bits=8, scheme=0):
    x = _f32(x).reshape(-1)
    scales = np.zeros(rows, np.float32)
    zps = np.zeros(rows, np.int32)
    st = lib().orc_minmax_calibrate(_p(x), _i64(rows), _i64(cols), bits, scheme, _p(scales), _p(zps))
    return scales, zps, st


def minmax_quantize(x, rows, cols, scales, zps, bits=8, scheme=0):
    x = _f32(x).reshape(-1)
    codes = np.zeros(rows * cols, np.int32)
    scales, zps = _f32(scales), np.ascontiguousarray(zps, np.int32)    # locals keep converted copies alive
    lib().orc_minmax_quantize(_p(x), _i64(rows), _i64(cols), _p(scales), _p(zps), bits, scheme, _p(codes))
    return codes


def minmax_dequantize(codes, rows, cols, scales, zps):
    codes = np.ascontiguousarray(codes, np.int32).reshape(-1)
    out = np.zeros(rows * cols, np.float32)
    scales, zps = _f32(scales), np.ascontiguousarray(zps, np.int32)
    lib().orc_minmax_dequantize(_p(codes), _i64(rows), _i64(cols), _p(scales), _p(zps), _p(out))
    return out


def fake_quant(x, scale, zp, qmin, qmax):
    x = _f32(x).reshape(-1)
    out = np.zeros_like(x)
    lib().orc_fake_quant(_p(x), _i64(x.size), C.c_float(scale), C.c_float(zp), C.c_float(qmin), C.c_float(qmax), _p(out))
    return out


# ---- FP8 ----
def fp8_encode(x, fmt=0, mode=0):
    """mode 0 = reference codec, 1 = RNE.  Returns (codes, index_of_first_nonfinite or -1)."""
    x = _f32(x).reshape(-1)
    out = np.zeros(x.size, np.uint8)
    bad = lib().orc_fp8_encode(_p(x), _i64(x.size), fmt, mode, _p(out))
    return out, int(bad)


def fp8_decode(codes, fmt=0, mode=0):
    codes = np.ascontiguousarray(codes, np.uint8).reshape(-1)
    out = np.zeros(codes.size, np.float32)
    lib().orc_fp8_decode(_p(codes), _i64(codes.size), fmt, mode, _p(out))
    return out


def fp8_quantize_rows(x, rows, cols, fmt=0, mode=0):
    x = _f32(x).reshape(-1)
    scales = np.zeros(rows, np.float32)
    codes = np.zeros(rows * cols, np.uint8)
    bad = lib().orc_fp8_quantize_rows(_p(x), _i64(rows), _i64(cols), fmt, mode, _p(scales), _p(codes))
    return codes, scales, int(bad)


# ---- FP4 ----
def fp4_quantize_one(v, fmt=0):
    return int(lib().orc_fp4_quantize_one(float(v), fmt))


def fp4_dequantize_one(raw, fmt=0):
    return float(lib().orc_fp4_dequantize_one(int(raw), fmt))


def e8m0_from_absmax(a):
    return int(lib().orc_e8m0_from_absmax(float(a)))


def fp4_quantize(x, fmt=0):
    x = _f32(x).reshape(-1)
    out = np.zeros(x.size // 2, np.uint8)
    lib().orc_fp4_quantize(_p(x), _i64(x.size), fmt, _p(out))
    return out


def fp4_dequantize(packed, fmt=0):
    packed = np.ascontiguousarray(packed, np.uint8).reshape(-1)
    out = np.zeros(packed.size * 2, np.float32)
    lib().orc_fp4_dequantize(_p(packed), _i64(packed.size), fmt, _p(out))
    return out


def fp4_block_quantize(x, block=32, fmt=0, scale_mode=0):
    """scale_mode 0: f32 scales (reference), 1: E8M0 bytes.  Returns (packed, scales)."""
    x = _f32(x).reshape(-1)
    nb = -(-x.size // block)
    packed = np.zeros((x.size + 1) // 2, np.uint8)
    sf = np.zeros(nb, np.float32)
    se = np.zeros(nb, np.uint8)
    lib().orc_fp4_block_quantize(_p(x), _i64(x.size), block, fmt, scale_mode, _p(packed), _p(sf), _p(se))
    return packed, (sf if scale_mode == 0 else se)


def fp4_block_dequantize(packed, scales, n, block=32, fmt=0):
    packed = np.ascontiguousarray(packed, np.uint8).reshape(-1)
    scale_mode = 1 if scales.dtype == np.uint8 else 0
    out = np.zeros(n, np.float32)
    s = np.ascontiguousarray(scales)
    lib().orc_fp4_block_dequantize(_p(packed), _i64(n), block, fmt, scale_mode,
                                   _p(s) if scale_mode == 0 else _p(None), _p(s) if scale_mode == 1 else _p(None), _p(out))
    return out


# ---- NF4 ----
def nf4_encode(x, block=64):
    x = _f32(x).reshape(-1)
    packed = np.zeros(x.size // 2, np.uint8)
    absmaxs = np.zeros(x.size // block, np.float32)
    lib().orc_nf4_encode(_p(x), _i64(x.size), block, _p(packed), _p(absmaxs))
    return packed, absmaxs


def nf4_decode(packed, absmaxs, block=64):
    packed = np.ascontiguousarray(packed, np.uint8).reshape(-1)
    out = np.zeros(packed.size * 2, np.float32)
    absmaxs = _f32(absmaxs)
    lib().orc_nf4_decode(_p(packed), _i64(packed.size), block, _p(absmaxs), _p(out))
    return out


# ---- dist-infer INT8-in-u8 ----
def distfp8_quantize_block(x, block):
    x = _f32(x).reshape(-1)
    block = max(1, int(block))
    q = np.zeros(x.size, np.uint8)
    absmaxs = np.zeros(-(-x.size // block), np.float32)
    lib().orc_distfp8_quantize_block(_p(x), _i64(x.size), _i64(block), _p(q), _p(absmaxs))
    return q, absmaxs


def distfp8_dequantize_block(q, absmaxs, block):
    q = np.ascontiguousarray(q, np.uint8).reshape(-1)
    out = np.zeros(q.size, np.float32)
    absmaxs = _f32(absmaxs)
    lib().orc_distfp8_dequantize_block(_p(q), _i64(q.size), _i64(max(1, int(block))), _p(absmaxs), _p(out))
    return out


# ---- LLM.int8 ----
def llm_int8_matmul(x, w, samples, rows, cols, threshold=6.0, row_wise=True):
    x = _f32(x).reshape(-1)
    w = _f32(w).reshape(-1)
    out = np.zeros(samples * rows, np.float32)
    wq = np.zeros(rows * cols, np.int8)
    sw = np.zeros(rows, np.float32)
    xq = np.zeros(samples * cols, np.int8)
    sx = np.zeros(samples, np.float32)
    acc = np.zeros(samples * rows, np.int32)
    mask = np.zeros(cols, np.uint8)
    n_out = lib().orc_llm_int8_matmul(_p(x), _p(w), _i64(samples), _i64(rows), _i64(cols), C.c_float(threshold),
                                      int(bool(row_wise)), _p(out), _p(wq), _p(sw), _p(xq), _p(sx), _p(acc), _p(mask))
    return dict(output=out, w_q=wq, s_w=sw, x_q=xq, s_x=sx, acc=acc, outlier_mask=mask, n_outliers=int(n_out))


def gemm_i8(a, b):
    a = np.ascontiguousarray(a, np.int8)
    b = np.ascontiguousarray(b, np.int8)
    M, K = a.shape
    N = b.shape[0]
    c = np.zeros((M, N), np.int32)
    lib().orc_gemm_i8(_p(a), _p(b), _i64(M), _i64(N), _i64(K), _p(c))
    return c


# ---- FP8 GEMM / FP4 GEMV compositions ----
def bf16_bits_to_f32(b):
    return (np.ascontiguousarray(b, np.uint16).astype(np.uint32) << 16).view(np.float32)


def f32_to_bf16_bits(x):
    u = _f32(x).view(np.uint32).astype(np.uint64)
    lsb = (u >> 16) & 1
    return ((u + 0x7FFF + lsb) >> 16).astype(np.uint16)


def gemm_fp8(a_codes, w_codes, sa, sw, fmt=0, decode_mode=0, want="bf16"):
    """a [M,K] u8, w [N,K] u8, sa 1 or M floats, sw 1 or N floats.  Returns f32 values
    (bf16-rounded when want == 'bf16')."""
    a = np.ascontiguousarray(a_codes, np.uint8)
    w = np.ascontiguousarray(w_codes, np.uint8)
    M, K = a.shape
    N = w.shape[0]
    sa = _f32(sa).reshape(-1)
    sw = _f32(sw).reshape(-1)
    ob = np.zeros((M, N), np.uint16) if want == "bf16" else None
    of = np.zeros((M, N), np.float32) if want != "bf16" else None
    lib().orc_gemm_fp8(_p(a), _p(w), _i64(M), _i64(N), _i64(K), fmt, decode_mode, _p(sa), int(sa.size > 1), _p(sw),
                       int(sw.size > 1), _p(ob), _p(of))
    return bf16_bits_to_f32(ob).reshape(M, N) if want == "bf16" else of


def gemv_fp4(codes, scales, x_bf16_bits, M, N, K, block=32, want="bf16"):
    codes = np.ascontiguousarray(codes, np.uint8).reshape(-1)
    scale_mode = 1 if scales.dtype == np.uint8 else 0
    s = np.ascontiguousarray(scales).reshape(-1)
    xb = np.ascontiguousarray(x_bf16_bits, np.uint16).reshape(-1)
    ob = np.zeros((M, N), np.uint16) if want == "bf16" else None
    of = np.zeros((M, N), np.float32) if want != "bf16" else None
    lib().orc_gemv_fp4(_p(codes), scale_mode, _p(s) if scale_mode == 0 else _p(None), _p(s) if scale_mode == 1 else _p(None),
                       block, _p(xb), _i64(M), _i64(N), _i64(K), _p(ob), _p(of))
    return bf16_bits_to_f32(ob).reshape(M, N) if want == "bf16" else of


# ---- tensor parallel ----
def column_linear(x, w, bias, batch, in_f, out_f, tp):
    x, w = _f32(x).reshape(-1), _f32(w).reshape(-1)          # keep the (possibly copied) arrays alive over the call
    b = None if bias is None else _f32(bias)
    out = np.zeros(batch * out_f, np.float32)
    lib().orc_column_linear(_p(x), _p(w), _p(b), _i64(batch), _i64(in_f), _i64(out_f), tp, _p(out))
    return out.reshape(batch, out_f)


def row_linear(x, w, bias, batch, in_f, out_f, tp):
    x, w = _f32(x).reshape(-1), _f32(w).reshape(-1)
    b = None if bias is None else _f32(bias)
    out = np.zeros(batch * out_f, np.float32)
    lib().orc_row_linear(_p(x), _p(w), _p(b), _i64(batch), _i64(in_f), _i64(out_f), tp, _p(out))
    return out.reshape(batch, out_f)


def swiglu(gate, up):
    g = _f32(gate).reshape(-1)
    u = _f32(up).reshape(-1)
    h = np.zeros_like(g)
    lib().orc_swiglu(_p(g), _p(u), _i64(g.size), _p(h))
    return h.reshape(np.shape(gate))


def swiglu_mlp_hidden(x_codes, x_scales, w_codes, w_scales, tokens, hidden, F, interleaved=False):
    """h = silu(gate) * up between the two projections of the FP8 SwiGLU MLP (SwiGluExpert::forward,
    crates/oxicuda-moe/src/expert/ffn.rs:208-243, over Fp8Codec operands; a composition: the reference has no quantized
    MLP, parity unpinned).  w_codes [2F x hidden] in one of the two layouts of the library:
      concatenated (rows [0, F) gate, [F, 2F) up): the gate | up product is a GEMM output, rounded to bf16; h in f32;
      interleaved per 128 rows (rows [256 j, 256 j + 128) gate rows [128 j, ...), then the same up rows): the product stays
      in f32 and h is rounded to bf16 (it is what the GEMM writes).
    The per-row E4M3 quantization that follows amplifies the difference between the two (a few per cent of the elements
    change code), so each layout is compared with its own statement."""
    gu = np.asarray(gemm_fp8(np.asarray(x_codes).reshape(tokens, hidden), np.asarray(w_codes).reshape(2 * F, hidden), x_scales, w_scales, 0, 1,
                             "f32" if interleaved else "bf16"), np.float32).reshape(tokens, 2 * F)
    if not interleaved:
        return swiglu(np.ascontiguousarray(gu[:, :F]), np.ascontiguousarray(gu[:, F:]))
    g4 = gu.reshape(tokens, F // 128, 2, 128)
    h = swiglu(np.ascontiguousarray(g4[:, :, 0, :]).reshape(tokens, F), np.ascontiguousarray(g4[:, :, 1, :]).reshape(tokens, F))
    return bf16_bits_to_f32(f32_to_bf16_bits(h)).reshape(tokens, F)


def interleave_rows128(a, b):
    """Rows of a and b interleaved per 128 rows (b2q_interleave_rows128)."""
    a, b = np.asarray(a), np.asarray(b)
    F = a.shape[0]
    return np.stack([a.reshape(F // 128, 128, *a.shape[1:]), b.reshape(F // 128, 128, *b.shape[1:])], axis=1).reshape(2 * F, *a.shape[1:])


# ---- GGML block codecs (crates/oxicuda-quant/src/scheme/ggml.rs) ----
GGML_Q8_0, GGML_Q4_0, GGML_Q4_1, GGML_Q4_K = 0, 1, 2, 3


def ggml_block_bytes(ty):
    return {0: 34, 1: 18, 2: 20, 3: 148}[ty]


def ggml_block_size(ty):
    return 256 if ty == 3 else 32


def ggml_f32_to_f16_bits(x):
    L = lib()
    L.orc_ggml_f32_to_f16_bits.restype = C.c_uint16
    L.orc_ggml_f32_to_f16_bits.argtypes = [C.c_float]
    return int(L.orc_ggml_f32_to_f16_bits(float(x)))


def ggml_f16_to_f32(h):
    L = lib()
    L.orc_ggml_f16_to_f32.restype = C.c_float
    L.orc_ggml_f16_to_f32.argtypes = [C.c_uint16]
    return float(L.orc_ggml_f16_to_f32(int(h)))


def ggml_quantize(w, ty):
    """Packed block records (uint8) of the flat weights; raises ValueError as check_block does (ggml.rs:522-534)."""
    w = _f32(w).reshape(-1)
    L = lib()
    L.orc_ggml_quantize.restype = C.c_int64
    out = np.zeros(max(1, w.size // ggml_block_size(ty)) * ggml_block_bytes(ty), np.uint8)
    nb = L.orc_ggml_quantize(ty, _p(w), _i64(w.size), _p(out))
    if nb == -1:
        raise ValueError("EmptyInput")
    if nb == -2:
        raise ValueError("GroupSizeMismatch")
    return out[:nb * ggml_block_bytes(ty)]


def ggml_dequantize(blocks, ty):
    blocks = np.ascontiguousarray(blocks, np.uint8).reshape(-1)
    n = blocks.size // ggml_block_bytes(ty) * ggml_block_size(ty)
    out = np.zeros(n, np.float32)
    lib().orc_ggml_dequantize(ty, _p(blocks), _i64(n), _p(out))
    return out


# ---- heuristics ----
# ---- KV cache / RMSNorm ----
def kv_cache_quantize(x, n_tokens, head_dim, bits=8, axis=0):
    """axis 0 = PerToken, 1 = PerChannel.  Returns (codes u8, scales, zero_points)."""
    x = _f32(x).reshape(-1)
    groups = n_tokens if axis == 0 else head_dim
    codes = np.zeros(n_tokens * head_dim, np.uint8)
    scales = np.zeros(groups, np.float32)
    zps = np.zeros(groups, np.float32)
    lib().orc_kv_cache_quantize(_p(x), _i64(n_tokens), _i64(head_dim), bits, axis, _p(codes), _p(scales), _p(zps))
    return codes, scales, zps


def kv_cache_dequantize(codes, n_tokens, head_dim, axis, scales, zps):
    codes = np.ascontiguousarray(codes, np.uint8).reshape(-1)
    scales, zps = _f32(scales), _f32(zps)
    out = np.zeros(n_tokens * head_dim, np.float32)
    lib().orc_kv_cache_dequantize(_p(codes), _i64(n_tokens), _i64(head_dim), axis, _p(scales), _p(zps), _p(out))
    return out


def kv_quantize_tokens(x, n_tokens, d, bits=8, symmetric=False):
    """Returns (codes i32, scales, zero_points), one (scale, zero point) per token."""
    x = _f32(x).reshape(-1)
    codes = np.zeros(n_tokens * d, np.int32)
    scales = np.zeros(n_tokens, np.float32)
    zps = np.zeros(n_tokens, np.float32)
    lib().orc_kv_quantize_tokens(_p(x), _i64(n_tokens), _i64(d), bits, int(bool(symmetric)), _p(codes), _p(scales), _p(zps))
    return codes, scales, zps


def kv_dequantize_tokens(codes, n_tokens, d, scales, zps):
    codes = np.ascontiguousarray(codes, np.int32).reshape(-1)
    scales, zps = _f32(scales), _f32(zps)
    out = np.zeros(n_tokens * d, np.float32)
    lib().orc_kv_dequantize_tokens(_p(codes), _i64(n_tokens), _i64(d), _p(scales), _p(zps), _p(out))
    return out


def rms_norm(x, gamma, rows, cols, eps, residual=None):
    """Returns y (and the updated residual when one is given)."""
    x = _f32(x).reshape(-1)
    gamma = _f32(gamma).reshape(-1)
    y = np.zeros(rows * cols, np.float32)
    res = None if residual is None else _f32(residual).reshape(-1).copy()
    lib().orc_rms_norm(_p(x), _p(res), _p(gamma), _i64(rows), _i64(cols), C.c_float(eps), _p(y))
    return y if residual is None else (y, res)


# ---- oxicuda-dnn quantize ----
def dnn_quantize_to_fp8(x):
    x = _f32(x).reshape(-1)
    codes, scale = np.zeros(x.size, np.uint8), np.zeros(1, np.float32)
    lib().orc_dnn_quantize_to_fp8(_p(x), _i64(x.size), _p(codes), _p(scale))
    return codes, scale


def dnn_dequantize_from_fp8(codes, scale):
    codes = np.ascontiguousarray(codes, np.uint8).reshape(-1)
    out = np.zeros(codes.size, np.float32)
    lib().orc_dnn_dequantize_from_fp8(_p(codes), C.c_float(float(scale)), _i64(codes.size), _p(out))
    return out


def dnn_quantize_to_int8(x):
    x = _f32(x).reshape(-1)
    q, scale = np.zeros(x.size, np.int8), np.zeros(1, np.float32)
    lib().orc_dnn_quantize_to_int8(_p(x), _i64(x.size), _p(q), _p(scale))
    return q, scale


def dnn_dequantize_from_int8(q, scale):
    q = np.ascontiguousarray(q, np.int8).reshape(-1)
    out = np.zeros(q.size, np.float32)
    lib().orc_dnn_dequantize_from_int8(_p(q), C.c_float(float(scale)), _i64(q.size), _p(out))
    return out


def dnn_quantize_block_scaled(x, block):
    x = _f32(x).reshape(-1)
    out, scales = np.zeros(x.size, np.uint8), np.zeros(-(-x.size // block), np.float32)
    lib().orc_dnn_quantize_block_scaled(_p(x), _i64(x.size), _i64(block), _p(out), _p(scales))
    return out, scales


def block_int8_quantize(x, block):
    x = _f32(x).reshape(-1)
    q, scales = np.zeros(x.size, np.int8), np.zeros(-(-x.size // block), np.float32)
    lib().orc_block_int8_quantize(_p(x), _i64(x.size), _i64(block), _p(q), _p(scales))
    return q, scales


def block_int8_dequantize(q, scales, block):
    q = np.ascontiguousarray(q, np.int8).reshape(-1)
    scales = _f32(scales)
    out = np.zeros(q.size, np.float32)
    lib().orc_block_int8_dequantize(_p(q), _p(scales), _i64(q.size), _i64(block), _p(out))
    return out


def block_absmax_scale(x, block, max_val=6.0):
    x = _f32(x).reshape(-1)
    scales = np.zeros(-(-x.size // block), np.float32)
    lib().orc_block_absmax_scale(_p(x), _i64(x.size), _i64(block), C.c_float(max_val), _p(scales))
    return scales


# ---- INT4 group-scaled weight-only GEMM ----
def pack_int4(values):
    """Returns (packed u32 array, status): 0 ok, 1 length not a multiple of 8, 2 + i first value out of [-8, 7]."""
    v = np.ascontiguousarray(values, np.int8).reshape(-1)
    packed = np.zeros(v.size // 8, np.uint32)
    lib().orc_pack_int4.restype = C.c_int64
    st = lib().orc_pack_int4(_p(v), _i64(v.size), _p(packed))
    return packed, int(st)


def unpack_int4(packed):
    p = np.ascontiguousarray(packed, np.uint32).reshape(-1)
    out = np.zeros(p.size * 8, np.int8)
    lib().orc_unpack_int4(_p(p), _i64(p.size), _p(out))
    return out


def gemm_int4(a_packed, scales_f16, b, M, N, K, group):
    """a_packed u32 [M, K/8], scales float16 [M, K/group], b f32 [K, N] -> c f32 [M, N] in the reference kernel's order."""
    a = np.ascontiguousarray(a_packed, np.uint32).reshape(-1)
    sc = np.ascontiguousarray(scales_f16, np.float16).reshape(-1).view(np.uint16)
    b = _f32(b).reshape(-1)
    c = np.zeros(M * N, np.float32)
    lib().orc_gemm_int4(_p(a), _p(sc), _p(b), _p(c), _i64(M), _i64(N), _i64(K), _i64(group))
    return c.reshape(M, N)


def classify_workload(m, n, k):
    return int(lib().orc_classify_workload(C.c_uint32(m), C.c_uint32(n), C.c_uint32(k)))


def tile_config(dtype, m, n, k):
    out = np.zeros(8, np.uint32)
    lib().orc_tile_config(dtype, C.c_uint32(m), C.c_uint32(n), C.c_uint32(k), _p(out))
    return tuple(int(v) for v in out)


def fp8_split_k(m, n, k):
    return int(lib().orc_fp8_split_k(C.c_uint32(m), C.c_uint32(n), C.c_uint32(k)))


# ---- GPTQ / AWQ kernels of oxicuda-dnn (crates/oxicuda-dnn/src/quantize/gptq_awq.rs) ----
def wq_packed_words(rows, cols, bits):
    """quantized_weight_info().packed_weight_elements (gptq_awq.rs:996-1001)."""
    epu = 32 // bits
    return (rows * cols + epu - 1) // epu


def gptq_quantize(w, hessian_diag, rows, cols, group, bits, symmetric):
    """dnn_gptq_quantize_f32 -> (packed u32 [ceil(rows*cols/epu)], scales f32 [rows x cols/group])."""
    w, hd = _f32(w).reshape(-1), _f32(hessian_diag).reshape(-1)
    packed = np.zeros(wq_packed_words(rows, cols, bits), np.uint32)
    scales = np.zeros(rows * (cols // group), np.float32)
    lib().orc_gptq_quantize(_p(w), _p(hd), _i64(rows), _i64(cols), _i64(group), int(bits), int(bool(symmetric)), _p(packed), _p(scales))
    return packed, scales


def wq_dequantize(packed, scales, zeros, rows, cols, group, bits):
    """dnn_gptq_dequantize_f32 -> f32 [rows*cols]; zeros None = the symmetric kernel."""
    packed = np.ascontiguousarray(packed, np.uint32)
    scales = _f32(scales).reshape(-1)
    zeros = None if zeros is None else _f32(zeros).reshape(-1)
    out = np.zeros(rows * cols, np.float32)
    lib().orc_wq_dequantize(_p(packed), _p(scales), _p(zeros), _i64(rows), _i64(cols), _i64(group), int(bits), _p(out))
    return out


def awq_scale_search(act_stats):
    act = _f32(act_stats).reshape(-1)
    out = np.zeros(act.size, np.float32)
    lib().orc_awq_scale_search(_p(act), _i64(act.size), _p(out))
    return out


def awq_quantize(w, channel_scales, group_scales, rows, cols, group, bits, zero_point=True):
    """dnn_awq_quantize_f32 -> (packed u32, zeros f32 [rows x cols/group] or None)."""
    w, cs, gs = _f32(w).reshape(-1), _f32(channel_scales).reshape(-1), _f32(group_scales).reshape(-1)
    packed = np.zeros(wq_packed_words(rows, cols, bits), np.uint32)
    zeros = np.full(rows * (cols // group), np.nan, np.float32) if zero_point else None
    lib().orc_awq_quantize(_p(w), _p(cs), _p(gs), _i64(rows), _i64(cols), _i64(group), int(bits), _p(packed), _p(zeros))
    return packed, zeros


def fused_dequant_gemv(packed, scales, zeros, x, rows, cols, group, bits):
    """dnn_fused_dequant_gemv_f32 -> y f32 [rows], the reference's column-ascending fma chain."""
    packed = np.ascontiguousarray(packed, np.uint32)
    scales, x = _f32(scales).reshape(-1), _f32(x).reshape(-1)
    zeros = None if zeros is None else _f32(zeros).reshape(-1)
    y = np.zeros(rows, np.float32)
    lib().orc_fused_dequant_gemv(_p(packed), _p(scales), _p(zeros), _p(x), _i64(rows), _i64(cols), _i64(group), int(bits), _p(y))
    return y
