// CPU oracle for the quantized-linear hot path.
//
// TEST INFRASTRUCTURE ONLY.  This file restates, function by function, the CPU
// arithmetic of the reference (OxiCUDA, a pure-Rust workspace) for the
// quantize/dequantize entry points and the INT8 / FP8 / block-scaled-FP4
// GEMM / GEMV compositions.  It is what the CUDA path is checked against and
// what the CPU baseline leg of the benchmark times; nothing in the shipped
// library may call it.
//
// The reference cannot be compiled in an environment without a Rust toolchain,
// so every function here cites the reference file:line it follows and is pinned
// against the known-answer vectors of the reference's own unit tests
// (tests/golden/reference_kat.json).  Items that exist in no reference test or
// source (E8M0 scales) are marked "parity unpinned".
//
// Build: g++ -O2 -ffp-contract=off -fno-fast-math -fopenmp -shared -fPIC
// (-ffp-contract=off matters: Rust never fuses a*b+c unless mul_add is written.)

#include <cmath>
#include <cstdint>
#include <cstring>
#include <cstdlib>
#include <vector>
#include <algorithm>
#include <limits>
#ifdef _OPENMP
#include <omp.h>
#endif

namespace {

inline uint32_t f2u(float f) { uint32_t u; std::memcpy(&u, &f, 4); return u; }
inline float u2f(uint32_t u) { float f; std::memcpy(&f, &u, 4); return f; }

// Rust `f32::max`: returns the non-NaN operand when one is NaN (IEEE maxNum).
inline float rmax(float a, float b) { return std::fmax(a, b); }
inline float rmin(float a, float b) { return std::fmin(a, b); }

// Rust `f32::clamp(lo, hi)`: NaN stays NaN; otherwise plain comparisons.
inline float rclamp(float v, float lo, float hi) {
  if (v < lo) return lo;
  if (v > hi) return hi;
  return v;
}

// Rust `as i32` from f32: saturating, NaN -> 0.
inline int32_t f32_as_i32(float v) {
  if (std::isnan(v)) return 0;
  if (v >= 2147483648.0f) return INT32_MAX;
  if (v <= -2147483648.0f) return INT32_MIN;
  return (int32_t)v;
}
inline int8_t f32_as_i8(float v) {
  if (std::isnan(v)) return 0;
  if (v >= 127.0f) return 127;
  if (v <= -128.0f) return -128;
  return (int8_t)v;
}

// bf16 <-> f32 (round to nearest even; the bf16 outputs of the GEMM/GEMV
// compositions use RNE, as the hardware cvt.rn.bf16.f32 does).
inline uint16_t f32_to_bf16_rne(float f) {
  uint32_t u = f2u(f);
  if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40);
  uint32_t lsb = (u >> 16) & 1u;
  u += 0x7fffu + lsb;
  return (uint16_t)(u >> 16);
}
inline float bf16_to_f32(uint16_t h) { return u2f((uint32_t)h << 16); }

// ---------------------------------------------------------------------------
// FP8 codecs
// ---------------------------------------------------------------------------
struct Fp8Fmt { int exp_bits, man_bits, bias; float max_val; uint8_t sat; };
const Fp8Fmt kE4M3 = {4, 3, 7, 448.0f, 0x7E};
const Fp8Fmt kE5M2 = {5, 2, 15, 57344.0f, 0x7B};
inline const Fp8Fmt& fmt_of(int f) { return f == 0 ? kE4M3 : kE5M2; }

// Fp8Codec::fp32_to_fp8 — crates/oxicuda-quant/src/scheme/fp8.rs:163-208.
// Mantissa is TRUNCATED; any biased exponent >= 2^eb-1 saturates (so E4M3
// magnitudes >= 256 all become 0x7E); the subnormal branch shifts one bit too
// far.  Reproduced as written.
uint8_t fp8_encode_ref(float v, const Fp8Fmt& F) {
  uint32_t bits = f2u(v);
  uint8_t sign = (uint8_t)(bits >> 31);
  int exp32 = (int)((bits >> 23) & 0xFF);
  uint32_t man32 = bits & 0x007FFFFFu;
  if (v == 0.0f) return (uint8_t)(sign << 7);
  int exp8_raw = exp32 - 127 + F.bias;
  uint32_t man_shift = 23 - F.man_bits;
  if (exp8_raw <= 0) {
    uint32_t full_man = (man32 | 0x00800000u) >> 1;
    uint32_t shift = (uint32_t)(1 - exp8_raw) + man_shift;
    if (shift >= 24) return (uint8_t)(sign << 7);
    uint8_t man8 = (uint8_t)((full_man >> shift) & ((1u << F.man_bits) - 1));
    return (uint8_t)((sign << 7) | man8);
  }
  int max_exp = (1 << F.exp_bits) - 1;
  if (exp8_raw >= max_exp) return (uint8_t)((sign << 7) | F.sat);
  uint8_t man8 = (uint8_t)((man32 >> man_shift) & ((1u << F.man_bits) - 1));
  return (uint8_t)((sign << 7) | ((uint8_t)exp8_raw << F.man_bits) | man8);
}

// Fp8Codec::fp8_to_fp32 — fp8.rs:210-261.  `leading` is always 0 in the
// reference (leading_zeros of a u32 clipped to man_bits-1), so subnormal codes
// decode as 2^(1-bias) * (1 + m/2^mb).
float fp8_decode_ref(uint8_t b, const Fp8Fmt& F) {
  uint32_t sign = b >> 7;
  uint32_t exp8 = (b >> F.man_bits) & ((1u << F.exp_bits) - 1);
  uint32_t man8 = b & ((1u << F.man_bits) - 1);
  uint32_t all_exp = (1u << F.exp_bits) - 1;
  if (F.exp_bits == 4) {
    if (exp8 == all_exp && man8 == (1u << F.man_bits) - 1) return std::numeric_limits<float>::quiet_NaN();
  } else if (exp8 == all_exp) {
    if (man8 == 0) return sign ? -INFINITY : INFINITY;
    return std::numeric_limits<float>::quiet_NaN();
  }
  uint32_t man_shift = 23 - F.man_bits;
  if (exp8 == 0) {
    if (man8 == 0) return u2f(sign << 31);
    uint32_t exp32 = (uint32_t)(127 + 1 - F.bias);
    uint32_t lz = (uint32_t)__builtin_clz(man8);           // u32::leading_zeros
    uint32_t leading = (uint32_t)F.man_bits - 1 - std::min<uint32_t>(lz, F.man_bits - 1);
    uint32_t exp32_adj = exp32 - leading;
    uint32_t m32 = ((man8 << leading) & ((1u << F.man_bits) - 1)) << man_shift;
    return u2f((sign << 31) | (exp32_adj << 23) | m32);
  }
  uint32_t exp32 = (uint32_t)((int)exp8 - F.bias + 127);
  return u2f((sign << 31) | (exp32 << 23) | (man8 << man_shift));
}

// Round-to-nearest-even, saturate-to-finite encoder.  For E4M3 this equals the
// RNE model in crates/oxicuda-dnn/src/quantize/fp8_quantize.rs:925-974 and the
// hardware cvt.rn.satfinite.e4m3x2.f32 on finite inputs.
uint8_t fp8_encode_rne(float v, const Fp8Fmt& F) {
  uint32_t bits = f2u(v);
  uint8_t sign = (uint8_t)((bits >> 31) << 7);
  float a = std::fabs(v);
  if (std::isnan(v)) return (uint8_t)(sign | 0x7F);
  if (a >= F.max_val) return (uint8_t)(sign | F.sat);
  int min_exp = 1 - F.bias;                         // exponent of the smallest normal
  float step_sub = std::ldexp(1.0f, min_exp - F.man_bits);
  if (a < std::ldexp(1.0f, min_exp)) {
    // subnormal: round a/step to nearest even integer
    float q = a / step_sub;                         // exact (power of two)
    float r = std::nearbyint(q);                    // default mode = RNE
    uint32_t m = (uint32_t)r;                       // 0..2^mb (2^mb == smallest normal code)
    return (uint8_t)(sign | m);
  }
  int e; float fr = std::frexp(a, &e);              // a = fr*2^e, fr in [0.5,1)
  (void)fr;
  int eu = e - 1;                                   // unbiased exponent
  float ulp = std::ldexp(1.0f, eu - F.man_bits);
  float q = a / ulp;                                // in [2^mb, 2^(mb+1)), exact
  uint32_t m = (uint32_t)std::nearbyint(q);
  if (m == (2u << F.man_bits)) { m >>= 1; eu += 1; }
  uint32_t code = ((uint32_t)(eu + F.bias) << F.man_bits) | (m & ((1u << F.man_bits) - 1));
  if (code > F.sat) code = F.sat;
  return (uint8_t)(sign | code);
}

// IEEE-style decode (true subnormals m * 2^(1-bias-mb)); what the tensor core sees.
float fp8_decode_ieee(uint8_t b, const Fp8Fmt& F) {
  uint32_t sign = b >> 7;
  uint32_t exp8 = (b >> F.man_bits) & ((1u << F.exp_bits) - 1);
  uint32_t man8 = b & ((1u << F.man_bits) - 1);
  uint32_t all_exp = (1u << F.exp_bits) - 1;
  float s = sign ? -1.0f : 1.0f;
  if (F.exp_bits == 4) {
    if (exp8 == all_exp && man8 == 7) return std::numeric_limits<float>::quiet_NaN();
  } else if (exp8 == all_exp) {
    if (man8 == 0) return sign ? -INFINITY : INFINITY;
    return std::numeric_limits<float>::quiet_NaN();
  }
  if (exp8 == 0) return s * std::ldexp((float)man8, 1 - F.bias - F.man_bits);
  return s * std::ldexp(1.0f + (float)man8 / (float)(1u << F.man_bits), (int)exp8 - F.bias);
}

// ---------------------------------------------------------------------------
// E2M1 (FP4)
// ---------------------------------------------------------------------------
// Fp4Quantizer::quantize_one (E2M1) — crates/oxicuda-blas/src/precision/fp4_fp6_ops.rs:638-663.
// The reference computes floor(log2(a)); only the thresholds 0.5, 1, 2, 4 change
// the biased exponent, and on them the IEEE exponent of `a` gives the same
// answer as a correctly rounded log2, so the exponent is extracted from the bits.
uint8_t e2m1_encode_ref(float value) {
  if (value == 0.0f) return 0;                      // -0.0 also returns 0 (sign lost)
  uint8_t sign = value < 0.0f ? 1 : 0;
  float a = rmin(std::fabs(value), 6.0f);           // NaN.min(6) == 6
  int eu;
  {
    uint32_t u = f2u(a);
    int e = (int)((u >> 23) & 0xFF);
    eu = e == 0 ? -127 : e - 127;                   // subnormal f32: far below 0.5 anyway
  }
  int eb = std::min(3, std::max(0, eu + 1));
  int ea = eb - 1;
  float sig = a / std::ldexp(1.0f, ea);
  uint8_t m = ((sig - 1.0f) >= 0.5f) ? 1 : 0;
  return (uint8_t)((sign << 3) | ((uint8_t)eb << 1) | m);
}
// Fp4Quantizer::quantize_one (Int4) — fp4_fp6_ops.rs:641-644.
uint8_t int4_encode_ref(float value) {
  float c = rclamp(std::round(value), -8.0f, 7.0f);
  int8_t q = f32_as_i8(c);
  return (uint8_t)q & 0x0F;
}
// Fp4Quantizer::dequantize_one — fp4_fp6_ops.rs:667-699.
float e2m1_decode_ref(uint8_t raw) {
  uint8_t sign = (raw >> 3) & 1, exponent = (raw >> 1) & 3, mant = raw & 1;
  if (exponent == 0 && mant == 0) return sign ? -0.0f : 0.0f;
  float v = exponent == 0 ? (float)mant * 0.5f
                          : (1.0f + (float)mant * 0.5f) * std::ldexp(1.0f, (int)exponent - 1);
  return sign ? -v : v;
}
float int4_decode_ref(uint8_t raw) {
  uint8_t nib = raw & 0x0F;
  return (nib & 8) ? (float)(int8_t)(0xF0u | nib) : (float)nib;
}

// E8M0 scale rule (NOT in the reference — parity unpinned): the smallest power
// of two that is >= absmax/6, exponent clamped to [-127,127], stored biased by
// 127; an all-zero block stores exponent 0 (scale 1.0).
uint8_t e8m0_from_absmax(float absmax) {
  if (!(absmax > 0.0f)) return 127;
  float s = absmax / 6.0f;
  int e; float fr = std::frexp(s, &e);              // s = fr * 2^e, fr in [0.5,1)
  int p = (fr == 0.5f) ? e - 1 : e;                 // ceil(log2 s)
  p = std::min(127, std::max(-127, p));
  return (uint8_t)(p + 127);
}
inline float e8m0_to_f32(uint8_t b) { return std::ldexp(1.0f, (int)b - 127); }

// NF4 — crates/oxicuda-quant/src/scheme/nf4.rs:33-50 (table), :181-203 (search).
const float NF4_LUT[16] = {
  -1.0f, -0.69619286f, -0.52507305f, -0.3949175f, -0.28444138f, -0.18477343f, -0.09105003f, 0.0f,
  0.0795803f, 0.1609302f, 0.2461123f, 0.33791524f, 0.44070983f, 0.562617f, 0.72295684f, 1.0f};
int nearest_nf4(float v) {
  int lo = 0, hi = 16;
  while (lo < hi) { int mid = lo + (hi - lo) / 2; if (NF4_LUT[mid] < v) lo = mid + 1; else hi = mid; }
  if (lo == 0) return 0;
  if (lo == 16) return 15;
  float d_lo = std::fabs(v - NF4_LUT[lo - 1]);
  float d_hi = std::fabs(NF4_LUT[lo] - v);
  return d_lo <= d_hi ? lo - 1 : lo;
}

}  // namespace

extern "C" {

int orc_num_threads() {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}
void orc_set_threads(int n) {
#ifdef _OPENMP
  omp_set_num_threads(n);
#else
  (void)n;
#endif
}

// ---------------------------------------------------------------------------
// MinMaxQuantizer — crates/oxicuda-quant/src/scheme/minmax.rs
// ---------------------------------------------------------------------------
// calibrate_slice (:209-243) applied to each of `rows` contiguous slices of
// `cols` elements (rows=1: per-tensor `calibrate`; rows=n/group: PerGroup
// `calibrate` :146-165; rows=channels: `calibrate_2d` :179-207).
// scheme: 0 symmetric, 1 asymmetric.  Returns 0, or 1+row of the first slice
// whose scale is not finite/positive (QuantError::InvalidScale).
int orc_minmax_calibrate(const float* x, int64_t rows, int64_t cols, int bits, int scheme,
                         float* scales, int32_t* zps) {
  for (int64_t r = 0; r < rows; ++r) {
    const float* s = x + r * cols;
    float fmin = INFINITY, fmax = -INFINITY;
    for (int64_t i = 0; i < cols; ++i) { float v = s[i]; if (v < fmin) fmin = v; if (v > fmax) fmax = v; }
    float scale; int32_t zp;
    if (scheme == 0) {
      float q_max = (float)(1 << (bits - 1)) - 1.0f;
      float abs_max = rmax(rmax(std::fabs(fmin), std::fabs(fmax)), 1e-8f);
      scale = abs_max / q_max; zp = 0;
    } else {
      float q_range = (float)((1 << bits) - 1);
      float range = rmax(fmax - fmin, 1e-8f);
      scale = range / q_range;
      zp = f32_as_i32(rclamp(std::round(-fmin / scale), 0.0f, q_range));
    }
    if (!std::isfinite(scale) || scale <= 0.0f) return (int)(1 + r);
    scales[r] = scale; zps[r] = zp;
  }
  return 0;
}

// quantize (:252-268) / quantize_grouped (:275-299): row r uses scales[r], zps[r].
void orc_minmax_quantize(const float* x, int64_t rows, int64_t cols, const float* scales,
                         const int32_t* zps, int bits, int scheme, int32_t* codes) {
  float q_max = scheme == 0 ? (float)(1 << (bits - 1)) - 1.0f : (float)(1 << bits) - 1.0f;
  float q_min = scheme == 0 ? -(float)(1 << (bits - 1)) : 0.0f;
  for (int64_t r = 0; r < rows; ++r) {
    float scale = scales[r], zp = (float)zps[r];
    for (int64_t i = 0; i < cols; ++i) {
      float xq = rclamp(std::round(x[r * cols + i] / scale + zp), q_min, q_max);
      codes[r * cols + i] = f32_as_i32(xq);
    }
  }
}

// dequantize (:302-306) / dequantize_grouped (:309-324).
void orc_minmax_dequantize(const int32_t* codes, int64_t rows, int64_t cols, const float* scales,
                           const int32_t* zps, float* out) {
  for (int64_t r = 0; r < rows; ++r)
    for (int64_t i = 0; i < cols; ++i)
      out[r * cols + i] = (float)(int32_t)((uint32_t)codes[r * cols + i] - (uint32_t)zps[r]) * scales[r];
}

// FakeQuantize::forward — crates/oxicuda-quant/src/qat/fake_quant.rs:118-133
// (the CPU oracle of the fake_quant PTX kernel, ptx_kernels.rs:55-121).
void orc_fake_quant(const float* x, int64_t n, float scale, float zp, float qmin, float qmax, float* out) {
  for (int64_t i = 0; i < n; ++i) {
    float q = rclamp(std::round(x[i] / scale + zp), qmin, qmax);
    out[i] = (q - zp) * scale;
  }
}

// ---------------------------------------------------------------------------
// Fp8Codec — crates/oxicuda-quant/src/scheme/fp8.rs
// ---------------------------------------------------------------------------
// encode (:135-137) -> encode_f32 (:115-122).  fmt: 0 E4M3, 1 E5M2.
// mode: 0 = reference codec (truncating), 1 = RNE/saturating (hardware).
// Returns -1, or the index of the first non-finite input (NonFiniteFp8).
int64_t orc_fp8_encode(const float* x, int64_t n, int fmt, int mode, uint8_t* out) {
  const Fp8Fmt& F = fmt_of(fmt);
  for (int64_t i = 0; i < n; ++i) {
    float v = x[i];
    if (!std::isfinite(v)) return i;
    float vs = rclamp(v, -F.max_val, F.max_val);
    out[i] = mode == 0 ? fp8_encode_ref(vs, F) : fp8_encode_rne(vs, F);
  }
  return -1;
}
// decode (:140-142).  mode 0 = reference decode, 1 = IEEE decode.
void orc_fp8_decode(const uint8_t* codes, int64_t n, int fmt, int mode, float* out) {
  const Fp8Fmt& F = fmt_of(fmt);
  for (int64_t i = 0; i < n; ++i) out[i] = mode == 0 ? fp8_decode_ref(codes[i], F) : fp8_decode_ieee(codes[i], F);
}

// Absmax-scaled FP8 quantization of `rows` slices of `cols` elements:
// scale = absmax/max_val (1.0 when the slice is all zero), code = encode(x/scale).
// Composition of the scale rule of crates/oxicuda-dnn/src/quantize/fp8_quantize.rs:28-34,
// :591-596 (div.rn then clamp) with the Fp8Codec above.  rows=1 is per-tensor.
int64_t orc_fp8_quantize_rows(const float* x, int64_t rows, int64_t cols, int fmt, int mode,
                              float* scales, uint8_t* codes) {
  const Fp8Fmt& F = fmt_of(fmt);
  for (int64_t r = 0; r < rows; ++r) {
    const float* s = x + r * cols;
    float amax = 0.0f;
    for (int64_t i = 0; i < cols; ++i) { if (!std::isfinite(s[i])) return r * cols + i; amax = rmax(amax, std::fabs(s[i])); }
    float scale = amax > 0.0f ? amax / F.max_val : 1.0f;
    scales[r] = scale;
    for (int64_t i = 0; i < cols; ++i) {
      float vs = rclamp(s[i] / scale, -F.max_val, F.max_val);
      codes[r * cols + i] = mode == 0 ? fp8_encode_ref(vs, F) : fp8_encode_rne(vs, F);
    }
  }
  return -1;
}

// ---------------------------------------------------------------------------
// FP4 / micro-scaling — crates/oxicuda-blas/src/precision/fp4_fp6_ops.rs
// ---------------------------------------------------------------------------
uint8_t orc_fp4_quantize_one(float v, int format) { return format == 0 ? e2m1_encode_ref(v) : int4_encode_ref(v); }
float orc_fp4_dequantize_one(uint8_t raw, int format) { return format == 0 ? e2m1_decode_ref(raw) : int4_decode_ref(raw); }
uint8_t orc_e8m0_from_absmax(float a) { return e8m0_from_absmax(a); }

// Fp4Quantizer::quantize (:708-723) + PackedFp4::pack (:465-472): n must be even;
// element 2i goes to the low nibble of byte i.
void orc_fp4_quantize(const float* x, int64_t n, int format, uint8_t* packed) {
  for (int64_t i = 0; i < n / 2; ++i) {
    uint8_t v0 = orc_fp4_quantize_one(x[2 * i], format), v1 = orc_fp4_quantize_one(x[2 * i + 1], format);
    packed[i] = (uint8_t)(v0 | (v1 << 4));
  }
}
void orc_fp4_dequantize(const uint8_t* packed, int64_t nbytes, int format, float* out) {
  for (int64_t i = 0; i < nbytes; ++i) {
    out[2 * i] = orc_fp4_dequantize_one(packed[i] & 0x0F, format);
    out[2 * i + 1] = orc_fp4_dequantize_one((packed[i] >> 4) & 0x0F, format);
  }
}

// MicroScalingQuantizer::compute_scales (:763-782) + quantize_fp4 (:849-876).
// Blocks of `block` run over the flat array; the last block may be short; an odd
// length is padded with one 0.0.  scale_mode 0: f32 scale absmax/target_max
// (reference); scale_mode 1: E8M0 byte (parity unpinned, see e8m0_from_absmax).
// `scales_f32` receives ceil(n/block) floats (mode 0) and/or `scales_e8m0`
// ceil(n/block) bytes (mode 1).  packed receives ceil(n/2) bytes.
void orc_fp4_block_quantize(const float* x, int64_t n, int block, int format, int scale_mode,
                            uint8_t* packed, float* scales_f32, uint8_t* scales_e8m0) {
  float target_max = format == 0 ? 6.0f : 8.0f;
  int64_t nb = (n + block - 1) / block;
  int64_t nbytes = (n + 1) / 2;
  std::memset(packed, 0, (size_t)nbytes);
#pragma omp parallel for schedule(static)
  for (int64_t b = 0; b < nb; ++b) {
    int64_t s = b * block, e = std::min<int64_t>(s + block, n);
    float amax = 0.0f;
    for (int64_t i = s; i < e; ++i) amax = rmax(amax, std::fabs(x[i]));
    float scale;
    if (scale_mode == 0) {
      scale = amax == 0.0f ? 1.0f : amax / target_max;
      scales_f32[b] = scale;
    } else {
      uint8_t eb = e8m0_from_absmax(amax);
      scales_e8m0[b] = eb;
      scale = e8m0_to_f32(eb);
    }
    for (int64_t i = s; i < e; ++i) {
      uint8_t c = orc_fp4_quantize_one(x[i] / scale, format);
      // block is even, so two elements of one byte never belong to different threads
      if (i & 1) packed[i >> 1] |= (uint8_t)(c << 4); else packed[i >> 1] |= c;
    }
  }
}

// dequantize_fp4 (:879-897): decode(code) * scale[i / block].
void orc_fp4_block_dequantize(const uint8_t* packed, int64_t n, int block, int format, int scale_mode,
                              const float* scales_f32, const uint8_t* scales_e8m0, float* out) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i) {
    uint8_t byte = packed[i >> 1];
    uint8_t raw = (i & 1) ? (byte >> 4) & 0x0F : byte & 0x0F;
    float scale = scale_mode == 0 ? scales_f32[i / block] : e8m0_to_f32(scales_e8m0[i / block]);
    out[i] = orc_fp4_dequantize_one(raw, format) * scale;
  }
}

// ---------------------------------------------------------------------------
// NF4 — crates/oxicuda-quant/src/scheme/nf4.rs:93-150
// ---------------------------------------------------------------------------
void orc_nf4_encode(const float* x, int64_t n, int block, uint8_t* packed, float* absmaxs) {
  std::memset(packed, 0, (size_t)(n / 2));
  for (int64_t b = 0; b < n / block; ++b) {
    const float* s = x + b * block;
    float amax = 0.0f;
    for (int i = 0; i < block; ++i) amax = rmax(amax, std::fabs(s[i]));
    if (amax < 1e-8f) amax = 1e-8f;
    absmaxs[b] = amax;
    int64_t base = b * block / 2;
    for (int i = 0; i < block; ++i) {
      float normed = rclamp(s[i] / amax, -1.0f, 1.0f);
      uint8_t code = (uint8_t)nearest_nf4(normed);
      if (i % 2 == 0) packed[base + i / 2] = code; else packed[base + i / 2] |= (uint8_t)(code << 4);
    }
  }
}
void orc_nf4_decode(const uint8_t* packed, int64_t nbytes, int block, const float* absmaxs, float* out) {
  for (int64_t i = 0; i < nbytes; ++i) {
    float amax = absmaxs[(2 * i) / block];
    out[2 * i] = NF4_LUT[packed[i] & 0x0F] * amax;
    out[2 * i + 1] = NF4_LUT[packed[i] >> 4] * amax;
  }
}

// ---------------------------------------------------------------------------
// dist-infer "FP8" (INT8 in a u8) — crates/oxicuda-dist-infer/src/quantisation/fp8_infer.rs:61-142
// ---------------------------------------------------------------------------
// quantize_fp8_block: per-block absmax is STORED (not a scale); block >= n is per-tensor.
void orc_distfp8_quantize_block(const float* x, int64_t n, int64_t block, uint8_t* q, float* absmaxs) {
  if (block < 1) block = 1;
  for (int64_t s = 0, b = 0; s < n; s += block, ++b) {
    int64_t e = std::min(s + block, n);
    float amax = 0.0f;
    for (int64_t i = s; i < e; ++i) amax = rmax(amax, std::fabs(x[i]));
    absmaxs[b] = amax;
    if (amax == 0.0f) { for (int64_t i = s; i < e; ++i) q[i] = 0; continue; }
    float scale = 127.0f / amax;
    for (int64_t i = s; i < e; ++i) q[i] = (uint8_t)f32_as_i8(std::round(rclamp(x[i] * scale, -127.0f, 127.0f)));
  }
}
void orc_distfp8_dequantize_block(const uint8_t* q, int64_t n, int64_t block, const float* absmaxs, float* out) {
  if (block < 1) block = 1;
  for (int64_t i = 0; i < n; ++i) out[i] = (float)(int8_t)q[i] * (absmaxs[i / block] / 127.0f);
}

// ---------------------------------------------------------------------------
// LLM.int8 — crates/oxicuda-quant/src/scheme/llm_int8.rs:175-288
// ---------------------------------------------------------------------------
// x [samples x cols], w [rows x cols] row-major -> out [samples x rows].
// Optional dumps (may be null): wq [rows x cols] i8, sw [rows], xq [samples x cols] i8,
// sx [samples], acc [samples x rows] i32 (the integer accumulator, exact),
// outlier [cols] u8.  Returns the number of outlier columns.
int64_t orc_llm_int8_matmul(const float* x, const float* w, int64_t samples, int64_t rows, int64_t cols,
                            float threshold, int row_wise, float* out,
                            int8_t* wq_out, float* sw_out, int8_t* xq_out, float* sx_out,
                            int32_t* acc_out, uint8_t* outlier_out) {
  // detect_outliers (:128-157)
  std::vector<float> col_max((size_t)cols, 0.0f);
  for (int64_t r = 0; r < samples; ++r)
    for (int64_t c = 0; c < cols; ++c) { float a = std::fabs(x[r * cols + c]); if (a > col_max[c]) col_max[c] = a; }
  std::vector<uint8_t> is_out((size_t)cols, 0);
  int64_t n_out = 0;
  for (int64_t c = 0; c < cols; ++c) if (col_max[c] >= threshold) { is_out[c] = 1; ++n_out; }
  if (outlier_out) std::memcpy(outlier_out, is_out.data(), (size_t)cols);

  // per-weight-row scales and codes (:207-229)
  std::vector<float> sw((size_t)rows);
  std::vector<int8_t> wq((size_t)(rows * cols), 0);
#pragma omp parallel for schedule(static)
  for (int64_t k = 0; k < rows; ++k) {
    float amax = 0.0f;
    for (int64_t c = 0; c < cols; ++c) if (!is_out[c]) amax = rmax(amax, std::fabs(w[k * cols + c]));
    sw[k] = amax > 0.0f ? amax / 127.0f : 1.0f;
    float inv = 1.0f / sw[k];
    for (int64_t c = 0; c < cols; ++c)
      if (!is_out[c]) wq[k * cols + c] = f32_as_i8(rclamp(std::round(w[k * cols + c] * inv), -127.0f, 127.0f));
  }
  if (sw_out) std::memcpy(sw_out, sw.data(), sizeof(float) * (size_t)rows);
  if (wq_out) std::memcpy(wq_out, wq.data(), (size_t)(rows * cols));

  float sx_global = 1.0f;
  if (!row_wise) {                                  // (:247-257)
    float amax = 0.0f;
    for (int64_t i = 0; i < samples * cols; ++i) if (!is_out[i % cols]) amax = rmax(amax, std::fabs(x[i]));
    sx_global = amax > 0.0f ? amax / 127.0f : 1.0f;
  }
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < samples; ++r) {
    const float* xr = x + r * cols;
    float sx;
    if (row_wise) {
      float amax = 0.0f;
      for (int64_t c = 0; c < cols; ++c) if (!is_out[c]) amax = rmax(amax, std::fabs(xr[c]));
      sx = amax > 0.0f ? amax / 127.0f : 1.0f;
    } else sx = sx_global;
    float inv_sx = 1.0f / sx;
    std::vector<int32_t> xq((size_t)cols, 0);
    for (int64_t c = 0; c < cols; ++c)
      if (!is_out[c]) xq[c] = f32_as_i32(rclamp(std::round(xr[c] * inv_sx), -127.0f, 127.0f));
    if (sx_out) sx_out[r] = sx;
    if (xq_out) for (int64_t c = 0; c < cols; ++c) xq_out[r * cols + c] = (int8_t)xq[c];
    for (int64_t k = 0; k < rows; ++k) {
      int64_t acc_int = 0; float acc_fp = 0.0f;
      for (int64_t c = 0; c < cols; ++c) {
        if (is_out[c]) acc_fp += xr[c] * w[k * cols + c];
        else acc_int += (int64_t)xq[c] * (int64_t)wq[k * cols + c];
      }
      if (acc_out) acc_out[r * rows + k] = (int32_t)acc_int;
      out[r * rows + k] = (float)acc_int * (sx * sw[k]) + acc_fp;
    }
  }
  return n_out;
}

// Exact INT8 GEMM with s32 accumulation: C[m,n] = sum_k A[m,k]*B[n,k].
// Semantics of generate_int8_gemm_ptx (crates/oxicuda-blas/src/precision/int_ops.rs:446-583):
// dp4a.s32.s32 over K, AccType::I32 store.  B is given here as [N x K] row-major
// (weight layout); the reference kernel's K-packed [K/4 x N] u32 operand holds the same values.
void orc_gemm_i8(const int8_t* a, const int8_t* b, int64_t M, int64_t N, int64_t K, int32_t* c) {
#pragma omp parallel for schedule(static) collapse(2)
  for (int64_t m = 0; m < M; ++m)
    for (int64_t n = 0; n < N; ++n) {
      int32_t acc = 0;
      for (int64_t k = 0; k < K; ++k) acc += (int32_t)a[m * K + k] * (int32_t)b[n * K + k];
      c[m * N + n] = acc;
    }
}

// ---------------------------------------------------------------------------
// FP8 GEMM composition (parity unpinned by any reference test: the reference's
// only complete GEMM generator rejects FP8, crates/oxicuda-ptx/src/templates/gemm.rs:800-809).
// Defined as: decode codes (Fp8Codec decode, or IEEE decode), then the arithmetic
// order of the reference's naive kernel (gemm.rs:373-447): k-ascending fma.rn.f32,
// acc*alpha, then scale, stored as bf16 (RNE) or f32.
// a [M x K] codes, w [N x K] codes ("out x in" weights).  sa: 1 or M floats
// (sa_rows = 0/1); sw: 1 or N floats.  out = acc * (sa * sw).
// ---------------------------------------------------------------------------
void orc_gemm_fp8(const uint8_t* a, const uint8_t* w, int64_t M, int64_t N, int64_t K, int fmt, int decode_mode,
                  const float* sa, int sa_rows, const float* sw, int sw_rows,
                  uint16_t* out_bf16, float* out_f32) {
  const Fp8Fmt& F = fmt_of(fmt);
  float lut[256];
  for (int i = 0; i < 256; ++i) lut[i] = decode_mode == 0 ? fp8_decode_ref((uint8_t)i, F) : fp8_decode_ieee((uint8_t)i, F);
  std::vector<float> af((size_t)(M * K)), wf((size_t)(N * K));
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < M * K; ++i) af[i] = lut[a[i]];
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < N * K; ++i) wf[i] = lut[w[i]];
#pragma omp parallel for schedule(static)
  for (int64_t m = 0; m < M; ++m) {
    const float* ar = af.data() + m * K;
    for (int64_t n = 0; n < N; ++n) {
      const float* wr = wf.data() + n * K;
      float acc = 0.0f;
      for (int64_t k = 0; k < K; ++k) acc = std::fmaf(ar[k], wr[k], acc);
      float s = (sa_rows ? sa[m] : sa[0]) * (sw_rows ? sw[n] : sw[0]);
      float v = acc * s;
      if (out_bf16) out_bf16[m * N + n] = f32_to_bf16_rne(v);
      if (out_f32) out_f32[m * N + n] = v;
    }
  }
}

// ---------------------------------------------------------------------------
// FP4 weight-only GEMV/GEMM composition: dequantize_fp4 (fp4_fp6_ops.rs:879-897)
// then an f32 dot product, k ascending, against bf16 activations widened to f32.
// The reference's own FP4 GEMM kernel text (fp4_fp6_ops.rs:1237-1362) is never
// launched and decodes nibbles as INT4, so the defined semantics are this
// composition (parity unpinned).
// codes [N x K/2], scales [N x K/block], x [M x K] bf16 -> out [M x N].
// ---------------------------------------------------------------------------
void orc_gemv_fp4(const uint8_t* codes, int scale_mode, const float* scales_f32, const uint8_t* scales_e8m0,
                  int block, const uint16_t* x_bf16, int64_t M, int64_t N, int64_t K,
                  uint16_t* out_bf16, float* out_f32) {
  std::vector<float> xf((size_t)(M * K));
  for (int64_t i = 0; i < M * K; ++i) xf[i] = bf16_to_f32(x_bf16[i]);
#pragma omp parallel
  {
    std::vector<float> wrow((size_t)K);
#pragma omp for schedule(static)
    for (int64_t n = 0; n < N; ++n) {
      for (int64_t k = 0; k < K; ++k) {
        uint8_t byte = codes[(n * K + k) >> 1];
        uint8_t raw = (k & 1) ? (byte >> 4) & 0x0F : byte & 0x0F;
        int64_t bi = (n * K + k) / block;
        float scale = scale_mode == 0 ? scales_f32[bi] : e8m0_to_f32(scales_e8m0[bi]);
        wrow[k] = e2m1_decode_ref(raw) * scale;
      }
      for (int64_t m = 0; m < M; ++m) {
        float acc = 0.0f;
        const float* xr = xf.data() + m * K;
        for (int64_t k = 0; k < K; ++k) acc += xr[k] * wrow[k];
        if (out_bf16) out_bf16[m * N + n] = f32_to_bf16_rne(acc);
        if (out_f32) out_f32[m * N + n] = acc;
      }
    }
  }
}

// ---------------------------------------------------------------------------
// Tensor-parallel linears — crates/oxicuda-dist-infer/src/tensor_parallel
// ---------------------------------------------------------------------------
// ColumnLinear: shard r owns rows [r*out/tp, (r+1)*out/tp) of W[out x in]
// (column_parallel.rs:115-166); forward acc = bias; acc += x*w, k ascending, unfused
// (:77-95); all_gather places shard r at columns [r*out/tp, ...) (:181-204).
// bias may be null (zeros).  Returns the gathered [batch x out].
void orc_column_linear(const float* x, const float* w, const float* bias, int64_t batch, int64_t in_f,
                       int64_t out_f, int tp, float* out) {
  int64_t local_out = out_f / tp;
  for (int r = 0; r < tp; ++r) {
#pragma omp parallel for schedule(static)
    for (int64_t b = 0; b < batch; ++b)
      for (int64_t o = 0; o < local_out; ++o) {
        int64_t row = r * local_out + o;
        float acc = bias ? bias[row] : 0.0f;
        for (int64_t i = 0; i < in_f; ++i) acc += x[b * in_f + i] * w[row * in_f + i];
        out[b * out_f + row] = acc;
      }
  }
}
// RowLinear: shard r owns columns [r*in/tp, ...) of every row (row_parallel.rs:109-168);
// forward_partial acc=0; acc += x_s*w_s; bias added on rank 0 only (:67-89);
// all_reduce sums the partials in rank order 0,1,... (:202-223).
void orc_row_linear(const float* x, const float* w, const float* bias, int64_t batch, int64_t in_f,
                    int64_t out_f, int tp, float* out) {
  int64_t local_in = in_f / tp;
#pragma omp parallel for schedule(static)
  for (int64_t b = 0; b < batch; ++b)
    for (int64_t o = 0; o < out_f; ++o) {
      float total = 0.0f;
      for (int r = 0; r < tp; ++r) {
        float acc = 0.0f;
        for (int64_t i = 0; i < local_in; ++i) acc += x[b * in_f + r * local_in + i] * w[o * in_f + r * local_in + i];
        if (r == 0 && bias) acc += bias[o];
        total = r == 0 ? acc : total + acc;
      }
      out[b * out_f + o] = total;
    }
}
// silu — crates/oxicuda-lm/src/layer/ffn.rs:25-27: x / (1 + exp(-x)).
void orc_swiglu(const float* gate, const float* up, int64_t n, float* h) {
  for (int64_t i = 0; i < n; ++i) h[i] = (gate[i] / (1.0f + std::exp(-gate[i]))) * up[i];
}

// ---------------------------------------------------------------------------
// KvCacheQuantizer — crates/oxicuda-quant/src/scheme/kv_cache.rs
// ---------------------------------------------------------------------------
// quantize (:146-221): asymmetric affine codes in [0, 2^bits-1] with one (scale, min) per group;
// axis 0 = KvAxis::PerToken (one group per row), 1 = KvAxis::PerChannel (one group per column).
// append_token (:254-282) is the per-token rule on a single row, so it is this function with n_tokens = 1.
void orc_kv_cache_quantize(const float* x, int64_t n_tokens, int64_t head_dim, int bits, int axis,
                           uint8_t* codes, float* scales, float* zero_points) {
  const float q_max = (float)((1u << bits) - 1u);
  const int64_t n_groups = axis == 0 ? n_tokens : head_dim;
  std::vector<float> gmin((size_t)n_groups, INFINITY), gmax((size_t)n_groups, -INFINITY);
  for (int64_t t = 0; t < n_tokens; ++t)
    for (int64_t c = 0; c < head_dim; ++c) {
      const float v = x[t * head_dim + c];
      const int64_t g = axis == 0 ? t : c;
      if (v < gmin[g]) gmin[g] = v;
      if (v > gmax[g]) gmax[g] = v;
    }
  for (int64_t g = 0; g < n_groups; ++g) {
    const float range = rmax(gmax[g] - gmin[g], 1e-8f);
    scales[g] = range / q_max;
    zero_points[g] = gmin[g];
  }
  for (int64_t t = 0; t < n_tokens; ++t)
    for (int64_t c = 0; c < head_dim; ++c) {
      const int64_t g = axis == 0 ? t : c;
      const float q = rclamp(std::round((x[t * head_dim + c] - zero_points[g]) / scales[g]), 0.0f, q_max);
      codes[t * head_dim + c] = (uint8_t)f32_as_i32(q != q ? 0.0f : q);   // `NaN as u8` is 0; q is already within [0, 255]
    }
}
// dequantize (:224-238): q * scale + zero_point, unfused.
void orc_kv_cache_dequantize(const uint8_t* codes, int64_t n_tokens, int64_t head_dim, int axis,
                             const float* scales, const float* zero_points, float* out) {
  for (int64_t t = 0; t < n_tokens; ++t)
    for (int64_t c = 0; c < head_dim; ++c) {
      const int64_t g = axis == 0 ? t : c;
      out[t * head_dim + c] = (float)codes[t * head_dim + c] * scales[g] + zero_points[g];
    }
}

// quantize_token — crates/oxicuda-infer/src/cache/kv_quant.rs:112-154, applied to each of `n_tokens` rows of `d`
// channels.  q_range (:69-76): symmetric [-(2^(bits-1)-1), 2^(bits-1)-1], asymmetric [0, 2^bits-1].
void orc_kv_quantize_tokens(const float* x, int64_t n_tokens, int64_t d, int bits, int symmetric,
                            int32_t* codes, float* scales, float* zero_points) {
  const int32_t qmin = symmetric ? -((1 << (bits - 1)) - 1) : 0;
  const int32_t qmax = symmetric ? (1 << (bits - 1)) - 1 : (1 << bits) - 1;
  const float qmin_f = (float)qmin, qmax_f = (float)qmax;
  for (int64_t t = 0; t < n_tokens; ++t) {
    const float* row = x + t * d;
    float x_min = INFINITY, x_max = -INFINITY;
    for (int64_t i = 0; i < d; ++i) { x_min = rmin(x_min, row[i]); x_max = rmax(x_max, row[i]); }
    float scale, zp;
    if (symmetric) {
      const float amax = rmax(std::fabs(x_min), std::fabs(x_max));
      scale = amax > 0.0f ? amax / qmax_f : 1.0f;
      zp = 0.0f;
    } else {
      const float range = x_max - x_min;
      scale = range > 0.0f ? range / (qmax_f - qmin_f) : 1.0f;
      zp = x_min - qmin_f * scale;
    }
    for (int64_t i = 0; i < d; ++i) {
      const int32_t q = f32_as_i32(std::round((row[i] - zp) / scale));
      codes[t * d + i] = q < qmin ? qmin : (q > qmax ? qmax : q);
    }
    scales[t] = scale; zero_points[t] = zp;
  }
}
// QuantizedToken::dequantize (:94-100): scale * code + zero_point, unfused.
void orc_kv_dequantize_tokens(const int32_t* codes, int64_t n_tokens, int64_t d, const float* scales,
                              const float* zero_points, float* out) {
  for (int64_t t = 0; t < n_tokens; ++t)
    for (int64_t i = 0; i < d; ++i) out[t * d + i] = scales[t] * (float)codes[t * d + i] + zero_points[t];
}

// RMSNorm — crates/oxicuda-dnn/src/norm/rms_norm.rs:29-33 (definition), :566-574 (CPU statement of the same):
// y = x / sqrt(mean(x^2) + eps) * gamma per row, sequential f32 sum.  With `residual` non-null the fused form of
// fused_add_rms_norm (:98-103): residual += x first, and the norm is taken of the updated residual.
void orc_rms_norm(const float* x, float* residual, const float* gamma, int64_t rows, int64_t cols, float eps, float* y) {
  for (int64_t r = 0; r < rows; ++r) {
    const float* row = x + r * cols;
    if (residual) {
      float* res = residual + r * cols;
      for (int64_t i = 0; i < cols; ++i) res[i] = res[i] + row[i];
      row = res;
    }
    float sum = 0.0f;
    for (int64_t i = 0; i < cols; ++i) sum += row[i] * row[i];
    const float rms = std::sqrt(sum / (float)cols + eps);
    for (int64_t i = 0; i < cols; ++i) y[r * cols + i] = row[i] / rms * gamma[i];
  }
}

// ---------------------------------------------------------------------------
// oxicuda-dnn quantize — crates/oxicuda-dnn/src/quantize/{fp8_quantize,int8_quantize,block_scale}.rs, in the form the
// reference's GPU tests state them (crates/oxicuda-dnn/src/gpu_tests/quantize.rs).
// ---------------------------------------------------------------------------
// rne (gpu_tests/quantize.rs:47-60): round to nearest, ties to even; NaN comes back as NaN.
static float dnn_rne(float x) {
  const float f = std::floor(x), diff = x - f;
  if (diff < 0.5f) return f;
  if (diff > 0.5f) return f + 1.0f;
  // ties (and NaN, whose `f as i64` is 0): even stays
  const long long fi = std::isnan(f) ? 0 : (long long)f;
  return fi % 2 == 0 ? f : f + 1.0f;
}
// cpu_e4m3_encode (gpu_tests/quantize.rs:64-109): sign | 0x7E from 448 up (NaN included: its bits compare above), zero
// below 2^-20, otherwise ties-to-even onto the E4M3 grid, which is fp8_encode_rne for finite input.
static uint8_t dnn_e4m3_encode(float v) {
  const uint32_t bits = f2u(v);
  if ((bits & 0x7fffffffu) >= 0x43E00000u) return (uint8_t)(((bits >> 24) & 0x80u) | 0x7Eu);
  return fp8_encode_rne(v, Fp8Fmt{4, 3, 7, 448.0f, 0x7E});
}
// cpu_e4m3_decode (gpu_tests/quantize.rs:112-125)
static float dnn_e4m3_decode(uint8_t b) {
  const uint32_t e = (b >> 3) & 0xF, m = b & 7;
  const float sign = (b & 0x80) ? -1.0f : 1.0f;
  if (e == 0) return sign * (float)m * (1.0f / 512.0f);
  return sign * u2f(((e + 120u) << 23) | (m << 20));
}
static float dnn_absmax(const float* x, int64_t n) {
  float m = 0.0f;
  for (int64_t i = 0; i < n; ++i) m = rmax(m, std::fabs(x[i]));
  return m;
}
// quantize_to_fp8 (fp8_quantize.rs:45-122; checked at gpu_tests/quantize.rs:279-293)
void orc_dnn_quantize_to_fp8(const float* x, int64_t n, uint8_t* codes, float* scale) {
  if (n == 0) return;
  const float s = rmax(dnn_absmax(x, n) / 448.0f, 1e-12f);
  *scale = s;
  for (int64_t i = 0; i < n; ++i) codes[i] = dnn_e4m3_encode(rclamp(x[i] / s, -448.0f, 448.0f));
}
// dequantize_from_fp8 (fp8_quantize.rs:125-170; gpu_tests/quantize.rs:319-320)
void orc_dnn_dequantize_from_fp8(const uint8_t* codes, float scale, int64_t n, float* out) {
  for (int64_t i = 0; i < n; ++i) out[i] = dnn_e4m3_decode(codes[i]) * scale;
}
// quantize_to_int8 (int8_quantize.rs:31-102; gpu_tests/quantize.rs:206-219)
void orc_dnn_quantize_to_int8(const float* x, int64_t n, int8_t* q, float* scale) {
  if (n == 0) return;
  const float s = rmax(dnn_absmax(x, n) / 127.0f, 1e-12f);
  *scale = s;
  for (int64_t i = 0; i < n; ++i) q[i] = (int8_t)f32_as_i32(dnn_rne(rclamp(x[i] / s, -127.0f, 127.0f)));
}
void orc_dnn_dequantize_from_int8(const int8_t* q, float scale, int64_t n, float* out) {
  for (int64_t i = 0; i < n; ++i) out[i] = (float)q[i] * scale;
}
// quantize_block_scaled (block_scale.rs:51-150; gpu_tests/quantize.rs:527-553)
void orc_dnn_quantize_block_scaled(const float* x, int64_t n, int64_t block, uint8_t* out, float* scales) {
  for (int64_t b = 0; b * block < n; ++b) {
    const int64_t lo = b * block, hi = std::min(n, lo + block);
    const float s = rmax(dnn_absmax(x + lo, hi - lo) / 6.0f, 1e-12f);
    scales[b] = s;
    for (int64_t i = lo; i < hi; ++i) {
      const int32_t q = f32_as_i32(dnn_rne(rclamp(x[i] / s, -6.0f, 6.0f))) + 6;
      out[i] = (uint8_t)std::min(255, std::max(0, q));
    }
  }
}
// BlockQuantizedInt8::quantize / dequantize (int8_quantize.rs:427-470)
void orc_block_int8_quantize(const float* x, int64_t n, int64_t block, int8_t* q, float* scales) {
  for (int64_t b = 0; b * block < n; ++b) {
    const int64_t lo = b * block, hi = std::min(n, lo + block);
    const float m = dnn_absmax(x + lo, hi - lo);
    const float s = m > 0.0f ? m / 127.0f : 1.0f;
    scales[b] = s;
    for (int64_t i = lo; i < hi; ++i) q[i] = (int8_t)f32_as_i32(rclamp(std::round(x[i] / s), -128.0f, 127.0f));
  }
}
void orc_block_int8_dequantize(const int8_t* q, const float* scales, int64_t n, int64_t block, float* out) {
  for (int64_t i = 0; i < n; ++i) out[i] = (float)q[i] * scales[i / block];
}
// Fp4BlockQuantizer::compute_scale (block_scale.rs:437-444) for every block
void orc_block_absmax_scale(const float* x, int64_t n, int64_t block, float max_val, float* scales) {
  for (int64_t b = 0; b * block < n; ++b) {
    const float m = dnn_absmax(x + b * block, std::min(block, n - b * block));
    scales[b] = m == 0.0f ? 1.0f : m / max_val;
  }
}

// ---------------------------------------------------------------------------
// INT4 group-scaled weight-only GEMM — crates/oxicuda-blas/src/precision/int_ops.rs
// ---------------------------------------------------------------------------
// pack_int4 (:375-403): eight two's-complement nibbles per u32, value j in bits [4j, 4j+4).  Returns 0, 1 when the
// length is not a multiple of 8, or 2 + index of the first value outside [-8, 7].
int64_t orc_pack_int4(const int8_t* values, int64_t n, uint32_t* packed) {
  if (n % 8 != 0) return 1;
  for (int64_t i = 0; i < n; ++i) if (values[i] < -8 || values[i] > 7) return 2 + i;
  for (int64_t w = 0; w < n / 8; ++w) {
    uint32_t p = 0;
    for (int j = 0; j < 8; ++j) p |= (uint32_t)((uint8_t)values[w * 8 + j] & 0x0F) << (j * 4);
    packed[w] = p;
  }
  return 0;
}
// unpack_int4 (:415-429)
void orc_unpack_int4(const uint32_t* packed, int64_t words, int8_t* out) {
  for (int64_t w = 0; w < words; ++w)
    for (int j = 0; j < 8; ++j) {
      const uint8_t nib = (packed[w] >> (j * 4)) & 0x0F;
      out[w * 8 + j] = (nib & 0x08) ? (int8_t)(0xF0u | nib) : (int8_t)nib;
    }
}
static float f16_bits_to_f32(uint16_t h) {
  const uint32_t sign = (uint32_t)(h & 0x8000) << 16, e = (h >> 10) & 0x1F, m = h & 0x3FF;
  if (e == 0) return u2f(sign) * 0.0f + (sign ? -1.0f : 1.0f) * (float)m * 5.9604644775390625e-8f;   // m * 2^-24
  if (e == 31) return u2f(sign | 0x7F800000u | (m << 13));
  return u2f(sign | ((e + 112) << 23) | (m << 13));
}
// The kernel of generate_int4_gemm_ptx (:602-757): C[row, col] = sum over k ascending of
// fma(float(int4[row, k]) * f32(scale_f16[row, k / group]), B[k, col], acc); A packed [M x K/8] u32, scales f16
// [M x K/group], B f32 [K x N] row-major, C f32 [M x N].
void orc_gemm_int4(const uint32_t* a_packed, const uint16_t* scales_f16, const float* b, float* c, int64_t M, int64_t N,
                   int64_t K, int64_t group) {
  const int64_t groups = K / group, kw = K / 8;
#pragma omp parallel for schedule(static)
  for (int64_t row = 0; row < M; ++row)
    for (int64_t col = 0; col < N; ++col) {
      float acc = 0.0f;
      for (int64_t k = 0; k < K; k += 8) {
        const float scale = f16_bits_to_f32(scales_f16[row * groups + k / group]);
        const uint32_t w = a_packed[row * kw + k / 8];
        for (int j = 0; j < 8; ++j) {
          const uint32_t nib = (w >> (4 * j)) & 0xF;
          const int32_t v = (nib & 8) ? (int32_t)(nib | 0xFFFFFFF0u) : (int32_t)nib;
          const float dq = (float)v * scale;
          acc = std::fmaf(dq, b[(k + j) * N + col], acc);
        }
      }
      c[row * N + col] = acc;
    }
}

// ---------------------------------------------------------------------------
// Tile heuristics — crates/oxicuda-blas/src/precision/fp8_ops.rs:67-87 (classify),
// :239-304 (Blackwell table), :389-396 (split-K); fp4_fp6_ops.rs:996-1075;
// int_ops.rs:141-176.  Class ids: 0 SmallSquare, 1 LargeSquare, 2 SkinnyM,
// 3 SkinnyN, 4 SkinnyK, 5 General.
// ---------------------------------------------------------------------------
int orc_classify_workload(uint32_t m, uint32_t n, uint32_t k) {
  uint64_t mn = (uint64_t)m * n;
  if (mn < 8192) return 0;
  if (m < 128 && n >= 128) return 2;
  if (n < 128 && m >= 128) return 3;
  if (k < 64) return 4;
  if (m >= 1024 && n >= 1024) return 1;
  return 5;
}
// out[8] = tile_m, tile_n, tile_k, warp_m, warp_n, stages, use_tensor_core, split_k
// dtype: 0 fp8, 1 fp4, 2 int8; sm: 100 (Blackwell table).
void orc_tile_config(int dtype, uint32_t m, uint32_t n, uint32_t k, uint32_t* out) {
  int cls = orc_classify_workload(m, n, k);
  uint32_t stages = k < 64 ? 2 : 4;
  if (dtype == 2) { uint32_t t[8] = {128, 128, 64, 64, 64, 4, 1, 1}; std::memcpy(out, t, 32); return; }
  uint32_t t[8] = {0, 0, 128, 0, 0, stages, 1, 1};
  switch (cls) {
    case 0: t[0] = 64; t[1] = 64; t[2] = 64; t[3] = 32; t[4] = 32; break;
    case 2: t[0] = 64; t[1] = 256; t[3] = 32; t[4] = 128; break;
    case 3: t[0] = 256; t[1] = 64; t[3] = 128; t[4] = 32; break;
    case 1: t[0] = 256; t[1] = 256; t[3] = 64; t[4] = 128; break;
    case 4: t[0] = 256; t[1] = 256; t[3] = 64; t[4] = 128; t[5] = 2; if (dtype == 1) t[2] = 64; break;
    default: t[0] = dtype == 1 ? 128 : 256; t[1] = 256; t[3] = 64; t[4] = 128; break;
  }
  std::memcpy(out, t, 32);
}
uint32_t orc_fp8_split_k(uint32_t m, uint32_t n, uint32_t k) {
  if (m * n < 2048 && k > 32768) { uint32_t f = k / 8192; return f < 2 ? 2 : (f > 64 ? 64 : f); }
  return 1;
}

}  // extern "C"

// ---------------------------------------------------------------------------------------------------------
// GGML block codecs Q8_0 / Q4_0 / Q4_1 / Q4_K: crates/oxicuda-quant/src/scheme/ggml.rs:44-139 (binary16
// conversions, round to nearest even with subnormals), :243-282 (Q8_0), :284-335 (Q4_0), :342-391 (Q4_1),
// :404-506 (Q4_K).  Blocks are laid out as packed little-endian records in the field order of the reference's
// structs: Q8_0 {d f16, qs i8[32]} 34 bytes; Q4_0 {d, qs u8[16]} 18; Q4_1 {d, m, qs[16]} 20;
// Q4_K {d, dmin, scales u8[8], mins u8[8], qs u8[128]} 148 (the reference keeps the 6-bit values one per byte
// and packs code 2i with code 2i+1, :459-462).
// ---------------------------------------------------------------------------------------------------------
namespace {
uint16_t ggml_f32_to_f16_bits(float x) {                    // ggml.rs:50-107
  uint32_t bits; std::memcpy(&bits, &x, 4);
  const uint16_t sign = (uint16_t)((bits >> 16) & 0x8000u);
  const int exp = (int)((bits >> 23) & 0xFF);
  const uint32_t mantissa = bits & 0x007FFFFFu;
  if (exp == 0xFF) return mantissa != 0 ? (uint16_t)(sign | 0x7E00) : (uint16_t)(sign | 0x7C00);
  int e = exp - 127 + 15;
  if (e >= 0x1F) return (uint16_t)(sign | 0x7C00);
  if (e <= 0) {
    if (e < -10) return sign;
    const uint32_t m = mantissa | 0x00800000u;
    const uint32_t shift = (uint32_t)(14 - e);
    uint16_t half = (uint16_t)(m >> shift);
    const uint32_t round_bit = 1u << (shift - 1);
    if ((m & round_bit) != 0 && ((m & (round_bit - 1)) != 0 || (half & 1) != 0)) half = (uint16_t)(half + 1);
    return (uint16_t)(sign | half);
  }
  uint16_t half_mant = (uint16_t)(mantissa >> 13);
  const uint32_t round_bit = mantissa & 0x00001000u;
  if (round_bit != 0 && ((mantissa & 0x00000FFFu) != 0 || (half_mant & 1) != 0)) {
    half_mant = (uint16_t)(half_mant + 1);
    if (half_mant == 0x0400) {
      half_mant = 0;
      e += 1;
      if (e >= 0x1F) return (uint16_t)(sign | 0x7C00);
    }
  }
  return (uint16_t)(sign | ((uint16_t)e << 10) | half_mant);
}
float ggml_f16_to_f32(uint16_t h) {                          // ggml.rs:110-139
  const uint32_t sign = ((uint32_t)(h & 0x8000u)) << 16;
  const uint32_t exp = (h >> 10) & 0x1F, mant = h & 0x03FF;
  uint32_t bits;
  if (exp == 0) {
    if (mant == 0) bits = sign;
    else {
      const float magnitude = (float)mant * (1.0f / 16777216.0f);
      return (sign >> 31) != 0 ? -magnitude : magnitude;
    }
  } else if (exp == 0x1F) bits = sign | 0x7F800000u | (mant << 13);
  else bits = sign | ((exp + (127 - 15)) << 23) | (mant << 13);
  float f; std::memcpy(&f, &bits, 4);
  return f;
}
inline float ggml_f16_round(float x) { return ggml_f16_to_f32(ggml_f32_to_f16_bits(x)); }
inline float clampf(float v, float lo, float hi) { return v < lo ? lo : (v > hi ? hi : v); }   // f32::clamp on non-NaN input
inline void put16(uint8_t* p, uint16_t v) { p[0] = (uint8_t)(v & 0xFF); p[1] = (uint8_t)(v >> 8); }
inline uint16_t get16(const uint8_t* p) { return (uint16_t)(p[0] | (p[1] << 8)); }
}  // namespace

extern "C" {

uint16_t orc_ggml_f32_to_f16_bits(float x) { return ggml_f32_to_f16_bits(x); }
float orc_ggml_f16_to_f32(uint16_t h) { return ggml_f16_to_f32(h); }

// type: 0 Q8_0, 1 Q4_0, 2 Q4_1, 3 Q4_K.  Bytes of one block / weights per block.
int64_t orc_ggml_block_bytes(int type) { return type == 0 ? 34 : type == 1 ? 18 : type == 2 ? 20 : type == 3 ? 148 : -1; }
int64_t orc_ggml_block_size(int type) { return type == 3 ? 256 : 32; }

// Returns the number of blocks, -1 for an empty input, -2 for a length that is not a multiple of the block size
// (check_block, ggml.rs:522-534).
int64_t orc_ggml_quantize(int type, const float* w, int64_t n, uint8_t* out) {
  if (n <= 0) return -1;
  const int64_t bs = orc_ggml_block_size(type), bb = orc_ggml_block_bytes(type);
  if (n % bs != 0) return -2;
  const int64_t nb = n / bs;
  for (int64_t b = 0; b < nb; ++b) {
    const float* c = w + b * bs;
    uint8_t* o = out + b * bb;
    if (type == 0) {                                          // ggml.rs:243-262
      float amax = 0.0f;
      for (int i = 0; i < 32; ++i) amax = std::fmax(amax, std::fabs(c[i]));
      const float d = amax / 127.0f, dq = ggml_f16_round(d), inv = dq > 0.0f ? 1.0f / dq : 0.0f;
      put16(o, ggml_f32_to_f16_bits(d));
      for (int i = 0; i < 32; ++i) o[2 + i] = (uint8_t)(int8_t)clampf(std::round(c[i] * inv), -127.0f, 127.0f);
    } else if (type == 1) {                                   // ggml.rs:284-316
      float max = 0.0f, amax = 0.0f;
      for (int i = 0; i < 32; ++i) if (std::fabs(c[i]) > amax) { amax = std::fabs(c[i]); max = c[i]; }
      const float d = max / -8.0f, dq = ggml_f16_round(d), inv = dq != 0.0f ? 1.0f / dq : 0.0f;
      uint8_t codes[32];
      for (int i = 0; i < 32; ++i) codes[i] = (uint8_t)clampf(std::round(c[i] * inv) + 8.0f, 0.0f, 15.0f);
      put16(o, ggml_f32_to_f16_bits(d));
      for (int i = 0; i < 16; ++i) o[2 + i] = (uint8_t)(codes[i] | (codes[i + 16] << 4));
    } else if (type == 2) {                                   // ggml.rs:342-372
      float mn = std::numeric_limits<float>::infinity(), mx = -std::numeric_limits<float>::infinity();
      for (int i = 0; i < 32; ++i) { mn = std::fmin(mn, c[i]); mx = std::fmax(mx, c[i]); }
      const float d = (mx - mn) / 15.0f, dq = ggml_f16_round(d), mq = ggml_f16_round(mn), inv = dq > 0.0f ? 1.0f / dq : 0.0f;
      uint8_t codes[32];
      for (int i = 0; i < 32; ++i) codes[i] = (uint8_t)clampf(std::round((c[i] - mq) * inv), 0.0f, 15.0f);
      put16(o, ggml_f32_to_f16_bits(d));
      put16(o + 2, ggml_f32_to_f16_bits(mn));
      for (int i = 0; i < 16; ++i) o[4 + i] = (uint8_t)(codes[i] | (codes[i + 16] << 4));
    } else {                                                  // ggml.rs:404-472
      float sub_scales[8], sub_mins[8];
      for (int sb = 0; sb < 8; ++sb) {
        float mn = std::numeric_limits<float>::infinity(), mx = -std::numeric_limits<float>::infinity();
        for (int i = 0; i < 32; ++i) { mn = std::fmin(mn, c[sb * 32 + i]); mx = std::fmax(mx, c[sb * 32 + i]); }
        mn = std::fmin(mn, 0.0f);
        sub_scales[sb] = (mx - mn) / 15.0f;
        sub_mins[sb] = -mn;
      }
      float max_scale = 0.0f, max_min = 0.0f;
      for (int sb = 0; sb < 8; ++sb) { max_scale = std::fmax(max_scale, sub_scales[sb]); max_min = std::fmax(max_min, sub_mins[sb]); }
      max_min = max_min + 0.0f;                 // (-0.0 + 0.0 = +0.0) f32::max(+0.0, -0.0) may return either zero: the stored dmin is taken as +0
      const float d = max_scale / 63.0f, dmin = max_min / 63.0f, dq = ggml_f16_round(d), dminq = ggml_f16_round(dmin);
      const float inv_d = dq > 0.0f ? 1.0f / dq : 0.0f, inv_dmin = dminq > 0.0f ? 1.0f / dminq : 0.0f;
      uint8_t scales[8], mins[8], codes[256];
      for (int sb = 0; sb < 8; ++sb) {
        scales[sb] = (uint8_t)clampf(std::round(sub_scales[sb] * inv_d), 0.0f, 63.0f);
        mins[sb] = (uint8_t)clampf(std::round(sub_mins[sb] * inv_dmin), 0.0f, 63.0f);
      }
      for (int sb = 0; sb < 8; ++sb) {
        const float sc = dq * (float)scales[sb], mnv = dminq * (float)mins[sb], inv_sc = sc > 0.0f ? 1.0f / sc : 0.0f;
        for (int i = 0; i < 32; ++i) codes[sb * 32 + i] = (uint8_t)clampf(std::round((c[sb * 32 + i] + mnv) * inv_sc), 0.0f, 15.0f);
      }
      put16(o, ggml_f32_to_f16_bits(d));
      put16(o + 2, ggml_f32_to_f16_bits(dmin));
      for (int sb = 0; sb < 8; ++sb) { o[4 + sb] = scales[sb]; o[12 + sb] = mins[sb]; }
      for (int i = 0; i < 128; ++i) o[20 + i] = (uint8_t)(codes[2 * i] | (codes[2 * i + 1] << 4));
    }
  }
  return nb;
}

// n = number of weights (a multiple of the block size).  ggml.rs:265-276, :319-333, :375-390, :476-503.
void orc_ggml_dequantize(int type, const uint8_t* blocks, int64_t n, float* out) {
  const int64_t bs = orc_ggml_block_size(type), bb = orc_ggml_block_bytes(type), nb = n / bs;
  for (int64_t b = 0; b < nb; ++b) {
    const uint8_t* p = blocks + b * bb;
    float* o = out + b * bs;
    if (type == 0) {
      const float d = ggml_f16_to_f32(get16(p));
      for (int i = 0; i < 32; ++i) o[i] = (float)(int8_t)p[2 + i] * d;
    } else if (type == 1) {
      const float d = ggml_f16_to_f32(get16(p));
      for (int i = 0; i < 16; ++i) {
        o[i] = (float)((int)(p[2 + i] & 0x0F) - 8) * d;
        o[i + 16] = (float)((int)(p[2 + i] >> 4) - 8) * d;
      }
    } else if (type == 2) {
      const float d = ggml_f16_to_f32(get16(p)), m = ggml_f16_to_f32(get16(p + 2));
      for (int i = 0; i < 16; ++i) {
        o[i] = (float)(p[4 + i] & 0x0F) * d + m;
        o[i + 16] = (float)(p[4 + i] >> 4) * d + m;
      }
    } else {
      const float d = ggml_f16_to_f32(get16(p)), dmin = ggml_f16_to_f32(get16(p + 2));
      for (int sb = 0; sb < 8; ++sb) {
        const float sc = d * (float)p[4 + sb], mn = dmin * (float)p[12 + sb];
        for (int i = 0; i < 32; ++i) {
          const int k = sb * 32 + i;
          const float q = (float)((k & 1) ? (p[20 + (k >> 1)] >> 4) : (p[20 + (k >> 1)] & 0x0F));
          o[k] = sc * q - mn;
        }
      }
    }
  }
}

}  // extern "C"

// ---------------------------------------------------------------------------
// GPTQ / AWQ kernels of oxicuda-dnn (crates/oxicuda-dnn/src/quantize/gptq_awq.rs), each PTX instruction of the generated
// kernels restated in C: div.rn / mul.rn / add.rn / sub.rn / fma.rn are the IEEE operations, cvt.rni.f32.f32 is
// nearbyintf under the default rounding mode, max.f32 / min.f32 return the non-NaN operand (fmaxf / fminf),
// cvt.rzi.u32.f32 truncates (its inputs are clamped to [0, 255] first).
// ---------------------------------------------------------------------------
namespace {
inline int wq_epu(int bits) { return 32 / bits; }
}  // namespace

extern "C" {

// dnn_gptq_quantize_f32 (:329-499): one thread per row walks the columns upwards; packed must arrive zeroed (atomic OR)
// and is cleared here; scale[row, group] is overwritten by every column of the group.
void orc_gptq_quantize(const float* w, const float* hdiag, int64_t rows, int64_t cols, int64_t group, int bits, int symmetric, uint32_t* packed,
                       float* scales) {
  const int epu = wq_epu(bits);
  const float qmax = (float)((1u << bits) - 1u), half = (float)(1u << (bits - 1));
  const int64_t total = rows * cols, gpr = cols / group;
  std::memset(packed, 0, (size_t)((total + epu - 1) / epu) * 4);
  for (int64_t row = 0; row < rows; ++row) {
    for (int64_t col = 0; col < cols; ++col) {
      const int64_t e = row * cols + col;
      const float safe_h = fmaxf(hdiag[col], 1e-6f);                // MIN_DAMP (:29), max.f32 (:425)
      const float scaled = w[e] / safe_h;                          // div.rn (:429)
      float rounded = nearbyintf(scaled);                          // cvt.rni (:433)
      if (symmetric) rounded = fmaxf(rounded + half, 0.0f);        // add.rn, max.f32 (:452-453)
      float clamped = fminf(rounded, qmax);                        // (:456)
      clamped = fmaxf(clamped, 0.0f);                              // (:457)
      const uint32_t q = (uint32_t)clamped;                        // cvt.rzi.u32.f32 (:461)
      scales[row * gpr + col / group] = safe_h / qmax;             // (:466-467)
      packed[e / epu] |= q << ((e % epu) * bits);                  // (:471-489)
    }
  }
}

// dnn_gptq_dequantize_f32 (:509-616); zeros == NULL is the symmetric kernel.
void orc_wq_dequantize(const uint32_t* packed, const float* scales, const float* zeros, int64_t rows, int64_t cols, int64_t group, int bits,
                       float* out) {
  const int epu = wq_epu(bits);
  const uint32_t mask = (1u << bits) - 1u;
  const int64_t gpr = cols / group;
  for (int64_t e = 0; e < rows * cols; ++e) {
    const float qf = (float)((packed[e / epu] >> ((e % epu) * bits)) & mask);    // shr, and, cvt.rn.f32.u32 (:560-567)
    const int64_t s_idx = (e / cols) * gpr + (e % cols) / group;                 // (:570-584)
    out[e] = zeros ? (qf - zeros[s_idx]) * scales[s_idx] : qf * scales[s_idx];   // (:592-603)
  }
}

// dnn_awq_scale_search_f32 (:626-713): a * rsqrt.approx(a); the approximate reciprocal square root is restated as the
// correctly rounded 1 / sqrt(a), so callers compare with a tolerance of a few units in the last place.
void orc_awq_scale_search(const float* act, int64_t n, float* out) {
  for (int64_t i = 0; i < n; ++i) {
    const float a = fmaxf(fabsf(act[i]), 1e-7f);                   // abs, max.f32 (:683-688)
    const float rsq = (float)(1.0 / std::sqrt((double)a));
    out[i] = a * rsq;                                              // mul.rn (:695)
  }
}

// dnn_awq_quantize_f32 (:723-857): group scales are an input; zeros (may be NULL) receive 0.0.
void orc_awq_quantize(const float* w, const float* ch_scales, const float* g_scales, int64_t rows, int64_t cols, int64_t group, int bits,
                      uint32_t* packed, float* zeros) {
  const int epu = wq_epu(bits);
  const float qmax = (float)((1u << bits) - 1u);
  const int64_t total = rows * cols, gpr = cols / group;
  std::memset(packed, 0, (size_t)((total + epu - 1) / epu) * 4);
  for (int64_t e = 0; e < total; ++e) {
    const int64_t col = e % cols, s_idx = (e / cols) * gpr + col / group;
    const float w_scaled = w[e] * ch_scales[col];                  // mul.rn (:777)
    const float safe = fmaxf(g_scales[s_idx], 1e-12f);             // (:799-802)
    const float rounded = nearbyintf(w_scaled / safe);             // div.rn, cvt.rni (:803-807)
    float clamped = fmaxf(rounded, 0.0f);                          // (:818)
    clamped = fminf(clamped, qmax);                                // (:819)
    packed[e / epu] |= (uint32_t)clamped << ((e % epu) * bits);    // (:822-841)
    if (zeros) zeros[s_idx] = 0.0f;                                // (:845-849)
  }
}

// dnn_fused_dequant_gemv_f32 (:867-986): one thread per row, packed words upwards, the values of a word upwards;
// row r starts at word r * (cols / epu).  zeros != NULL is the library's extension ((q - zero) * scale).
void orc_fused_dequant_gemv(const uint32_t* packed, const float* scales, const float* zeros, const float* x, int64_t rows, int64_t cols,
                            int64_t group, int bits, float* y) {
  const int epu = wq_epu(bits);
  const uint32_t mask = (1u << bits) - 1u;
  const int64_t packed_cols = cols / epu, gpr = cols / group;
#pragma omp parallel for schedule(static)
  for (int64_t row = 0; row < rows; ++row) {
    float acc = 0.0f;
    for (int64_t pw = 0; pw < packed_cols; ++pw) {
      const uint32_t word = packed[row * packed_cols + pw];
      for (int sub = 0; sub < epu; ++sub) {
        const int64_t col = pw * epu + sub;
        const float qf = (float)((word >> (sub * bits)) & mask);
        const int64_t s_idx = row * gpr + col / group;
        const float dq = zeros ? (qf - zeros[s_idx]) * scales[s_idx] : qf * scales[s_idx];   // mul.rn (:961)
        acc = fmaf(dq, x[col], acc);                                                          // fma.rn (:966)
      }
    }
    y[row] = acc;
  }
}

}  // extern "C"
