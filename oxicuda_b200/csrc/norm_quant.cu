// RMSNorm (optionally with the residual add in front of it) fused with the per-token FP8 quantization that feeds the
// next quantized linear: one launch reads the bf16 activations once and writes FP8 codes plus one scale per token,
// instead of a normalisation kernel that writes bf16 and a quantizer that reads it back.
//   y = x / sqrt(mean(x^2) + eps) * gamma           (crates/oxicuda-dnn/src/norm/rms_norm.rs:29-33, :566-574)
//   residual += x first, norm of the sum            (fused_add_rms_norm, rms_norm.rs:98-103)
//   scale = absmax(y) / max_val (1 for a zero row), code = encode(clamp(y / scale))   (the per-token rule of
//   b2q_fp8_quantize_rows_*).
// HBM-bound: 2 bytes read and 1 byte written per element (6 and 3 with the residual).
#include "common.cuh"

namespace {

__device__ __forceinline__ float block_reduce(float v, bool take_max, float* sh) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float t = __shfl_xor_sync(0xffffffffu, v, o);
    v = take_max ? fmaxf(v, t) : v + t;
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  __syncthreads();                         // sh may still be read from the previous reduction
  if (lane == 0) sh[warp] = v;
  __syncthreads();
  v = lane < nw ? sh[lane] : (take_max ? 0.0f : 0.0f);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float t = __shfl_xor_sync(0xffffffffu, v, o);
    v = take_max ? fmaxf(v, t) : v + t;
  }
  return v;
}

__device__ __forceinline__ void unpack8(const uint4 q, float (&v)[8]) {
  const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
  for (int j = 0; j < 4; ++j) { v[2 * j] = __uint_as_float(w[j] << 16); v[2 * j + 1] = __uint_as_float(w[j] & 0xFFFF0000u); }
}
__device__ __forceinline__ uint32_t bf16_bits(float f) { return (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(f)); }

// One CTA per token; thread t keeps chunks t, t + blockDim, ... (8 elements each, NCH at most) of the row in registers.
// FULL: every thread has all NCH chunks (cols == 8 * NCH * blockDim), so the bounds predicates drop out.
template <int NCH, bool FULL>
__global__ void __launch_bounds__(1024) rms_norm_quantize_fp8_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* residual,
                                                                     const __nv_bfloat16* __restrict__ gamma, int64_t cols, float eps, int fmt,
                                                                     int rounding, float* __restrict__ scales, uint8_t* __restrict__ codes,
                                                                     __nv_bfloat16* __restrict__ y_out) {
  __shared__ float sh[32];
  const int64_t r = blockIdx.x;
  const int chunks = (int)(cols >> 3);
  const uint4* xr = reinterpret_cast<const uint4*>(x + r * cols);
  uint4* rr = residual ? reinterpret_cast<uint4*>(residual + r * cols) : nullptr;
  float v[NCH][8];
  float ss = 0.0f;
#pragma unroll
  for (int k = 0; k < NCH; ++k) {
    const int c = (int)threadIdx.x + k * (int)blockDim.x;
    if (FULL || c < chunks) {
      unpack8(xr[c], v[k]);
      if (rr) {
        float res[8];
        unpack8(rr[c], res);
        uint32_t w[4];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const uint32_t b = bf16_bits(__fadd_rn(res[j], v[k][j]));   // the norm is taken of the sum as it is stored
          v[k][j] = __uint_as_float(b << 16);
          if (j & 1) w[j >> 1] |= b << 16; else w[j >> 1] = b;
        }
        rr[c] = make_uint4(w[0], w[1], w[2], w[3]);
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) ss = fmaf(v[k][j], v[k][j], ss);
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) v[k][j] = 0.0f;
    }
  }
  ss = block_reduce(ss, false, sh);
  // x * (1 / rms) * gamma and y * (1 / scale): one rounding more than the divisions of the CPU statement (the
  // reference's own kernel multiplies by rsqrt.approx); an IEEE division per element would make the kernel
  // instruction-bound instead of HBM-bound.
  const float inv_rms = __frcp_rn(sqrtf(__fadd_rn(__fdiv_rn(ss, (float)cols), eps)));
  const uint4* gr = reinterpret_cast<const uint4*>(gamma);
  float amax = 0.0f;
#pragma unroll
  for (int k = 0; k < NCH; ++k) {
    const int c = (int)threadIdx.x + k * (int)blockDim.x;
    if (FULL || c < chunks) {
      float g[8];
      unpack8(gr[c], g);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        v[k][j] = __fmul_rn(__fmul_rn(v[k][j], inv_rms), g[j]);
        amax = fmaxf(amax, fabsf(v[k][j]));
      }
    }
  }
  amax = block_reduce(amax, true, sh);
  const Fp8Fmt F = fp8_fmt(fmt);
  const float scale = amax > 0.0f ? __fdiv_rn(amax, F.max_val) : 1.0f;
  const float inv_scale = __frcp_rn(scale);
  if (threadIdx.x == 0) scales[r] = scale;
  uint2* cr = reinterpret_cast<uint2*>(codes + r * cols);
  uint4* yr = y_out ? reinterpret_cast<uint4*>(y_out + r * cols) : nullptr;
#pragma unroll
  for (int k = 0; k < NCH; ++k) {
    const int c = (int)threadIdx.x + k * (int)blockDim.x;
    if (FULL || c < chunks) {
      uint32_t lo = 0, hi = 0;
      if (rounding == 1) {     // the conversion saturates to +-max_val by itself
        uint32_t p[4];
#pragma unroll
        for (int j = 0; j < 4; ++j)
          p[j] = (uint32_t)__nv_cvt_float2_to_fp8x2(make_float2(__fmul_rn(v[k][2 * j], inv_scale), __fmul_rn(v[k][2 * j + 1], inv_scale)),
                                                    __NV_SATFINITE, fmt == 0 ? __NV_E4M3 : __NV_E5M2);
        lo = __byte_perm(p[0], p[1], 0x5410);
        hi = __byte_perm(p[2], p[3], 0x5410);
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          float q = __fmul_rn(v[k][j], inv_scale);
          q = q < -F.max_val ? -F.max_val : (q > F.max_val ? F.max_val : q);
          const uint32_t b = fp8_encode_ref_dev(q, F);
          if (j < 4) lo |= b << (8 * j); else hi |= b << (8 * (j - 4));
        }
      }
      cr[c] = make_uint2(lo, hi);
      if (yr) {
        uint32_t w[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) w[j] = bf16_bits(v[k][2 * j]) | (bf16_bits(v[k][2 * j + 1]) << 16);
        yr[c] = make_uint4(w[0], w[1], w[2], w[3]);
      }
    }
  }
}

// Any row length and alignment: the row is re-read from L1/L2 instead of kept in registers.
__global__ void __launch_bounds__(256) rms_norm_quantize_fp8_generic_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* residual,
                                                                            const __nv_bfloat16* __restrict__ gamma, int64_t cols, float eps,
                                                                            int fmt, int rounding, float* __restrict__ scales,
                                                                            uint8_t* __restrict__ codes, __nv_bfloat16* __restrict__ y_out) {
  __shared__ float sh[32];
  const int64_t r = blockIdx.x;
  const __nv_bfloat16* row = x + r * cols;
  __nv_bfloat16* res = residual ? residual + r * cols : nullptr;
  float ss = 0.0f;
  for (int64_t i = threadIdx.x; i < cols; i += blockDim.x) {
    float v = __bfloat162float(row[i]);
    if (res) {
      const __nv_bfloat16 s = __float2bfloat16_rn(__fadd_rn(__bfloat162float(res[i]), v));
      res[i] = s;                       // read back below by the thread that wrote it
      v = __bfloat162float(s);
    }
    ss = fmaf(v, v, ss);
  }
  ss = block_reduce(ss, false, sh);
  const float inv_rms = __frcp_rn(sqrtf(__fadd_rn(__fdiv_rn(ss, (float)cols), eps)));   // same arithmetic as the register kernel
  const __nv_bfloat16* src = res ? res : row;
  float amax = 0.0f;
  for (int64_t i = threadIdx.x; i < cols; i += blockDim.x)
    amax = fmaxf(amax, fabsf(__fmul_rn(__fmul_rn(__bfloat162float(src[i]), inv_rms), __bfloat162float(gamma[i]))));
  amax = block_reduce(amax, true, sh);
  const Fp8Fmt F = fp8_fmt(fmt);
  const float scale = amax > 0.0f ? __fdiv_rn(amax, F.max_val) : 1.0f;
  const float inv_scale = __frcp_rn(scale);
  if (threadIdx.x == 0) scales[r] = scale;
  for (int64_t i = threadIdx.x; i < cols; i += blockDim.x) {
    const float y = __fmul_rn(__fmul_rn(__bfloat162float(src[i]), inv_rms), __bfloat162float(gamma[i]));
    float q = __fmul_rn(y, inv_scale);
    q = q < -F.max_val ? -F.max_val : (q > F.max_val ? F.max_val : q);
    codes[r * cols + i] = (uint8_t)(rounding == 0 ? fp8_encode_ref_dev(q, F) : fp8_encode_rne_dev(q, fmt));
    if (y_out) y_out[r * cols + i] = __float2bfloat16_rn(y);
  }
}

}  // namespace

extern "C" int32_t b2q_rms_norm_quantize_fp8_bf16(b2q_handle h, const void* x, void* residual, const void* gamma, int64_t rows, int64_t cols,
                                                  float eps, int fmt, int rounding, float* scales, uint8_t* codes, void* y_out) {
  B2Q_REQUIRE_HANDLE(h);
  if (rows <= 0 || cols <= 0) B2Q_FAIL(h, B2Q_ERR_EMPTY_INPUT, "rms_norm_quantize_fp8: empty input");
  if (!x || !gamma || !scales || !codes) B2Q_FAIL(h, B2Q_ERR_INVALID_ARGUMENT, "rms_norm_quantize_fp8: null pointer");
  if (fmt < 0 || fmt > 1 || rounding < 0 || rounding > 1) B2Q_FAIL(h, B2Q_ERR_INVALID_ARGUMENT, "rms_norm_quantize_fp8: bad format/rounding");
  if (rows > 0x7FFFFFFF) B2Q_FAIL(h, B2Q_ERR_INVALID_DIMENSION, "rms_norm_quantize_fp8: %lld rows", (long long)rows);
  const __nv_bfloat16* xp = static_cast<const __nv_bfloat16*>(x);
  __nv_bfloat16* rp = static_cast<__nv_bfloat16*>(residual);
  const __nv_bfloat16* gp = static_cast<const __nv_bfloat16*>(gamma);
  __nv_bfloat16* yp = static_cast<__nv_bfloat16*>(y_out);
  const uintptr_t align = reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(residual) | reinterpret_cast<uintptr_t>(gamma) |
                          reinterpret_cast<uintptr_t>(y_out) | (reinterpret_cast<uintptr_t>(codes) << 1);
  const int64_t chunks = cols >> 3;
  if (cols % 8 == 0 && (align & 15) == 0 && chunks <= 4 * 1024) {
    // threads: a multiple of 32 covering the chunks in at most NCH passes
    int nch = chunks <= 1024 ? 1 : (chunks <= 2048 ? 2 : 4);
    if (chunks <= 1024 && chunks > 256 && rows >= 4 * (int64_t)h->sm_count) nch = chunks <= 512 ? 2 : 4;   // many rows: smaller CTAs, more of them per SM
    int threads = (int)((ceil_div64(chunks, nch) + 31) / 32 * 32);
    if (threads < 32) threads = 32;
    const bool full = chunks == (int64_t)nch * threads;
#define RMS_LAUNCH(N, F) rms_norm_quantize_fp8_kernel<N, F><<<(unsigned)rows, threads, 0, h->stream>>>(xp, rp, gp, cols, eps, fmt, rounding, scales, codes, yp)
    if (nch == 1) { if (full) RMS_LAUNCH(1, true); else RMS_LAUNCH(1, false); }
    else if (nch == 2) { if (full) RMS_LAUNCH(2, true); else RMS_LAUNCH(2, false); }
    else { if (full) RMS_LAUNCH(4, true); else RMS_LAUNCH(4, false); }
#undef RMS_LAUNCH
    B2Q_LAUNCH_CHECK(h, "rms_norm_quantize_fp8_kernel");
    return B2Q_OK;
  }
  rms_norm_quantize_fp8_generic_kernel<<<(unsigned)rows, 256, 0, h->stream>>>(xp, rp, gp, cols, eps, fmt, rounding, scales, codes, yp);
  B2Q_LAUNCH_CHECK(h, "rms_norm_quantize_fp8_generic_kernel");
  return B2Q_OK;
}
