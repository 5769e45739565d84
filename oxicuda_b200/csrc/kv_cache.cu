// KV-cache quantizers (HBM-bound byte work): the asymmetric per-token / per-channel scheme of
// KvCacheQuantizer (crates/oxicuda-quant/src/scheme/kv_cache.rs:146-282) and the per-token symmetric / asymmetric
// scheme of quantize_token (crates/oxicuda-infer/src/cache/kv_quant.rs:112-154), one code per byte.
// Every arithmetic step is an explicit IEEE intrinsic in the reference's order, so codes, scales and zero points are
// bit-identical to the reference's f32 arithmetic whatever the compiler's contraction settings.
#include "common.cuh"

namespace {

constexpr int kThreads = 256;
constexpr int kWarpsPerBlock = kThreads / 32;

enum KvRule { kRuleCache = 0, kRuleTokenAsym = 1, kRuleTokenSym = 2 };

template <typename T> __device__ __forceinline__ float ld1(const T* p, int64_t i);
template <> __device__ __forceinline__ float ld1<float>(const float* p, int64_t i) { return p[i]; }
template <> __device__ __forceinline__ float ld1<__nv_bfloat16>(const __nv_bfloat16* p, int64_t i) { return __bfloat162float(p[i]); }

// four consecutive elements starting at element index i (i % 4 == 0, the address aligned to 4 elements)
template <typename T> __device__ __forceinline__ void ld4(const T* p, int64_t i, float (&v)[4]);
template <> __device__ __forceinline__ void ld4<float>(const float* p, int64_t i, float (&v)[4]) {
  const float4 q = *reinterpret_cast<const float4*>(p + i);
  v[0] = q.x; v[1] = q.y; v[2] = q.z; v[3] = q.w;
}
template <> __device__ __forceinline__ void ld4<__nv_bfloat16>(const __nv_bfloat16* p, int64_t i, float (&v)[4]) {
  const uint2 q = *reinterpret_cast<const uint2*>(p + i);
  v[0] = __uint_as_float(q.x << 16); v[1] = __uint_as_float(q.x & 0xFFFF0000u);
  v[2] = __uint_as_float(q.y << 16); v[3] = __uint_as_float(q.y & 0xFFFF0000u);
}

template <typename T> __device__ __forceinline__ void st1(T* p, int64_t i, float v);
template <> __device__ __forceinline__ void st1<float>(float* p, int64_t i, float v) { p[i] = v; }
template <> __device__ __forceinline__ void st1<__nv_bfloat16>(__nv_bfloat16* p, int64_t i, float v) { p[i] = __float2bfloat16_rn(v); }

struct KvParams { float scale, zp; };

// The (scale, zero point) of one group from its minimum and maximum.
__device__ __forceinline__ KvParams kv_params(int rule, float mn, float mx, float qmin_f, float qmax_f) {
  KvParams p;
  if (rule == kRuleCache) {            // kv_cache.rs:188-192: range.max(1e-8) / q_max, zero point = min
    p.scale = __fdiv_rn(fmaxf(__fsub_rn(mx, mn), 1e-8f), qmax_f);
    p.zp = mn;
  } else if (rule == kRuleTokenAsym) { // kv_quant.rs:128-137
    const float range = __fsub_rn(mx, mn);
    p.scale = range > 0.0f ? __fdiv_rn(range, __fsub_rn(qmax_f, qmin_f)) : 1.0f;
    p.zp = __fsub_rn(mn, __fmul_rn(qmin_f, p.scale));
  } else {                             // kv_quant.rs:123-127
    const float amax = fmaxf(fabsf(mn), fabsf(mx));
    p.scale = amax > 0.0f ? __fdiv_rn(amax, qmax_f) : 1.0f;
    p.zp = 0.0f;
  }
  return p;
}

// One code: round((v - zp) / scale) half away from zero, clamped to [qmin, qmax]; NaN gives 0 before the clamp
// (Rust's saturating `as` casts), so the byte is the low 8 bits of the clamped integer.  The exact statement is
//   qi = __float2int_rz(roundf(__fdiv_rn(__fsub_rn(v, zp), scale)))   (integral value; the cast saturates, NaN -> 0);
// the code below reaches the same integer with one multiplication instead of the IEEE division where that is provable.
// inv = RN(1 / scale) (or NaN when the scale is outside [1e-30, 1e30]), so a * inv lies within 2 ulp of RN(a / scale).
// When that product is further than 3e-4 (> 4 ulp below 1024) from every half-integer, it and the exact quotient
// lie strictly between the same two half-integers and round to the same integer under any tie rule.  Everything
// else (near ties, |q| >= 1024, NaN, unusable reciprocal) takes the exact path.
__device__ __forceinline__ float kv_inv_scale(float scale) {
  return (scale > 1e-30f && scale < 1e30f) ? __frcp_rn(scale) : __uint_as_float(0x7FC00000u);
}
__device__ __forceinline__ uint32_t kv_code_exact(float v, float scale, float zp, int qmin, int qmax) {
  int qi = __float2int_rz(roundf(__fdiv_rn(__fsub_rn(v, zp), scale)));
  qi = qi < qmin ? qmin : (qi > qmax ? qmax : qi);
  return (uint32_t)qi & 0xFFu;
}
__device__ __forceinline__ uint32_t kv_code_fast(float v, KvParams p, float inv, int qmin, int qmax) {
  const float a = __fsub_rn(v, p.zp);
  const float q = __fmul_rn(a, inv);
  int qi = __float2int_rn(q);
  const float d = __fsub_rn(q, (float)qi);
  if (!(fabsf(d) < 0.4997f && fabsf(q) < 1024.0f)) return kv_code_exact(v, p.scale, p.zp, qmin, qmax);
  qi = qi < qmin ? qmin : (qi > qmax ? qmax : qi);
  return (uint32_t)qi & 0xFFu;
}
// Four codes packed into a word, all on full-rate pipes.  q is clamped to [qmin, qmax] as a float, then
// t = clamp + 1.5 * 2^23 holds round-to-nearest(clamp) in its low mantissa bits (the low byte of t is the code, in
// two's complement for negative ones).  The distance d = q - (t - 1.5 * 2^23) is measured from the unclamped q, so a
// quotient outside the range, next to a tie, NaN or infinite fails |d| < 0.4997 and sends the four elements down the
// exact path.
__device__ __forceinline__ uint32_t kv_codes4(const float (&v)[4], const float (&scale)[4], const float (&zp)[4], const float (&inv)[4],
                                              int qmin, int qmax) {
  const float magic = 12582912.0f, lo = (float)qmin, hi = (float)qmax;
  uint32_t t[4];
  bool ok = true;
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const float q = __fmul_rn(__fsub_rn(v[e], zp[e]), inv[e]);
    const float tf = __fadd_rn(fminf(fmaxf(q, lo), hi), magic);
    ok = ok && (fabsf(__fsub_rn(q, __fsub_rn(tf, magic))) < 0.4997f);
    t[e] = __float_as_uint(tf);
  }
  if (ok) return __byte_perm(__byte_perm(t[0], t[1], 0x0040), __byte_perm(t[2], t[3], 0x0040), 0x5410);
  return kv_code_exact(v[0], scale[0], zp[0], qmin, qmax) | (kv_code_exact(v[1], scale[1], zp[1], qmin, qmax) << 8) |
         (kv_code_exact(v[2], scale[2], zp[2], qmin, qmax) << 16) | (kv_code_exact(v[3], scale[3], zp[3], qmin, qmax) << 24);
}
__device__ __forceinline__ uint32_t kv_codes4(const float (&v)[4], KvParams p, float inv, int qmin, int qmax) {
  const float s[4] = {p.scale, p.scale, p.scale, p.scale}, z[4] = {p.zp, p.zp, p.zp, p.zp}, n[4] = {inv, inv, inv, inv};
  return kv_codes4(v, s, z, n, qmin, qmax);
}

// ---------------------------------------------------------------------------
// One group per token, rows of at most 1024 elements (every head dimension in use).  G lanes share a row, so a warp
// works on 32 / G rows at a time; a lane keeps NV chunks of 4 elements (chunk lane_in_group + G * k) in registers, so
// each input byte is read once, NV 16-byte loads are in flight per lane, the reduction takes log2(G) shuffle rounds
// and the parameters are derived once per 4 * NV elements of a lane.
// ---------------------------------------------------------------------------
// FULL: cols == G * NV * 4, every lane has all its chunks and the column predicates drop out.
template <typename T, int G, int NV, bool FULL>
__global__ void __launch_bounds__(kThreads) kv_quantize_per_token_reg_kernel(const T* __restrict__ x, int64_t rows, int64_t cols, int rule,
                                                                             int qmin, int qmax, uint8_t* __restrict__ codes,
                                                                             float* __restrict__ scales, float* __restrict__ zps) {
  constexpr int kRowsPerWarp = 32 / G;
  const int lane = threadIdx.x & 31, sub = lane % G, grp = lane / G;
  const float qmin_f = (float)qmin, qmax_f = (float)qmax;
  const float nan = __uint_as_float(0x7FC00000u);   // never wins fminf / fmaxf
  const int64_t warp = (int64_t)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
  for (int64_t r0 = warp * kRowsPerWarp; r0 < rows; r0 += (int64_t)gridDim.x * kWarpsPerBlock * kRowsPerWarp) {
    const int64_t r = r0 + grp;
    const bool live = r < rows;
    float v[NV][4];
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      const int64_t c = (int64_t)(sub + G * k) * 4;
      if (live && (FULL || c < cols)) ld4<T>(x + r * cols, c, v[k]);
      else v[k][0] = v[k][1] = v[k][2] = v[k][3] = nan;
    }
    float mn = __uint_as_float(0x7F800000u), mx = __uint_as_float(0xFF800000u);
#pragma unroll
    for (int k = 0; k < NV; ++k)
#pragma unroll
      for (int e = 0; e < 4; ++e) { mn = fminf(mn, v[k][e]); mx = fmaxf(mx, v[k][e]); }
#pragma unroll
    for (int o = G / 2; o > 0; o >>= 1) {
      mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    }
    if (!live) continue;
    const KvParams p = kv_params(rule, mn, mx, qmin_f, qmax_f);
    const float inv = kv_inv_scale(p.scale);
    if (sub == 0) { scales[r] = p.scale; zps[r] = p.zp; }
    uint8_t* out = codes + r * cols;
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      const int64_t c = (int64_t)(sub + G * k) * 4;
      if (FULL || c < cols) *reinterpret_cast<uint32_t*>(out + c) = kv_codes4(v[k], p, inv, qmin, qmax);
    }
  }
}

// ---------------------------------------------------------------------------
// One group per token, any row length and alignment: a warp per row, statistics and codes in one launch.  The second
// pass re-reads the row from L1/L2, so DRAM sees each input byte once.
// ---------------------------------------------------------------------------
template <typename T, bool VEC>
__global__ void __launch_bounds__(kThreads) kv_quantize_per_token_kernel(const T* __restrict__ x, int64_t rows, int64_t cols, int rule,
                                                                         int qmin, int qmax, uint8_t* __restrict__ codes,
                                                                         float* __restrict__ scales, float* __restrict__ zps) {
  const int lane = threadIdx.x & 31;
  const float qmin_f = (float)qmin, qmax_f = (float)qmax;
  for (int64_t r = (int64_t)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5); r < rows; r += (int64_t)gridDim.x * kWarpsPerBlock) {
    const T* row = x + r * cols;
    float mn = __uint_as_float(0x7F800000u), mx = __uint_as_float(0xFF800000u);
    if (VEC) {
      for (int64_t i = (int64_t)lane * 4; i < cols; i += 128) {
        float v[4];
        ld4<T>(row, i, v);
#pragma unroll
        for (int j = 0; j < 4; ++j) { mn = fminf(mn, v[j]); mx = fmaxf(mx, v[j]); }
      }
    } else {
      for (int64_t i = lane; i < cols; i += 32) { const float v = ld1<T>(row, i); mn = fminf(mn, v); mx = fmaxf(mx, v); }
    }
    mn = warp_min(mn);
    mx = warp_max(mx);
    const KvParams p = kv_params(rule, mn, mx, qmin_f, qmax_f);
    const float inv = kv_inv_scale(p.scale);
    if (lane == 0) { scales[r] = p.scale; zps[r] = p.zp; }
    uint8_t* out = codes + r * cols;
    if (VEC) {
      for (int64_t i = (int64_t)lane * 4; i < cols; i += 128) {
        float v[4];
        ld4<T>(row, i, v);
        *reinterpret_cast<uint32_t*>(out + i) = kv_codes4(v, p, inv, qmin, qmax);
      }
    } else {
      for (int64_t i = lane; i < cols; i += 32) out[i] = (uint8_t)kv_code_fast(ld1<T>(row, i), p, inv, qmin, qmax);
    }
  }
}

// ---------------------------------------------------------------------------
// One group per channel (keys): column minima / maxima over all tokens through ordered-key atomics in the handle's
// scratch (keys[c] = minimum, keys[head_dim + c] = maximum), then the parameters, then the codes.
// ---------------------------------------------------------------------------
__global__ void kv_channel_keys_init_kernel(uint32_t* keys, int64_t head_dim) {
  const int64_t c = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (c < head_dim) {
    keys[c] = float_order_key(__uint_as_float(0x7F800000u));             // +inf: nothing seen yet
    keys[head_dim + c] = float_order_key(__uint_as_float(0xFF800000u));  // -inf
  }
}

// grid.x covers the columns 32 at a time, grid.y the tokens in chunks of `rows_per_block`; warp w of a block scans
// rows w, w + 8, ... of its chunk, a lane per column (128 contiguous bytes per warp load for f32).
template <typename T>
__global__ void __launch_bounds__(kThreads) kv_channel_stats_kernel(const T* __restrict__ x, int64_t rows, int64_t cols,
                                                                    int64_t rows_per_block, uint32_t* keys) {
  __shared__ float s_mn[kWarpsPerBlock][32], s_mx[kWarpsPerBlock][32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t c = (int64_t)blockIdx.x * 32 + lane;
  const int64_t r0 = (int64_t)blockIdx.y * rows_per_block;
  const int64_t r1 = r0 + rows_per_block < rows ? r0 + rows_per_block : rows;
  float mn = __uint_as_float(0x7F800000u), mx = __uint_as_float(0xFF800000u);
  if (c < cols) {
    int64_t r = r0 + warp;
    for (; r + 3 * kWarpsPerBlock < r1; r += 4 * kWarpsPerBlock) {
      float v[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) v[j] = ld1<T>(x, (r + j * kWarpsPerBlock) * cols + c);
#pragma unroll
      for (int j = 0; j < 4; ++j) { mn = fminf(mn, v[j]); mx = fmaxf(mx, v[j]); }
    }
    for (; r < r1; r += kWarpsPerBlock) { const float v = ld1<T>(x, r * cols + c); mn = fminf(mn, v); mx = fmaxf(mx, v); }
  }
  s_mn[warp][lane] = mn;
  s_mx[warp][lane] = mx;
  __syncthreads();
  if (warp == 0 && c < cols) {
#pragma unroll
    for (int w = 1; w < kWarpsPerBlock; ++w) { mn = fminf(mn, s_mn[w][lane]); mx = fmaxf(mx, s_mx[w][lane]); }
    atomicMin(keys + c, float_order_key(mn));
    atomicMax(keys + cols + c, float_order_key(mx));
  }
}

__global__ void kv_channel_params_kernel(const uint32_t* keys, int64_t head_dim, float qmax_f, float* scales, float* zps, float* inv_scales) {
  const int64_t c = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (c < head_dim) {
    const KvParams p = kv_params(kRuleCache, float_from_order_key(keys[c]), float_from_order_key(keys[head_dim + c]), 0.0f, qmax_f);
    scales[c] = p.scale;
    zps[c] = p.zp;
    inv_scales[c] = kv_inv_scale(p.scale);
  }
}

template <typename T, bool VEC>
__global__ void __launch_bounds__(kThreads) kv_quantize_per_channel_kernel(const T* __restrict__ x, int64_t n, int64_t cols, int qmax,
                                                                           const float* __restrict__ scales, const float* __restrict__ zps,
                                                                           const float* __restrict__ inv_scales, uint8_t* __restrict__ codes) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  if (VEC) {   // cols % 4 == 0: four consecutive elements share a row and are four consecutive channels
    for (int64_t i = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 4; i < n; i += stride * 4) {
      const int64_t c = i % cols;
      float v[4];
      ld4<T>(x, i, v);
      const float4 s = *reinterpret_cast<const float4*>(scales + c);
      const float4 z = *reinterpret_cast<const float4*>(zps + c);
      const float4 n = *reinterpret_cast<const float4*>(inv_scales + c);
      const float sc[4] = {s.x, s.y, s.z, s.w}, zp[4] = {z.x, z.y, z.z, z.w}, nv[4] = {n.x, n.y, n.z, n.w};
      *reinterpret_cast<uint32_t*>(codes + i) = kv_codes4(v, sc, zp, nv, 0, qmax);
    }
  } else {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
      const int64_t c = i % cols;
      codes[i] = (uint8_t)kv_code_fast(ld1<T>(x, i), KvParams{scales[c], zps[c]}, inv_scales[c], 0, qmax);
    }
  }
}

// code * scale + zero point, unfused (kv_cache.rs:224-238, kv_quant.rs:94-100).  axis 0: group = row, 1: group = column.
// n = rows * cols.
template <typename T>
__global__ void __launch_bounds__(kThreads) kv_dequantize_kernel(const uint8_t* __restrict__ codes, int64_t n, int64_t cols, int axis,
                                                                 int signed_codes, const float* __restrict__ scales,
                                                                 const float* __restrict__ zps, T* __restrict__ out) {
  // a warp per row (grid-stride), four codes per lane and step when the rows allow 32-bit code loads
  const int lane = threadIdx.x & 31;
  const int64_t rows = n / cols;
  const bool vec = (cols & 3) == 0 && (reinterpret_cast<uintptr_t>(codes) & 3) == 0 && (reinterpret_cast<uintptr_t>(out) & (4 * sizeof(T) - 1)) == 0;
  for (int64_t r = (int64_t)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5); r < rows; r += (int64_t)gridDim.x * kWarpsPerBlock) {
    const uint8_t* crow = codes + r * cols;
    T* orow = out + r * cols;
    const float s_row = axis == 0 ? scales[r] : 0.0f, z_row = axis == 0 ? zps[r] : 0.0f;
    if (vec) {
      for (int64_t c = (int64_t)lane * 4; c < cols; c += 128) {
        const uint32_t w = *reinterpret_cast<const uint32_t*>(crow + c);
        float o[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const uint32_t b = (w >> (8 * e)) & 0xFFu;
          const float q = signed_codes ? (float)(int)(int8_t)b : (float)b;
          o[e] = __fadd_rn(__fmul_rn(q, axis == 0 ? s_row : scales[c + e]), axis == 0 ? z_row : zps[c + e]);
        }
        if constexpr (sizeof(T) == 4) {
          *reinterpret_cast<float4*>(orow + c) = make_float4(o[0], o[1], o[2], o[3]);
        } else {
          const uint32_t lo = (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(o[0])) | ((uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(o[1])) << 16);
          const uint32_t hi = (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(o[2])) | ((uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(o[3])) << 16);
          *reinterpret_cast<uint2*>(orow + c) = make_uint2(lo, hi);
        }
      }
    } else {
      for (int64_t c = lane; c < cols; c += 32) {
        const uint32_t b = crow[c];
        const float q = signed_codes ? (float)(int)(int8_t)b : (float)b;
        st1<T>(orow, c, __fadd_rn(__fmul_rn(q, axis == 0 ? s_row : scales[c]), axis == 0 ? z_row : zps[c]));
      }
    }
  }
}

inline int grid_cap(const b2q_handle h, int64_t blocks) {
  const int64_t cap = (int64_t)h->sm_count * 16;
  return (int)(blocks < 1 ? 1 : (blocks > cap ? cap : blocks));
}

template <typename T>
int32_t kv_quantize_rows(b2q_handle h, const T* x, int64_t rows, int64_t cols, int rule, int qmin, int qmax, uint8_t* codes,
                         float* scales, float* zps) {
  const bool vec = cols % 4 == 0 && (reinterpret_cast<uintptr_t>(x) % (4 * sizeof(T))) == 0 && (reinterpret_cast<uintptr_t>(codes) & 3) == 0;
  if (vec && cols <= 1024) {
#define KV_REG_LAUNCH(G, NV)                                                                                                                \
  do {                                                                                                                                      \
    const int grid_ = grid_cap(h, ceil_div64(rows, kWarpsPerBlock * (32 / G)));                                                             \
    if (cols == G * NV * 4)                                                                                                                 \
      kv_quantize_per_token_reg_kernel<T, G, NV, true><<<grid_, kThreads, 0, h->stream>>>(x, rows, cols, rule, qmin, qmax, codes, scales, zps); \
    else                                                                                                                                    \
      kv_quantize_per_token_reg_kernel<T, G, NV, false><<<grid_, kThreads, 0, h->stream>>>(x, rows, cols, rule, qmin, qmax, codes, scales, zps); \
  } while (0)
    if (cols <= 32) KV_REG_LAUNCH(4, 2);          // G lanes x NV chunks x 4 elements cover the row
    else if (cols <= 64) KV_REG_LAUNCH(4, 4);
    else if (cols <= 128) KV_REG_LAUNCH(8, 4);
    else if (cols <= 256) KV_REG_LAUNCH(16, 4);
    else if (cols <= 512) KV_REG_LAUNCH(32, 4);
    else KV_REG_LAUNCH(32, 8);
#undef KV_REG_LAUNCH
    B2Q_LAUNCH_CHECK(h, "kv_quantize_per_token_reg_kernel");
    return B2Q_OK;
  }
  const int grid = grid_cap(h, ceil_div64(rows, kWarpsPerBlock));
  if (vec) kv_quantize_per_token_kernel<T, true><<<grid, kThreads, 0, h->stream>>>(x, rows, cols, rule, qmin, qmax, codes, scales, zps);
  else kv_quantize_per_token_kernel<T, false><<<grid, kThreads, 0, h->stream>>>(x, rows, cols, rule, qmin, qmax, codes, scales, zps);
  B2Q_LAUNCH_CHECK(h, "kv_quantize_per_token_kernel");
  return B2Q_OK;
}

template <typename T>
int32_t kv_quantize_channels(b2q_handle h, const T* x, int64_t rows, int64_t cols, int qmax, uint8_t* codes, float* scales, float* zps) {
  const int64_t cols_pad = (cols + 3) & ~(int64_t)3;   // keeps the reciprocals 16-byte aligned
  if ((size_t)(2 * cols_pad + cols) > kScratchWords) B2Q_FAIL(h, B2Q_ERR_UNSUPPORTED, "kv_cache_quantize: per-channel head_dim %lld above %zu", (long long)cols, kScratchWords / 3 - 4);
  uint32_t* keys = h->d_scratch;
  float* inv_scales = reinterpret_cast<float*>(h->d_scratch + 2 * cols_pad);
  kv_channel_keys_init_kernel<<<(unsigned)ceil_div64(cols, kThreads), kThreads, 0, h->stream>>>(keys, cols);
  const int64_t col_blocks = ceil_div64(cols, 32);
  // about 8 blocks per SM over the whole grid, at least 64 rows per block
  int64_t row_blocks = ceil_div64((int64_t)h->sm_count * 8, col_blocks);
  int64_t rows_per_block = ceil_div64(rows, row_blocks);
  if (rows_per_block < 64) rows_per_block = 64;
  row_blocks = ceil_div64(rows, rows_per_block);
  if (row_blocks > 65535) { row_blocks = 65535; rows_per_block = ceil_div64(rows, row_blocks); row_blocks = ceil_div64(rows, rows_per_block); }
  kv_channel_stats_kernel<T><<<dim3((unsigned)col_blocks, (unsigned)row_blocks), kThreads, 0, h->stream>>>(x, rows, cols, rows_per_block, keys);
  kv_channel_params_kernel<<<(unsigned)ceil_div64(cols, kThreads), kThreads, 0, h->stream>>>(keys, cols, (float)qmax, scales, zps, inv_scales);
  const int64_t n = rows * cols;
  const bool vec = cols % 4 == 0 && (reinterpret_cast<uintptr_t>(x) % (4 * sizeof(T))) == 0 && (reinterpret_cast<uintptr_t>(codes) & 3) == 0 &&
                   (reinterpret_cast<uintptr_t>(scales) & 15) == 0 && (reinterpret_cast<uintptr_t>(zps) & 15) == 0;
  if (vec) kv_quantize_per_channel_kernel<T, true><<<grid_cap(h, ceil_div64(n, kThreads * 4)), kThreads, 0, h->stream>>>(x, n, cols, qmax, scales, zps, inv_scales, codes);
  else kv_quantize_per_channel_kernel<T, false><<<grid_cap(h, ceil_div64(n, kThreads)), kThreads, 0, h->stream>>>(x, n, cols, qmax, scales, zps, inv_scales, codes);
  B2Q_LAUNCH_CHECK(h, "kv_quantize_per_channel");
  return B2Q_OK;
}

template <typename T>
int32_t kv_cache_quantize_impl(b2q_handle h, const T* x, int64_t n_tokens, int64_t head_dim, int bits, int axis, uint8_t* codes,
                               float* scales, float* zps) {
  if (n_tokens <= 0 || head_dim <= 0) B2Q_FAIL(h, B2Q_ERR_EMPTY_INPUT, "KvCacheQuantizer::quantize");
  if (bits < 2 || bits > 8) B2Q_FAIL(h, B2Q_ERR_INVALID_BIT_WIDTH, "invalid bit-width %d: must be in [2, 8]", bits);
  if (axis < 0 || axis > 1) B2Q_FAIL(h, B2Q_ERR_INVALID_ARGUMENT, "kv_cache_quantize: axis %d", axis);
  if (!x || !codes || !scales || !zps) B2Q_FAIL(h, B2Q_ERR_INVALID_ARGUMENT, "kv_cache_quantize: null pointer");
  const int qmax = (1 << bits) - 1;
  return axis == 0 ? kv_quantize_rows<T>(h, x, n_tokens, head_dim, kRuleCache, 0, qmax, codes, scales, zps)
                   : kv_quantize_channels<T>(h, x, n_tokens, head_dim, qmax, codes, scales, zps);
}

template <typename T>
int32_t kv_quantize_tokens_impl(b2q_handle h, const T* x, int64_t n_tokens, int64_t d, int bits, int symmetric, uint8_t* codes,
                                float* scales, float* zps) {
  if (bits != 4 && bits != 8) B2Q_FAIL(h, B2Q_ERR_INVALID_CONFIG, "KV quant bits must be 4 or 8");
  if (n_tokens <= 0 || d <= 0) B2Q_FAIL(h, B2Q_ERR_INVALID_CONFIG, "quantize_token: empty vector");
  if (!x || !codes || !scales || !zps) B2Q_FAIL(h, B2Q_ERR_INVALID_ARGUMENT, "kv_quantize_tokens: null pointer");
  const int half = 1 << (bits - 1);
  const int qmin = symmetric ? -(half - 1) : 0, qmax = symmetric ? half - 1 : (1 << bits) - 1;
  return kv_quantize_rows<T>(h, x, n_tokens, d, symmetric ? kRuleTokenSym : kRuleTokenAsym, qmin, qmax, codes, scales, zps);
}

template <typename T>
int32_t kv_dequantize_impl(b2q_handle h, const uint8_t* codes, int64_t n_tokens, int64_t head_dim, int axis, int signed_codes,
                           const float* scales, const float* zps, T* out) {
  if (n_tokens <= 0 || head_dim <= 0) return B2Q_OK;   // an empty cache dequantizes to an empty vector
  if (axis < 0 || axis > 1) B2Q_FAIL(h, B2Q_ERR_INVALID_ARGUMENT, "kv_cache_dequantize: axis %d", axis);
  if (!codes || !scales || !zps || !out) B2Q_FAIL(h, B2Q_ERR_INVALID_ARGUMENT, "kv_cache_dequantize: null pointer");
  const int64_t n = n_tokens * head_dim;
  kv_dequantize_kernel<T><<<grid_cap(h, ceil_div64(n_tokens, kWarpsPerBlock)), kThreads, 0, h->stream>>>(codes, n, head_dim, axis, signed_codes, scales, zps, out);
  B2Q_LAUNCH_CHECK(h, "kv_dequantize_kernel");
  return B2Q_OK;
}

}  // namespace

extern "C" {

int32_t b2q_kv_cache_quantize_f32(b2q_handle h, const float* x, int64_t n_tokens, int64_t head_dim, int bits, int axis,
                                  uint8_t* codes, float* scales, float* zero_points) {
  B2Q_REQUIRE_HANDLE(h);
  return kv_cache_quantize_impl<float>(h, x, n_tokens, head_dim, bits, axis, codes, scales, zero_points);
}
int32_t b2q_kv_cache_quantize_bf16(b2q_handle h, const void* x, int64_t n_tokens, int64_t head_dim, int bits, int axis,
                                   uint8_t* codes, float* scales, float* zero_points) {
  B2Q_REQUIRE_HANDLE(h);
  return kv_cache_quantize_impl<__nv_bfloat16>(h, static_cast<const __nv_bfloat16*>(x), n_tokens, head_dim, bits, axis, codes, scales, zero_points);
}
int32_t b2q_kv_cache_dequantize_f32(b2q_handle h, const uint8_t* codes, int64_t n_tokens, int64_t head_dim, int axis,
                                    const float* scales, const float* zero_points, float* out) {
  B2Q_REQUIRE_HANDLE(h);
  return kv_dequantize_impl<float>(h, codes, n_tokens, head_dim, axis, 0, scales, zero_points, out);
}
int32_t b2q_kv_cache_dequantize_bf16(b2q_handle h, const uint8_t* codes, int64_t n_tokens, int64_t head_dim, int axis,
                                     const float* scales, const float* zero_points, void* out) {
  B2Q_REQUIRE_HANDLE(h);
  return kv_dequantize_impl<__nv_bfloat16>(h, codes, n_tokens, head_dim, axis, 0, scales, zero_points, static_cast<__nv_bfloat16*>(out));
}
int32_t b2q_kv_quantize_tokens_f32(b2q_handle h, const float* x, int64_t n_tokens, int64_t d, int bits, int symmetric,
                                   uint8_t* codes, float* scales, float* zero_points) {
  B2Q_REQUIRE_HANDLE(h);
  return kv_quantize_tokens_impl<float>(h, x, n_tokens, d, bits, symmetric, codes, scales, zero_points);
}
int32_t b2q_kv_quantize_tokens_bf16(b2q_handle h, const void* x, int64_t n_tokens, int64_t d, int bits, int symmetric,
                                    uint8_t* codes, float* scales, float* zero_points) {
  B2Q_REQUIRE_HANDLE(h);
  return kv_quantize_tokens_impl<__nv_bfloat16>(h, static_cast<const __nv_bfloat16*>(x), n_tokens, d, bits, symmetric, codes, scales, zero_points);
}
int32_t b2q_kv_dequantize_tokens_f32(b2q_handle h, const uint8_t* codes, int64_t n_tokens, int64_t d, int symmetric,
                                     const float* scales, const float* zero_points, float* out) {
  B2Q_REQUIRE_HANDLE(h);
  return kv_dequantize_impl<float>(h, codes, n_tokens, d, 0, symmetric ? 1 : 0, scales, zero_points, out);
}
int32_t b2q_kv_dequantize_tokens_bf16(b2q_handle h, const uint8_t* codes, int64_t n_tokens, int64_t d, int symmetric,
                                      const float* scales, const float* zero_points, void* out) {
  B2Q_REQUIRE_HANDLE(h);
  return kv_dequantize_impl<__nv_bfloat16>(h, codes, n_tokens, d, 0, symmetric ? 1 : 0, scales, zero_points, static_cast<__nv_bfloat16*>(out));
}

}  // extern "C"
