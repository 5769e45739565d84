// Quantize / dequantize kernels (HBM-bound byte and integer work): MinMax INT-N,
// FP8 codec + absmax-scaled FP8, block-scaled FP4, NF4, INT8 scalar-scale and the
// dist-infer INT8-in-u8 flavour.  All kernels are grid-stride, 128-bit vectorised
// where the pointers allow it, and launched on the handle's stream.
#include "common.cuh"
#include <cooperative_groups.h>
namespace cg = cooperative_groups;

namespace {

constexpr int kThreads = 256;

inline int grid_for(const b2q_handle h, int64_t work_items, int per_block) {
  int64_t g = ceil_div64(work_items, per_block);
  int64_t cap = (int64_t)h->sm_count * 16;
  if (g > cap) g = cap;
  if (g < 1) g = 1;
  return (int)g;
}

template <typename T> __device__ __forceinline__ float load_as_f32(const T* p, int64_t i);
template <> __device__ __forceinline__ float load_as_f32<float>(const float* p, int64_t i) { return p[i]; }
template <> __device__ __forceinline__ float load_as_f32<__nv_bfloat16>(const __nv_bfloat16* p, int64_t i) {
  return __bfloat162float(p[i]);
}

// ---------------------------------------------------------------------------
// Row statistics.  One warp per row (rows of any length, good up to a few
// thousand columns) or several blocks per row with ordered-key atomics in the
// handle scratch (long rows, e.g. per-tensor over millions of elements).
// NaN never wins a comparison, exactly like the reference's `<` / `>` scan and
// f32::max.  `nonfinite` (optional) is set when an Inf/NaN is seen.
// ---------------------------------------------------------------------------
struct RowStat { float fmin, fmax, amax; int bad; };

template <typename T>
__device__ __forceinline__ RowStat scan_segment(const T* row, int64_t begin, int64_t end, int lane, int stride) {
  RowStat s{__uint_as_float(0x7F800000u), __uint_as_float(0xFF800000u), 0.0f, 0};
  for (int64_t i = begin + lane; i < end; i += stride) {
    float v = load_as_f32<T>(row, i);
    if (v < s.fmin) s.fmin = v;
    if (v > s.fmax) s.fmax = v;
    s.amax = fmaxf(s.amax, fabsf(v));
    s.bad |= !isfinite(v);
  }
  return s;
}

// Specialisation with float4 loads for f32 rows whose start is 16-byte aligned.
__device__ __forceinline__ RowStat scan_segment_f4(const float* row, int64_t n, int lane, int stride) {
  RowStat s{__uint_as_float(0x7F800000u), __uint_as_float(0xFF800000u), 0.0f, 0};
  const float4* r4 = reinterpret_cast<const float4*>(row);
  int64_t n4 = n >> 2;
  for (int64_t i = lane; i < n4; i += stride) {
    float4 q = r4[i];
    float vv[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float v = vv[j];
      if (v < s.fmin) s.fmin = v;
      if (v > s.fmax) s.fmax = v;
      s.amax = fmaxf(s.amax, fabsf(v));
      s.bad |= !isfinite(v);
    }
  }
  for (int64_t i = (n4 << 2) + lane; i < n; i += stride) {
    float v = row[i];
    if (v < s.fmin) s.fmin = v;
    if (v > s.fmax) s.fmax = v;
    s.amax = fmaxf(s.amax, fabsf(v));
    s.bad |= !isfinite(v);
  }
  return s;
}

__device__ __forceinline__ RowStat warp_reduce_stat(RowStat s) {
  s.fmin = warp_min(s.fmin);
  s.fmax = warp_max(s.fmax);
  s.amax = warp_max(s.amax);
  s.bad = __any_sync(0xffffffffu, s.bad) ? 1 : 0;
  return s;
}

// What to do with a finished row statistic.
enum StatMode { kMinMaxParams = 0, kFp8Scale = 1, kAbsmaxOnly = 2 };
struct StatArgs {
  int mode;
  int bits, scheme;        // kMinMaxParams
  float max_val;           // kFp8Scale
  float* scales;           // per-row output (scale or absmax)
  int32_t* zps;            // kMinMaxParams
  int32_t* status;
  int flag_nonfinite;      // record B2Q_ERR_NON_FINITE_FP8 when an Inf/NaN was scanned
};

__device__ __forceinline__ void finish_row(const StatArgs& a, int64_t r, RowStat s) {
  if (a.flag_nonfinite && s.bad) atomicCAS(a.status, 0, (int)B2Q_ERR_NON_FINITE_FP8);
  if (a.mode == kMinMaxParams) {
    float scale; int32_t zp;
    if (a.scheme == 0) {
      float q_max = (float)(1 << (a.bits - 1)) - 1.0f;
      float abs_max = fmaxf(fmaxf(fabsf(s.fmin), fabsf(s.fmax)), 1e-8f);
      scale = __fdiv_rn(abs_max, q_max);
      zp = 0;
    } else {
      float q_range = (float)((1 << a.bits) - 1);
      float range = fmaxf(__fsub_rn(s.fmax, s.fmin), 1e-8f);
      scale = __fdiv_rn(range, q_range);
      float z = roundf(__fdiv_rn(-s.fmin, scale));
      z = z < 0.0f ? 0.0f : (z > q_range ? q_range : z);   // f32::clamp keeps NaN
      zp = isnan(z) ? 0 : (int32_t)z;
    }
    if (!isfinite(scale) || scale <= 0.0f) atomicCAS(a.status, 0, (int)B2Q_ERR_INVALID_SCALE);
    a.scales[r] = scale;
    a.zps[r] = zp;
  } else if (a.mode == kFp8Scale) {
    a.scales[r] = s.amax > 0.0f ? __fdiv_rn(s.amax, a.max_val) : 1.0f;
  } else {
    a.scales[r] = s.amax;
  }
}

template <typename T>
__global__ void __launch_bounds__(kThreads) row_stat_warp_kernel(const T* x, int64_t rows, int64_t cols, StatArgs a) {
  const int lane = threadIdx.x & 31;
  const int64_t warp = (int64_t)blockIdx.x * (kThreads / 32) + (threadIdx.x >> 5);
  const int64_t nwarps = (int64_t)gridDim.x * (kThreads / 32);
  for (int64_t r = warp; r < rows; r += nwarps) {
    const T* row = x + r * cols;
    RowStat s;
    if (sizeof(T) == 4 && ((reinterpret_cast<uintptr_t>(row) & 15) == 0))
      s = scan_segment_f4(reinterpret_cast<const float*>(row), cols, lane, 32);
    else
      s = scan_segment<T>(row, 0, cols, lane, 32);
    s = warp_reduce_stat(s);
    if (lane == 0) finish_row(a, r, s);
  }
}

// Short f32 rows (groups of up to 1024 elements, a multiple of 4, 16-byte aligned): G lanes share a row, so a warp
// works on 32 / G rows at a time with NV 16-byte loads in flight per lane and log2(G) shuffle rounds per row.
template <int G, int NV>
__global__ void __launch_bounds__(kThreads) row_stat_subwarp_kernel(const float* __restrict__ x, int64_t rows, int64_t cols, StatArgs a) {
  constexpr int kRowsPerWarp = 32 / G;
  const int lane = threadIdx.x & 31, sub = lane % G, grp = lane / G;
  const int64_t warp = (int64_t)blockIdx.x * (kThreads / 32) + (threadIdx.x >> 5);
  for (int64_t r0 = warp * kRowsPerWarp; r0 < rows; r0 += (int64_t)gridDim.x * (kThreads / 32) * kRowsPerWarp) {
    const int64_t r = r0 + grp;
    const bool live = r < rows;
    RowStat s{__uint_as_float(0x7F800000u), __uint_as_float(0xFF800000u), 0.0f, 0};
    float4 q[NV];
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      const int64_t c = (int64_t)(sub + G * k) * 4;
      if (live && c < cols) q[k] = *reinterpret_cast<const float4*>(x + r * cols + c);
      else q[k] = make_float4(__uint_as_float(0x7FC00000u), __uint_as_float(0x7FC00000u), __uint_as_float(0x7FC00000u), __uint_as_float(0x7FC00000u));
    }
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      const int64_t c = (int64_t)(sub + G * k) * 4;
      if (live && c < cols) {
        const float vv[4] = {q[k].x, q[k].y, q[k].z, q[k].w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float v = vv[j];
          s.fmin = fminf(s.fmin, v);          // NaN never wins, like the `<` / `>` scan
          s.fmax = fmaxf(s.fmax, v);
          s.amax = fmaxf(s.amax, fabsf(v));
          s.bad |= !isfinite(v);
        }
      }
    }
#pragma unroll
    for (int o = G / 2; o > 0; o >>= 1) {
      s.fmin = fminf(s.fmin, __shfl_xor_sync(0xffffffffu, s.fmin, o));
      s.fmax = fmaxf(s.fmax, __shfl_xor_sync(0xffffffffu, s.fmax, o));
      s.amax = fmaxf(s.amax, __shfl_xor_sync(0xffffffffu, s.amax, o));
      s.bad |= __shfl_xor_sync(0xffffffffu, s.bad, o);
    }
    if (live && sub == 0) finish_row(a, r, s);
  }
}

// keys: [rows][4] = {min key, max key, absmax bits, bad flag}
__global__ void stat_keys_init_kernel(uint32_t* keys, int64_t rows) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < rows) {
    keys[4 * i + 0] = 0xFFFFFFFFu;
    keys[4 * i + 1] = 0u;
    keys[4 * i + 2] = 0u;
    keys[4 * i + 3] = 0u;
  }
}

template <typename T>
__global__ void __launch_bounds__(kThreads) row_stat_split_kernel(const T* x, int64_t cols, int64_t seg, uint32_t* keys) {
  const int64_t r = blockIdx.y;
  const int64_t begin = (int64_t)blockIdx.x * seg;
  const int64_t end = begin + seg < cols ? begin + seg : cols;
  const T* row = x + r * cols;
  RowStat s;
  if (sizeof(T) == 4 && ((reinterpret_cast<uintptr_t>(row + begin) & 15) == 0) && begin < end)
    s = scan_segment_f4(reinterpret_cast<const float*>(row + begin), end - begin, threadIdx.x, kThreads);
  else
    s = scan_segment<T>(row, begin, end, threadIdx.x, kThreads);
  s = warp_reduce_stat(s);
  __shared__ RowStat sh[kThreads / 32];
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < kThreads / 32; ++w) {
      s.fmin = fminf(s.fmin, sh[w].fmin);
      s.fmax = fmaxf(s.fmax, sh[w].fmax);
      s.amax = fmaxf(s.amax, sh[w].amax);
      s.bad |= sh[w].bad;
    }
    atomicMin(&keys[4 * r + 0], float_order_key(s.fmin));
    atomicMax(&keys[4 * r + 1], float_order_key(s.fmax));
    atomicMax(&keys[4 * r + 2], __float_as_uint(s.amax));
    if (s.bad) atomicOr(&keys[4 * r + 3], 1u);
  }
}

__global__ void stat_keys_finish_kernel(const uint32_t* keys, int64_t rows, StatArgs a) {
  int64_t r = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (r < rows) {
    RowStat s{float_from_order_key(keys[4 * r + 0]), float_from_order_key(keys[4 * r + 1]),
              __uint_as_float(keys[4 * r + 2]), (int)keys[4 * r + 3]};
    finish_row(a, r, s);
  }
}

template <typename T>
int32_t launch_row_stats(b2q_handle h, const T* x, int64_t rows, int64_t cols, const StatArgs& a) {
  if constexpr (sizeof(T) == 4) {
    if (cols % 4 == 0 && cols <= 1024 && rows >= 256 && (reinterpret_cast<uintptr_t>(x) & 15) == 0) {
      const float* xf = reinterpret_cast<const float*>(x);
#define STAT_SUBWARP(G, NV) \
  row_stat_subwarp_kernel<G, NV><<<grid_for(h, rows, (kThreads / 32) * (32 / G)), kThreads, 0, h->stream>>>(xf, rows, cols, a)
      if (cols <= 32) STAT_SUBWARP(4, 2);
      else if (cols <= 64) STAT_SUBWARP(4, 4);
      else if (cols <= 128) STAT_SUBWARP(8, 4);
      else if (cols <= 256) STAT_SUBWARP(16, 4);
      else if (cols <= 512) STAT_SUBWARP(32, 4);
      else STAT_SUBWARP(32, 8);
#undef STAT_SUBWARP
      B2Q_LAUNCH_CHECK(h, "row_stat_subwarp_kernel");
      return B2Q_OK;
    }
  }
  const bool split = cols >= (1 << 15) && rows * 4 <= (int64_t)kScratchWords && rows <= 65535;
  if (!split) {
    int grid = grid_for(h, rows, kThreads / 32);
    row_stat_warp_kernel<T><<<grid, kThreads, 0, h->stream>>>(x, rows, cols, a);
    B2Q_LAUNCH_CHECK(h, "row_stat_warp_kernel");
    return B2Q_OK;
  }
  int64_t want_blocks = (int64_t)h->sm_count * 8;
  int64_t bpr = ceil_div64(want_blocks, rows);
  int64_t seg = ceil_div64(cols, bpr);
  seg = ceil_div64(seg, 4 * kThreads) * 4 * kThreads;     // keeps segment starts 16-byte aligned
  bpr = ceil_div64(cols, seg);
  stat_keys_init_kernel<<<(int)ceil_div64(rows, 256), 256, 0, h->stream>>>(h->d_scratch, rows);
  row_stat_split_kernel<T><<<dim3((unsigned)bpr, (unsigned)rows), kThreads, 0, h->stream>>>(x, cols, seg, h->d_scratch);
  stat_keys_finish_kernel<<<(int)ceil_div64(rows, 256), 256, 0, h->stream>>>(h->d_scratch, rows, a);
  B2Q_LAUNCH_CHECK(h, "row_stat_split_kernel");
  return B2Q_OK;
}

// ---------------------------------------------------------------------------
// MinMax quantize / dequantize / fake-quant
// ---------------------------------------------------------------------------
__device__ __forceinline__ int32_t minmax_code(float v, float scale, float zp, float q_min, float q_max) {
  float t = roundf(__fadd_rn(__fdiv_rn(v, scale), zp));
  t = t < q_min ? q_min : (t > q_max ? q_max : t);
  return isnan(t) ? 0 : (int32_t)t;
}
// vec_ok: cols % 4 == 0 and 16-byte aligned pointers, so four consecutive elements share a row
__global__ void __launch_bounds__(kThreads) minmax_quantize_kernel(const float* __restrict__ x, int64_t n, int64_t cols,
                                                                   const float* __restrict__ scales, const int32_t* __restrict__ zps,
                                                                   float q_min, float q_max, int32_t* __restrict__ codes, int vec_ok) {
  const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x, nth = (int64_t)gridDim.x * blockDim.x;
  if (vec_ok) {
    const int64_t c4 = cols >> 2;
    for (int64_t i = tid; i < (n >> 2); i += nth) {
      const int64_t r = c4 == (n >> 2) ? 0 : i / c4;
      const float s = scales[r], z = (float)zps[r];
      const float4 q = reinterpret_cast<const float4*>(x)[i];
      reinterpret_cast<int4*>(codes)[i] = make_int4(minmax_code(q.x, s, z, q_min, q_max), minmax_code(q.y, s, z, q_min, q_max),
                                                    minmax_code(q.z, s, z, q_min, q_max), minmax_code(q.w, s, z, q_min, q_max));
    }
    return;
  }
  for (int64_t i = tid; i < n; i += nth) {
    const int64_t r = i / cols;
    codes[i] = minmax_code(x[i], scales[r], (float)zps[r], q_min, q_max);
  }
}
__global__ void __launch_bounds__(kThreads) minmax_dequantize_kernel(const int32_t* __restrict__ codes, int64_t n, int64_t cols,
                                                                     const float* __restrict__ scales, const int32_t* __restrict__ zps,
                                                                     float* __restrict__ out, int vec_ok) {
  const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x, nth = (int64_t)gridDim.x * blockDim.x;
  if (vec_ok) {
    const int64_t c4 = cols >> 2;
    for (int64_t i = tid; i < (n >> 2); i += nth) {
      const int64_t r = c4 == (n >> 2) ? 0 : i / c4;
      const float s = scales[r];
      const uint32_t z = (uint32_t)zps[r];
      const int4 c = reinterpret_cast<const int4*>(codes)[i];
      reinterpret_cast<float4*>(out)[i] = make_float4(__fmul_rn((float)(int32_t)((uint32_t)c.x - z), s), __fmul_rn((float)(int32_t)((uint32_t)c.y - z), s),
                                                      __fmul_rn((float)(int32_t)((uint32_t)c.z - z), s), __fmul_rn((float)(int32_t)((uint32_t)c.w - z), s));
    }
    return;
  }
  for (int64_t i = tid; i < n; i += nth) {
    int64_t r = i / cols;
    int32_t d = (int32_t)((uint32_t)codes[i] - (uint32_t)zps[r]);
    out[i] = __fmul_rn((float)d, scales[r]);
  }
}
__device__ __forceinline__ float fake_quant_one(float v, float scale, float zp, float qmin, float qmax) {
  float q = roundf(__fadd_rn(__fdiv_rn(v, scale), zp));
  q = q < qmin ? qmin : (q > qmax ? qmax : q);
  return __fmul_rn(__fsub_rn(q, zp), scale);
}
__global__ void __launch_bounds__(kThreads) fake_quant_kernel(float* x, int64_t n, float scale, float zp, float qmin, float qmax) {
  const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x, nth = (int64_t)gridDim.x * blockDim.x;
  const int64_t n4 = (reinterpret_cast<uintptr_t>(x) & 15) == 0 ? n >> 2 : 0;
  for (int64_t i = tid; i < n4; i += nth) {
    float4 v = reinterpret_cast<float4*>(x)[i];
    v.x = fake_quant_one(v.x, scale, zp, qmin, qmax);
    v.y = fake_quant_one(v.y, scale, zp, qmin, qmax);
    v.z = fake_quant_one(v.z, scale, zp, qmin, qmax);
    v.w = fake_quant_one(v.w, scale, zp, qmin, qmax);
    reinterpret_cast<float4*>(x)[i] = v;
  }
  for (int64_t i = (n4 << 2) + tid; i < n; i += nth) x[i] = fake_quant_one(x[i], scale, zp, qmin, qmax);
}

// ---------------------------------------------------------------------------
// FP8 encode / decode
// ---------------------------------------------------------------------------
// SCALED: divide by scales[row] first.  Four elements per thread when aligned.
template <typename T, bool SCALED>
__global__ void __launch_bounds__(kThreads) fp8_encode_kernel(const T* x, int64_t n, int64_t cols, const float* scales,
                                                              int fmt, int rounding, uint8_t* codes, int32_t* status,
                                                              int vec_ok) {
  const Fp8Fmt F = fp8_fmt(fmt);
  const bool one_slice = cols >= n;               // per-tensor: no row index to derive
  const float scale0 = SCALED ? scales[0] : 1.0f;
  auto enc1 = [&](float v, int64_t idx) -> uint32_t {
    if (!isfinite(v)) { atomicCAS(status, 0, (int)B2Q_ERR_NON_FINITE_FP8); }
    if (SCALED) v = __fdiv_rn(v, one_slice ? scale0 : scales[idx / cols]);
    v = v < -F.max_val ? -F.max_val : (v > F.max_val ? F.max_val : v);
    return rounding == 0 ? fp8_encode_ref_dev(v, F) : fp8_encode_rne_dev(v, fmt);
  };
  const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t nth = (int64_t)gridDim.x * blockDim.x;
  if (vec_ok) {
    const int64_t n4 = n >> 2;
    for (int64_t i = tid; i < n4; i += nth) {
      float v[4];
      if (sizeof(T) == 4) {
        float4 q = reinterpret_cast<const float4*>(x)[i];
        v[0] = q.x; v[1] = q.y; v[2] = q.z; v[3] = q.w;
      } else {
        uint2 q = reinterpret_cast<const uint2*>(x)[i];
        v[0] = __uint_as_float(q.x << 16); v[1] = __uint_as_float(q.x & 0xFFFF0000u);
        v[2] = __uint_as_float(q.y << 16); v[3] = __uint_as_float(q.y & 0xFFFF0000u);
      }
      uint32_t w = 0;
#pragma unroll
      for (int j = 0; j < 4; ++j) w |= enc1(v[j], 4 * i + j) << (8 * j);
      reinterpret_cast<uint32_t*>(codes)[i] = w;
    }
    for (int64_t i = (n4 << 2) + tid; i < n; i += nth) codes[i] = (uint8_t)enc1(load_as_f32<T>(x, i), i);
  } else {
    for (int64_t i = tid; i < n; i += nth) codes[i] = (uint8_t)enc1(load_as_f32<T>(x, i), i);
  }
}

__global__ void __launch_bounds__(kThreads) fp8_decode_kernel(const uint8_t* codes, int64_t n, int fmt, int mode, float* out) {
  __shared__ float lut[256];
  const Fp8Fmt F = fp8_fmt(fmt);
  for (int i = threadIdx.x; i < 256; i += blockDim.x)
    lut[i] = mode == 0 ? fp8_decode_ref_dev((uint32_t)i, F) : fp8_decode_ieee_dev((uint32_t)i, F);
  __syncthreads();
  const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t nth = (int64_t)gridDim.x * blockDim.x;
  const bool vec = ((reinterpret_cast<uintptr_t>(codes) & 3) == 0) && ((reinterpret_cast<uintptr_t>(out) & 15) == 0);
  if (vec) {
    const int64_t n4 = n >> 2;
    for (int64_t i = tid; i < n4; i += nth) {
      uint32_t w = reinterpret_cast<const uint32_t*>(codes)[i];
      reinterpret_cast<float4*>(out)[i] =
          make_float4(lut[w & 0xFF], lut[(w >> 8) & 0xFF], lut[(w >> 16) & 0xFF], lut[w >> 24]);
    }
    for (int64_t i = (n4 << 2) + tid; i < n; i += nth) out[i] = lut[codes[i]];
  } else {
    for (int64_t i = tid; i < n; i += nth) out[i] = lut[codes[i]];
  }
}

// Rewrites the subnormal codes (exponent field 0, mantissa m != 0) to exponent field 1 with the same
// mantissa.  The reference decoder reads a subnormal code as 2^(1-bias) * (1 + m/2^mb), which is exactly
// the IEEE value of that rewritten code, so a tensor-core GEMM over rewritten codes multiplies the very
// values the reference's decode -> f32 matmul composition multiplies.
__global__ void __launch_bounds__(kThreads) fp8_remap_ref_subnormals_kernel(uint8_t* codes, int64_t n, int fmt) {
  const uint32_t mb = fmt == 0 ? 3u : 2u;
  const uint32_t exp_mask = fmt == 0 ? 0x78u : 0x7Cu, man_mask = (1u << mb) - 1u;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    uint32_t c = codes[i];
    if ((c & exp_mask) == 0 && (c & man_mask) != 0) codes[i] = (uint8_t)(c | (1u << mb));
  }
}

// ---------------------------------------------------------------------------
// Block-scaled FP4.  block/4 lanes cooperate on one block: each lane loads one
// float4, the absmax is reduced with xor-shuffles inside the lane group, and each
// lane emits two bytes (four codes).  A warp therefore reads 512 contiguous bytes
// per instruction and writes 64.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(kThreads) fp4_block_quantize_kernel(const float* x, int64_t n, int block, int format,
                                                                      int scale_format, uint8_t* packed,
                                                                      float* scales_f32, uint8_t* scales_e8m0) {
  const int lanes = block >> 2;                               // 8, 16 or 32
  const float target = format == 0 ? 6.0f : 8.0f;
  const int64_t n4 = n >> 2;                                  // n is a multiple of block
  const int64_t span = (int64_t)gridDim.x * blockDim.x;
  // every lane of a warp runs the same number of iterations (n4 is a multiple of `lanes`, span of 32)
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < ((n4 + 31) & ~(int64_t)31); i += span) {
    const bool live = i < n4;
    float4 q = live ? reinterpret_cast<const float4*>(x)[i] : make_float4(0.f, 0.f, 0.f, 0.f);
    float amax = fmaxf(fmaxf(fabsf(q.x), fabsf(q.y)), fmaxf(fabsf(q.z), fabsf(q.w)));
    for (int o = lanes >> 1; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    float scale;
    uint32_t eb = 127;
    float inv_pow2 = 0.0f;   // E8M0: dividing by 2^e is multiplying by 2^-e, exactly (both are representable for every scale byte)
    if (scale_format == 0) scale = amax == 0.0f ? 1.0f : __fdiv_rn(amax, target);
    else { eb = e8m0_from_absmax_dev(amax); scale = e8m0_to_f32_dev(eb); inv_pow2 = e8m0_to_f32_dev(254u - eb); }
    if (live) {
      float v[4] = {q.x, q.y, q.z, q.w};
      uint32_t c[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float s = scale_format == 0 ? __fdiv_rn(v[j], scale) : __fmul_rn(v[j], inv_pow2);
        c[j] = format == 0 ? e2m1_encode_ref_dev(s) : int4_encode_ref_dev(s);
      }
      reinterpret_cast<uint16_t*>(packed)[i] = (uint16_t)(c[0] | (c[1] << 4) | (c[2] << 8) | (c[3] << 12));
      if ((i & (lanes - 1)) == 0) {                       // lanes is 8, 16 or 32
        int64_t b = i >> (lanes == 8 ? 3 : (lanes == 16 ? 4 : 5));
        if (scale_format == 0) scales_f32[b] = scale; else scales_e8m0[b] = (uint8_t)eb;
      }
    }
  }
}

__global__ void __launch_bounds__(kThreads) fp4_block_dequantize_kernel(const uint8_t* packed, int64_t n, int block,
                                                                        int format, int scale_format,
                                                                        const float* scales_f32,
                                                                        const uint8_t* scales_e8m0, float* out) {
  const int64_t n4 = n >> 2;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (int64_t)gridDim.x * blockDim.x) {
    uint32_t w = reinterpret_cast<const uint16_t*>(packed)[i];
    int64_t b = (block & (block - 1)) == 0 ? (4 * i) >> (31 - __clz(block)) : (4 * i) / block;
    float scale = scale_format == 0 ? scales_f32[b] : e8m0_to_f32_dev(scales_e8m0[b]);
    float r[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      uint32_t c = (w >> (4 * j)) & 0xF;
      r[j] = __fmul_rn(format == 0 ? e2m1_decode_dev(c) : int4_decode_dev(c), scale);
    }
    reinterpret_cast<float4*>(out)[i] = make_float4(r[0], r[1], r[2], r[3]);
  }
}

// ---------------------------------------------------------------------------
// NF4
// ---------------------------------------------------------------------------
__constant__ float kNf4Lut[16] = {
    -1.0f, -0.69619286f, -0.52507305f, -0.3949175f, -0.28444138f, -0.18477343f, -0.09105003f, 0.0f,
    0.0795803f, 0.1609302f, 0.2461123f, 0.33791524f, 0.44070983f, 0.562617f, 0.72295684f, 1.0f};

__global__ void __launch_bounds__(kThreads) nf4_decode_kernel(const uint8_t* packed, int64_t nbytes, int block,
                                                              const float* absmaxs, float* out) {
  __shared__ float lut[16];
  if (threadIdx.x < 16) lut[threadIdx.x] = kNf4Lut[threadIdx.x];
  __syncthreads();
  const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x, nth = (int64_t)gridDim.x * blockDim.x;
  // four bytes (eight values of one block) per thread when the block size and the pointers allow it
  const bool vec = block % 8 == 0 && (reinterpret_cast<uintptr_t>(packed) & 3) == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0;
  const int64_t n4 = vec ? nbytes >> 2 : 0;
  const bool pow2 = (block & (block - 1)) == 0;          // block index by a shift where the block size allows it
  const int bsh = 31 - __clz(block);
  for (int64_t i = tid; i < n4; i += nth) {
    const uint32_t w = reinterpret_cast<const uint32_t*>(packed)[i];
    const float amax = absmaxs[pow2 ? (8 * i) >> bsh : (8 * i) / block];
    reinterpret_cast<float4*>(out)[2 * i] = make_float4(__fmul_rn(lut[w & 0xF], amax), __fmul_rn(lut[(w >> 4) & 0xF], amax),
                                                        __fmul_rn(lut[(w >> 8) & 0xF], amax), __fmul_rn(lut[(w >> 12) & 0xF], amax));
    reinterpret_cast<float4*>(out)[2 * i + 1] = make_float4(__fmul_rn(lut[(w >> 16) & 0xF], amax), __fmul_rn(lut[(w >> 20) & 0xF], amax),
                                                            __fmul_rn(lut[(w >> 24) & 0xF], amax), __fmul_rn(lut[w >> 28], amax));
  }
  for (int64_t i = (n4 << 2) + tid; i < nbytes; i += nth) {
    uint32_t b = packed[i];
    float amax = absmaxs[(2 * i) / block];
    reinterpret_cast<float2*>(out)[i] = make_float2(__fmul_rn(lut[b & 0xF], amax), __fmul_rn(lut[b >> 4], amax));
  }
}

__device__ __forceinline__ uint32_t nearest_nf4_dev(const float* lut, float v) {
  int lo = 0, hi = 16;
  while (lo < hi) {
    int mid = lo + (hi - lo) / 2;
    if (lut[mid] < v) lo = mid + 1; else hi = mid;
  }
  if (lo == 0) return 0;
  if (lo == 16) return 15;
  float d_lo = fabsf(__fsub_rn(v, lut[lo - 1]));
  float d_hi = fabsf(__fsub_rn(lut[lo], v));
  return d_lo <= d_hi ? lo - 1 : lo;
}

// Blocks of 32, 64, 128 or 256 elements, 16-byte aligned input: G = block / 8 lanes share a block, eight elements (two
// 16-byte loads) and one 4-byte store per lane, log2(G) shuffle rounds for the block maximum.  Same arithmetic as the
// warp-per-block kernel below.
template <int G>
__global__ void __launch_bounds__(kThreads) nf4_encode_subwarp_kernel(const float* __restrict__ x, int64_t nblocks, uint8_t* __restrict__ packed,
                                                                      float* __restrict__ absmaxs) {
  __shared__ float lut[16];
  if (threadIdx.x < 16) lut[threadIdx.x] = kNf4Lut[threadIdx.x];
  __syncthreads();
  constexpr int kPerWarp = 32 / G;
  const int lane = threadIdx.x & 31, sub = lane % G, grp = lane / G;
  const int64_t warp = (int64_t)blockIdx.x * (kThreads / 32) + (threadIdx.x >> 5);
  for (int64_t b0 = warp * kPerWarp; b0 < nblocks; b0 += (int64_t)gridDim.x * (kThreads / 32) * kPerWarp) {
    const int64_t b = b0 + grp;
    const bool live = b < nblocks;
    float v[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    if (live) {
      const float4* p = reinterpret_cast<const float4*>(x + b * (G * 8) + sub * 8);
      const float4 q0 = p[0], q1 = p[1];
      v[0] = q0.x; v[1] = q0.y; v[2] = q0.z; v[3] = q0.w; v[4] = q1.x; v[5] = q1.y; v[6] = q1.z; v[7] = q1.w;
    }
    float amax = 0.0f;
#pragma unroll
    for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(v[j]));
#pragma unroll
    for (int o = G / 2; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    if (amax < 1e-8f) amax = 1e-8f;
    if (!live) continue;
    if (sub == 0) absmaxs[b] = amax;
    uint32_t w = 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float a = __fdiv_rn(v[j], amax);
      a = a < -1.0f ? -1.0f : (a > 1.0f ? 1.0f : a);
      w |= nearest_nf4_dev(lut, a) << (4 * j);
    }
    reinterpret_cast<uint32_t*>(packed)[b * G + sub] = w;
  }
}

// one warp per block of `block` (even) elements
__global__ void __launch_bounds__(kThreads) nf4_encode_kernel(const float* x, int64_t nblocks, int block, uint8_t* packed,
                                                              float* absmaxs) {
  __shared__ float lut[16];
  if (threadIdx.x < 16) lut[threadIdx.x] = kNf4Lut[threadIdx.x];
  __syncthreads();
  const int lane = threadIdx.x & 31;
  const int64_t warp = (int64_t)blockIdx.x * (kThreads / 32) + (threadIdx.x >> 5);
  const int64_t nwarps = (int64_t)gridDim.x * (kThreads / 32);
  for (int64_t b = warp; b < nblocks; b += nwarps) {
    const float* s = x + b * block;
    float amax = 0.0f;
    for (int i = lane; i < block; i += 32) amax = fmaxf(amax, fabsf(s[i]));
    amax = warp_max(amax);
    if (amax < 1e-8f) amax = 1e-8f;
    if (lane == 0) absmaxs[b] = amax;
    for (int p = lane; p < block / 2; p += 32) {
      float a = __fdiv_rn(s[2 * p], amax), c = __fdiv_rn(s[2 * p + 1], amax);
      a = a < -1.0f ? -1.0f : (a > 1.0f ? 1.0f : a);
      c = c < -1.0f ? -1.0f : (c > 1.0f ? 1.0f : c);
      packed[b * (block / 2) + p] = (uint8_t)(nearest_nf4_dev(lut, a) | (nearest_nf4_dev(lut, c) << 4));
    }
  }
}

// ---------------------------------------------------------------------------
// INT8 with a scalar scale (quant: ties-to-even as cvt.rni, clamp +-127)
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t int8_quant_one(float v, float scale) {
  float t = rintf(__fdiv_rn(v, scale));
  t = fminf(fmaxf(t, -127.0f), 127.0f);
  return (uint32_t)(int)t & 0xFFu;
}
__global__ void __launch_bounds__(kThreads) int8_quant_kernel(const float* __restrict__ x, int64_t n, float scale, int8_t* __restrict__ out, int vec_ok) {
  const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x, nth = (int64_t)gridDim.x * blockDim.x;
  const int64_t n4 = vec_ok ? n >> 2 : 0;
  for (int64_t i = tid; i < n4; i += nth) {
    const float4 q = reinterpret_cast<const float4*>(x)[i];
    reinterpret_cast<uint32_t*>(out)[i] = int8_quant_one(q.x, scale) | (int8_quant_one(q.y, scale) << 8) | (int8_quant_one(q.z, scale) << 16) |
                                          (int8_quant_one(q.w, scale) << 24);
  }
  for (int64_t i = (n4 << 2) + tid; i < n; i += nth) out[i] = (int8_t)int8_quant_one(x[i], scale);
}
__global__ void __launch_bounds__(kThreads) int8_dequant_kernel(const int8_t* __restrict__ q, int64_t n, float scale, float* __restrict__ out, int vec_ok) {
  const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x, nth = (int64_t)gridDim.x * blockDim.x;
  const int64_t n4 = vec_ok ? n >> 2 : 0;
  for (int64_t i = tid; i < n4; i += nth) {
    const uint32_t w = reinterpret_cast<const uint32_t*>(q)[i];
    reinterpret_cast<float4*>(out)[i] = make_float4(__fmul_rn((float)(int8_t)(w & 0xFF), scale), __fmul_rn((float)(int8_t)((w >> 8) & 0xFF), scale),
                                                    __fmul_rn((float)(int8_t)((w >> 16) & 0xFF), scale), __fmul_rn((float)(int8_t)(w >> 24), scale));
  }
  for (int64_t i = (n4 << 2) + tid; i < n; i += nth) out[i] = __fmul_rn((float)q[i], scale);
}

// ---------------------------------------------------------------------------
// dist-infer INT8-in-u8 ("fp8_infer"): q = round(clamp(v*(127/absmax), +-127)) as i8 as u8
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t distfp8_code(float v, float amax, float scale) {
  if (amax == 0.0f) return 0u;
  float t = __fmul_rn(v, scale);
  t = t < -127.0f ? -127.0f : (t > 127.0f ? 127.0f : t);
  t = roundf(t);
  return (uint32_t)(isnan(t) ? 0 : (int)t) & 0xFFu;
}
// vec_ok: block % 4 == 0 and aligned pointers, so four consecutive elements share a block (one index division and one
// scale division per four elements)
__global__ void __launch_bounds__(kThreads) distfp8_quantize_kernel(const float* __restrict__ x, int64_t n, int64_t block,
                                                                    const float* __restrict__ absmaxs, uint8_t* __restrict__ q, int vec_ok) {
  const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x, nth = (int64_t)gridDim.x * blockDim.x;
  const int64_t n4 = vec_ok ? n >> 2 : 0;
  for (int64_t i = tid; i < n4; i += nth) {
    const float amax = absmaxs[(4 * i) / block];
    const float scale = __fdiv_rn(127.0f, amax);
    const float4 v = reinterpret_cast<const float4*>(x)[i];
    reinterpret_cast<uint32_t*>(q)[i] = distfp8_code(v.x, amax, scale) | (distfp8_code(v.y, amax, scale) << 8) |
                                        (distfp8_code(v.z, amax, scale) << 16) | (distfp8_code(v.w, amax, scale) << 24);
  }
  for (int64_t i = (n4 << 2) + tid; i < n; i += nth) {
    const float amax = absmaxs[i / block];
    q[i] = (uint8_t)distfp8_code(x[i], amax, __fdiv_rn(127.0f, amax));
  }
}
__global__ void __launch_bounds__(kThreads) distfp8_dequantize_kernel(const uint8_t* __restrict__ q, int64_t n, int64_t block,
                                                                      const float* __restrict__ absmaxs, float* __restrict__ out, int vec_ok) {
  const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x, nth = (int64_t)gridDim.x * blockDim.x;
  const int64_t n4 = vec_ok ? n >> 2 : 0;      // block % 4 == 0: four consecutive elements share a block
  for (int64_t i = tid; i < n4; i += nth) {
    const float s = __fdiv_rn(absmaxs[(4 * i) / block], 127.0f);
    const uint32_t w = reinterpret_cast<const uint32_t*>(q)[i];
    reinterpret_cast<float4*>(out)[i] = make_float4(__fmul_rn((float)(int8_t)(w & 0xFF), s), __fmul_rn((float)(int8_t)((w >> 8) & 0xFF), s),
                                                    __fmul_rn((float)(int8_t)((w >> 16) & 0xFF), s), __fmul_rn((float)(int8_t)(w >> 24), s));
  }
  for (int64_t i = (n4 << 2) + tid; i < n; i += nth)
    out[i] = __fmul_rn((float)(int8_t)q[i], __fdiv_rn(absmaxs[i / block], 127.0f));
}

// Few long rows (per-token quantization of a decode step): one CTA of 1024 threads per row does the statistics and the
// encoding in one launch, with the arithmetic of the two-kernel path (finish_row, then divide, clamp, encode).
template <typename T>
__global__ void __launch_bounds__(1024) fp8_quantize_rows_fused_kernel(const T* x, int64_t cols, StatArgs a, int fmt, int rounding,
                                                                       uint8_t* codes) {
  __shared__ RowStat sh[32];
  __shared__ float s_scale;
  b2q_pdl_entry();
  const int64_t r = blockIdx.x;
  const T* row = x + r * cols;
  RowStat s = scan_segment<T>(row, 0, cols, (int)threadIdx.x, (int)blockDim.x);
  s = warp_reduce_stat(s);
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x < 32) {
    RowStat t = threadIdx.x < (blockDim.x >> 5) ? sh[threadIdx.x] : RowStat{__uint_as_float(0x7F800000u), __uint_as_float(0xFF800000u), 0.0f, 0};
    t = warp_reduce_stat(t);
    if (threadIdx.x == 0) {
      finish_row(a, r, t);
      s_scale = a.scales[r];
    }
  }
  __syncthreads();
  const float scale = s_scale;
  const Fp8Fmt F = fp8_fmt(fmt);
  uint8_t* out = codes + r * cols;
  for (int64_t i = threadIdx.x; i < cols; i += blockDim.x) {
    float v = __fdiv_rn(load_as_f32<T>(row, i), scale);
    v = v < -F.max_val ? -F.max_val : (v > F.max_val ? F.max_val : v);
    out[i] = (uint8_t)(rounding == 0 ? fp8_encode_ref_dev(v, F) : fp8_encode_rne_dev(v, fmt));
  }
}

// Many rows of up to 65536 elements (per-token quantization of a prefill batch): one CTA per row keeps the row in
// registers (thread t holds chunks t, t + blockDim, ... of 8 elements), so the input is read once and nothing is
// divided per element but the value itself.  Same arithmetic as the two-kernel path (finish_row, divide, clamp, encode).
template <typename T> __device__ __forceinline__ void load_chunk8(const T* row, int c, float (&v)[8]);
template <> __device__ __forceinline__ void load_chunk8<float>(const float* row, int c, float (&v)[8]) {
  const float4 a = reinterpret_cast<const float4*>(row)[2 * c], b = reinterpret_cast<const float4*>(row)[2 * c + 1];
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
template <> __device__ __forceinline__ void load_chunk8<__nv_bfloat16>(const __nv_bfloat16* row, int c, float (&v)[8]) {
  const uint4 q = reinterpret_cast<const uint4*>(row)[c];
  const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
  for (int j = 0; j < 4; ++j) { v[2 * j] = __uint_as_float(w[j] << 16); v[2 * j + 1] = __uint_as_float(w[j] & 0xFFFF0000u); }
}

// RNE codes of x / scale without a division where that is provably the same.  r_lo and r_hi are RN(1 / scale)
// narrowed and widened by 2^-21: the exact quotient lies between x * r_lo and x * r_hi (three roundings of 2^-24 each
// against a margin of 2^-21), the saturating conversion is monotonic, so if both ends convert to the same code every
// value between them does.  Otherwise (a quotient within 2^-20 of a rounding boundary) the IEEE division decides.
// (x0, x1) * r in one instruction: the packed fp32 multiply of sm_100 (each lane rounded to nearest even, as __fmul_rn).
__device__ __forceinline__ float2 mul2_rn(float x0, float x1, float r) {
  float2 o;
  asm("{\n\t.reg .b64 a, b, c;\n\tmov.b64 a, {%2, %3};\n\tmov.b64 b, {%4, %4};\n\tmul.rn.f32x2 c, a, b;\n\tmov.b64 {%0, %1}, c;\n\t}"
      : "=f"(o.x), "=f"(o.y) : "f"(x0), "f"(x1), "f"(r));
  return o;
}
// Eight RNE codes of v / scale.  With the bracket: both ends of every pair are converted and compared once per eight
// values; if any pair disagrees (about one chunk in 10^4) the eight are divided.  The format is a template parameter so
// that one conversion instruction is emitted, not a selection between two.
template <bool E5M2>
__device__ __forceinline__ void fp8x8_quotient_rne(const float (&v)[8], float scale, float r_lo, float r_hi, bool bracket, uint32_t& lo, uint32_t& hi) {
  constexpr __nv_fp8_interpretation_t f = E5M2 ? __NV_E5M2 : __NV_E4M3;
  uint32_t p[4];
  bool redo = !bracket;
  if (bracket) {
    uint32_t diff = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      p[j] = (uint32_t)__nv_cvt_float2_to_fp8x2(mul2_rn(v[2 * j], v[2 * j + 1], r_lo), __NV_SATFINITE, f);
      diff |= p[j] ^ (uint32_t)__nv_cvt_float2_to_fp8x2(mul2_rn(v[2 * j], v[2 * j + 1], r_hi), __NV_SATFINITE, f);
    }
    redo = diff != 0;
  }
  if (redo) {
#pragma unroll
    for (int j = 0; j < 4; ++j)
      p[j] = (uint32_t)__nv_cvt_float2_to_fp8x2(make_float2(__fdiv_rn(v[2 * j], scale), __fdiv_rn(v[2 * j + 1], scale)), __NV_SATFINITE, f);
  }
  lo = __byte_perm(p[0], p[1], 0x5410);
  hi = __byte_perm(p[2], p[3], 0x5410);
}
// The bracket needs a normal scale and a normal reciprocal; rows outside (all-zero rows have scale 1) divide.
__device__ __forceinline__ bool quotient_bracket(float scale, float& r_lo, float& r_hi) {
  const float r = __frcp_rn(scale);
  r_lo = __fmul_rn(r, 1.0f - 4.76837158203125e-7f);          // 1 - 2^-21
  r_hi = __fmul_rn(r, 1.0f + 4.76837158203125e-7f);
  return scale > 1e-30f && scale < 1e30f;
}

// raw chunk of 8 elements: two float4 (f32) or one uint4 (bf16)
template <typename T> struct RawChunk;
template <> struct RawChunk<float> {
  float4 a, b;
  __device__ __forceinline__ void load(const float* row, int c) { a = reinterpret_cast<const float4*>(row)[2 * c]; b = reinterpret_cast<const float4*>(row)[2 * c + 1]; }
  __device__ __forceinline__ void get(float (&v)[8]) const { v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w; }
  // |x| as an integer: NaN and infinities compare above every finite value, so one maximum finds both the absmax and bad input
  __device__ __forceinline__ uint32_t amax_bits(uint32_t m) const {
    const float v[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
    for (int j = 0; j < 8; ++j) m = max(m, __float_as_uint(v[j]) & 0x7FFFFFFFu);
    return m;
  }
};
template <> struct RawChunk<__nv_bfloat16> {
  uint4 q;
  __device__ __forceinline__ void load(const __nv_bfloat16* row, int c) { q = reinterpret_cast<const uint4*>(row)[c]; }
  __device__ __forceinline__ void get(float (&v)[8]) const {
    const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) { v[2 * j] = __uint_as_float(w[j] << 16); v[2 * j + 1] = __uint_as_float(w[j] & 0xFFFF0000u); }
  }
  // two bf16 lanes per word: one packed maximum per word (NaN propagates, so a NaN or an infinity ends up in the
  // result and is caught by the same integer comparison as in the f32 case)
  __device__ __forceinline__ uint32_t amax_bits(uint32_t m) const {
    const uint32_t w[4] = {q.x, q.y, q.z, q.w};
    __nv_bfloat162 acc = *reinterpret_cast<const __nv_bfloat162*>(&m);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const uint32_t a = w[j] & 0x7FFF7FFFu;
      acc = __hmax2_nan(acc, *reinterpret_cast<const __nv_bfloat162*>(&a));
    }
    return *reinterpret_cast<const uint32_t*>(&acc);
  }
};

// FULL: every thread has all NCH chunks (cols == 8 * NCH * blockDim), so the bounds predicates drop out.
// A CTA walks rows blockIdx.x, blockIdx.x + gridDim.x, ...  PIPE (long rows, CTAs of 512 threads or more, of which only one or
// two fit an SM): the NEXT row's chunks are fetched before the current row is reduced and encoded, so loads stay in flight
// through the barrier (4096 x 28672 bf16: 105 -> 88 us).  Short rows run one row per CTA with many CTAs per SM, where the
// second register set only costs occupancy (8192 x 8192 bf16: 45 us without, 50 us with).
template <typename T, int NCH, bool FULL, bool PIPE>
__global__ void __launch_bounds__(1024) fp8_quantize_rows_reg_kernel(const T* __restrict__ x, int64_t rows, int64_t cols, StatArgs a, int fmt,
                                                                     int rounding, uint8_t* __restrict__ codes) {
  __shared__ uint32_t sh_amax[2][32];
  b2q_pdl_entry();
  const int chunks = (int)(cols >> 3);
  const Fp8Fmt F = fp8_fmt(fmt);
  // the next row's chunks are held only where two sets fit the register budget of a 1024-thread CTA (up to 16 registers
  // a set: bf16 rows of up to 32768 elements, f32 rows of up to 4096); longer rows load at the top of their iteration
  constexpr bool PREFETCH = PIPE && sizeof(RawChunk<T>) * NCH <= 64;
  RawChunk<T> raw[NCH], nxt[PREFETCH ? NCH : 1];
  int64_t r = blockIdx.x;
  if (PREFETCH && r < rows) {
#pragma unroll
    for (int k = 0; k < NCH; ++k) {
      const int c = (int)threadIdx.x + k * (int)blockDim.x;
      if (FULL || c < chunks) raw[k].load(x + r * cols, c);
    }
  }
  for (int it = 0; r < rows && (PIPE || it == 0); r += gridDim.x, ++it) {     // !PIPE: one row per CTA (the grid is the row count)
    const int64_t rn = r + gridDim.x;
    if constexpr (PREFETCH) {
      if (rn < rows) {
#pragma unroll
        for (int k = 0; k < NCH; ++k) {
          const int c = (int)threadIdx.x + k * (int)blockDim.x;
          if (FULL || c < chunks) nxt[k].load(x + rn * cols, c);
        }
      }
    } else {
#pragma unroll
      for (int k = 0; k < NCH; ++k) {
        const int c = (int)threadIdx.x + k * (int)blockDim.x;
        if (FULL || c < chunks) raw[k].load(x + r * cols, c);
      }
    }
    uint32_t mb = 0;
#pragma unroll
    for (int k = 0; k < NCH; ++k) {
      const int c = (int)threadIdx.x + k * (int)blockDim.x;
      if (FULL || c < chunks) mb = raw[k].amax_bits(mb);
    }
    if constexpr (sizeof(T) == 2) {                                               // the larger lane (NaN: 0x7FFF), as f32 bits
      const uint32_t hi = mb >> 16, lo = mb & 0xFFFFu;
      mb = max(hi, lo) << 16;
    }
    mb = __reduce_max_sync(0xffffffffu, mb);
    uint32_t* sh = sh_amax[it & 1];                                               // two sets: one barrier per row is enough
    if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = mb;
    __syncthreads();
    const int nw = blockDim.x >> 5;
    mb = (int)(threadIdx.x & 31) < nw ? sh[threadIdx.x & 31] : 0u;
    mb = __reduce_max_sync(0xffffffffu, mb);
    const int bad = mb >= 0x7F800000u;
    const float amax = bad ? 0.0f : __uint_as_float(mb);
    if (threadIdx.x == 0) finish_row(a, r, RowStat{0.0f, 0.0f, amax, bad});   // kFp8Scale reads amax and bad only
    const float scale = amax > 0.0f ? __fdiv_rn(amax, F.max_val) : 1.0f;      // finish_row's value
    float r_lo, r_hi;
    const bool bracket = quotient_bracket(scale, r_lo, r_hi);
    uint2* out = reinterpret_cast<uint2*>(codes + r * cols);
#pragma unroll
    for (int k = 0; k < NCH; ++k) {
      const int c = (int)threadIdx.x + k * (int)blockDim.x;
      if (FULL || c < chunks) {
        float v[8];
        raw[k].get(v);
        uint32_t lo = 0, hi = 0;
        if (rounding == 1) {   // the conversion saturates at +-max_val, which is what the clamp of the other path does
          if (fmt == 0) fp8x8_quotient_rne<false>(v, scale, r_lo, r_hi, bracket, lo, hi);
          else fp8x8_quotient_rne<true>(v, scale, r_lo, r_hi, bracket, lo, hi);
        } else {
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            float q = __fdiv_rn(v[j], scale);
            q = q < -F.max_val ? -F.max_val : (q > F.max_val ? F.max_val : q);
            const uint32_t b = fp8_encode_ref_dev(q, F);
            if (j < 4) lo |= b << (8 * j); else hi |= b << (8 * (j - 4));
          }
        }
        out[c] = make_uint2(lo, hi);
      }
    }
    if constexpr (PREFETCH) {
#pragma unroll
      for (int k = 0; k < NCH; ++k) raw[k] = nxt[k];
    }
  }
}

template <typename T>
int32_t fp8_quantize_rows_impl(b2q_handle h, const T* x, int64_t rows, int64_t cols, int fmt, int rounding,
                               float* scales, uint8_t* codes, int flag_nonfinite = 1) {
  if (rows <= 0 || cols <= 0) B2Q_FAIL(h, B2Q_ERR_EMPTY_INPUT, "fp8_quantize_rows: empty input");
  if (!x || !scales || !codes) B2Q_FAIL(h, B2Q_ERR_INVALID_ARGUMENT, "fp8_quantize_rows: null pointer");
  if (fmt < 0 || fmt > 1 || rounding < 0 || rounding > 1) B2Q_FAIL(h, B2Q_ERR_INVALID_ARGUMENT, "fp8_quantize_rows: bad format/rounding");
  StatArgs a{kFp8Scale, 0, 0, fp8_fmt(fmt).max_val, scales, nullptr, h->d_status, flag_nonfinite};
  if (cols % 8 == 0 && cols >= 256 && cols <= (sizeof(T) == 2 ? 65536 : 32768) && rows <= 0x7FFFFFFF && (reinterpret_cast<uintptr_t>(x) & 15) == 0 &&
      (reinterpret_cast<uintptr_t>(codes) & 7) == 0 && (rows >= 64 || cols <= 2048)) {
    const int64_t chunks = cols >> 3;
    // 1, 2, 4 or 8 chunks of 8 elements per thread; many rows prefer small CTAs (several per SM)
    const int nch = chunks <= 128 ? 1 : (chunks <= 512 ? 2 : (chunks <= 4096 ? 4 : 8));
    const int threads = (int)((ceil_div64(chunks, nch) + 31) / 32 * 32);
    const bool full = chunks == (int64_t)nch * threads;
    // enough CTAs to fill every SM's thread slots; each walks rows with a stride of the grid
    const bool pipe = threads >= 512;
    const int by_threads = 2048 / threads, by_regs = 65536 / (threads * 64);          // the pipelined kernels use up to 64 registers
    const int64_t resident = (int64_t)h->sm_count * (by_regs < 1 ? 1 : (by_regs < by_threads ? by_regs : by_threads));
    const unsigned grid = (unsigned)(!pipe || rows < resident ? rows : resident);
#define ROWS_LAUNCH(N, F)                                                                                                          \
  do {                                                                                                                             \
    const bool pdl = h->sw.chain_pdl != 0;                                                                                          \
    if (pipe) B2Q_CUDA(h, b2q_pdl_launch(pdl, fp8_quantize_rows_reg_kernel<T, N, F, true>, dim3(grid), dim3(threads), 0, h->stream, x, rows, cols, a, fmt, rounding, codes)); \
    else B2Q_CUDA(h, b2q_pdl_launch(pdl, fp8_quantize_rows_reg_kernel<T, N, F, false>, dim3(grid), dim3(threads), 0, h->stream, x, rows, cols, a, fmt, rounding, codes));     \
  } while (0)
    if (nch == 1) { if (full) ROWS_LAUNCH(1, true); else ROWS_LAUNCH(1, false); }
    else if (nch == 2) { if (full) ROWS_LAUNCH(2, true); else ROWS_LAUNCH(2, false); }
    else if (nch == 4) { if (full) ROWS_LAUNCH(4, true); else ROWS_LAUNCH(4, false); }
    else if constexpr (sizeof(T) == 2) { if (full) ROWS_LAUNCH(8, true); else ROWS_LAUNCH(8, false); }
#undef ROWS_LAUNCH
    B2Q_LAUNCH_CHECK(h, "fp8_quantize_rows_reg_kernel");
    return B2Q_OK;
  }
  if (rows <= 128 && cols >= 2048 && cols <= (1 << 20)) {
    B2Q_CUDA(h, b2q_pdl_launch(h->sw.chain_pdl != 0, fp8_quantize_rows_fused_kernel<T>, dim3((unsigned)rows), dim3(1024), 0, h->stream, x, cols, a,
                               fmt, rounding, codes));
    B2Q_LAUNCH_CHECK(h, "fp8_quantize_rows_fused_kernel");
    return B2Q_OK;
  }
  int32_t st = launch_row_stats<T>(h, x, rows, cols, a);
  if (st != B2Q_OK) return st;
  const int64_t n = rows * cols;
  const int vec_ok = ((reinterpret_cast<uintptr_t>(x) & 15) == 0) && ((reinterpret_cast<uintptr_t>(codes) & 3) == 0);
  fp8_encode_kernel<T, true><<<grid_for(h, n, kThreads * 4), kThreads, 0, h->stream>>>(
      x, n, cols, scales, fmt, rounding, codes, h->d_status, vec_ok);
  B2Q_LAUNCH_CHECK(h, "fp8_encode_kernel");
  return B2Q_OK;
}

}  // namespace

extern "C" {

int32_t b2q_minmax_calibrate_f32(b2q_handle h, const float* x, int64_t rows, int64_t cols, int bits, int scheme,
                                 float* scales, int32_t* zero_points) {
  B2Q_REQUIRE_HANDLE(h);
  if (rows <= 0) B2Q_FAIL(h, B2Q_ERR_EMPTY_INPUT, "minmax_calibrate: rows == 0");
  if (cols <= 0) B2Q_FAIL(h, B2Q_ERR_DIMENSION_MISMATCH, "minmax_calibrate: cols == 0");
  if (bits < 1 || bits > 16) B2Q_FAIL(h, B2Q_ERR_INVALID_ARGUMENT, "bits must be in [1, 16]");
  if (scheme < 0 || scheme > 1 || !x || !scales || !zero_points) B2Q_FAIL(h, B2Q_ERR_INVALID_ARGUMENT, "minmax_calibrate: bad argument");
  StatArgs a{kMinMaxParams, bits, scheme, 0.0f, scales, zero_points, h->d_status, 0};
  return launch_row_stats<float>(h, x, rows, cols, a);
}

int32_t b2q_minmax_quantize_f32(b2q_handle h, const float* x, int64_t rows, int64_t cols, const float* scales,
                                const int32_t* zero_points, int bits, int scheme, int32_t* codes) {
  B2Q_REQUIRE_HANDLE(h);
  if (rows <= 0 || cols <= 0) B2Q_FAIL(h, B2Q_ERR_EMPTY_INPUT, "minmax_quantize: empty input");
  if (bits < 1 || bits > 16 || scheme < 0 || scheme > 1 || !x || !scales || !zero_points || !codes)
    B2Q_FAIL(h, B2Q_ERR_INVALID_ARGUMENT, "minmax_quantize: bad argument");
  float q_max = scheme == 0 ? (float)(1 << (bits - 1)) - 1.0f : (float)(1 << bits) - 1.0f;
  float q_min = scheme == 0 ? -(float)(1 << (bits - 1)) : 0.0f;
  int64_t n = rows * cols;
  const int vec_ok = cols % 4 == 0 && ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(codes)) & 15) == 0;
  minmax_quantize_kernel<<<grid_for(h, n, kThreads * (vec_ok ? 4 : 1)), kThreads, 0, h->stream>>>(x, n, cols, scales, zero_points, q_min, q_max,
                                                                                               codes, vec_ok);
  B2Q_LAUNCH_CHECK(h, "minmax_quantize_kernel");
  return B2Q_OK;
}

int32_t b2q_minmax_dequantize_f32(b2q_handle h, const int32_t* codes, int64_t rows, int64_t cols, const float* scales,
                                  const int32_t* zero_points, float* out) {
  B2Q_REQUIRE_HANDLE(h);
  if (rows <= 0 || cols <= 0) B2Q_FAIL(h, B2Q_ERR_EMPTY_INPUT, "minmax_dequantize: empty input");
  if (!codes || !scales || !zero_points || !out) B2Q_FAIL(h, B2Q_ERR_INVALID_ARGUMENT, "minmax_dequantize: null pointer");
  int64_t n = rows * cols;
  const int vec_ok = cols % 4 == 0 && ((reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(codes)) & 15) == 0;
  minmax_dequantize_kernel<<<grid_for(h, n, kThreads * (vec_ok ? 4 : 1)), kThreads, 0, h->stream>>>(codes, n, cols, scales, zero_points, out, vec_ok);
  B2Q_LAUNCH_CHECK(h, "minmax_dequantize_kernel");
  return B2Q_OK;
}

int32_t b2q_fake_quant_inplace_f32(b2q_handle h, float* x, int64_t n, float scale, float zero_point, float qmin, float qmax) {
  B2Q_REQUIRE_HANDLE(h);
  if (n <= 0) B2Q_FAIL(h, B2Q_ERR_EMPTY_INPUT, "fake_quant: empty input");
  if (!(scale > 0.0f) || !isfinite(scale)) B2Q_FAIL(h, B2Q_ERR_INVALID_SCALE, "fake_quant: scale %g", (double)scale);
  if (!x) B2Q_FAIL(h, B2Q_ERR_INVALID_ARGUMENT, "fake_quant: null pointer");
  fake_quant_kernel<<<grid_for(h, n, kThreads), kThreads, 0, h->stream>>>(x, n, scale, zero_point, qmin, qmax);
  B2Q_LAUNCH_CHECK(h, "fake_quant_kernel");
  return B2Q_OK;
}

int32_t b2q_fp8_encode_f32(b2q_handle h, const float* x, int64_t n, int fmt, int rounding, uint8_t* codes) {
  B2Q_REQUIRE_HANDLE(h);
  if (n == 0) return B2Q_OK;  // encode of an empty slice is an empty Vec
  if (n < 0 || !x || !codes || fmt < 0 || fmt > 1 || rounding < 0 || rounding > 1)
    B2Q_FAIL(h, B2Q_ERR_INVALID_ARGUMENT, "fp8_encode: bad argument");
  const int vec_ok = ((reinterpret_cast<uintptr_t>(x) & 15) == 0) && ((reinterpret_cast<uintptr_t>(codes) & 3) == 0);
  fp8_encode_kernel<float, false><<<grid_for(h, n, kThreads * 4), kThreads, 0, h->stream>>>(
      x, n, 1, nullptr, fmt, rounding, codes, h->d_status, vec_ok);
  B2Q_LAUNCH_CHECK(h, "fp8_encode_kernel");
  return B2Q_OK;
}

int32_t b2q_fp8_decode_f32(b2q_handle h, const uint8_t* codes, int64_t n, int fmt, int rounding, float* out) {
  B2Q_REQUIRE_HANDLE(h);
  if (n == 0) return B2Q_OK;
  if (n < 0 || !codes || !out || fmt < 0 || fmt > 1 || rounding < 0 || rounding > 1)
    B2Q_FAIL(h, B2Q_ERR_INVALID_ARGUMENT, "fp8_decode: bad argument");
  fp8_decode_kernel<<<grid_for(h, n, kThreads * 4), kThreads, 0, h->stream>>>(codes, n, fmt, rounding, out);
  B2Q_LAUNCH_CHECK(h, "fp8_decode_kernel");
  return B2Q_OK;
}

int32_t b2q_fp8_remap_ref_subnormals(b2q_handle h, uint8_t* codes, int64_t n, int fmt) {
  B2Q_REQUIRE_HANDLE(h);
  if (n == 0) return B2Q_OK;
  if (n < 0 || !codes || fmt < 0 || fmt > 1) B2Q_FAIL(h, B2Q_ERR_INVALID_ARGUMENT, "fp8_remap_ref_subnormals: bad argument");
  fp8_remap_ref_subnormals_kernel<<<grid_for(h, n, kThreads), kThreads, 0, h->stream>>>(codes, n, fmt);
  B2Q_LAUNCH_CHECK(h, "fp8_remap_ref_subnormals_kernel");
  return B2Q_OK;
}

int32_t b2q_fp8_quantize_rows_f32(b2q_handle h, const float* x, int64_t rows, int64_t cols, int fmt, int rounding,
                                  float* scales, uint8_t* codes) {
  B2Q_REQUIRE_HANDLE(h);
  return fp8_quantize_rows_impl<float>(h, x, rows, cols, fmt, rounding, scales, codes);
}
int32_t b2q_fp8_quantize_rows_bf16(b2q_handle h, const void* x, int64_t rows, int64_t cols, int fmt, int rounding,
                                   float* scales, uint8_t* codes) {
  B2Q_REQUIRE_HANDLE(h);
  return fp8_quantize_rows_impl<__nv_bfloat16>(h, (const __nv_bfloat16*)x, rows, cols, fmt, rounding, scales, codes);
}

}  // extern "C"
// Rows of a scratch buffer of which only some hold results (the slots of a mixture-of-experts step; which ones is known
// on the device only): the unused rows may hold anything, so non-finite input is not recorded as an error.
int32_t b2q_fp8_quantize_rows_bf16_scratch(b2q_handle h, const void* x, int64_t rows, int64_t cols, int fmt, int rounding, float* scales,
                                           uint8_t* codes) {
  return fp8_quantize_rows_impl<__nv_bfloat16>(h, (const __nv_bfloat16*)x, rows, cols, fmt, rounding, scales, codes, 0);
}
extern "C" {

int32_t b2q_fp4_block_quantize_f32(b2q_handle h, const float* x, int64_t n, int block, int format, int scale_format,
                                   uint8_t* packed, void* scales) {
  B2Q_REQUIRE_HANDLE(h);
  if (block != 32 && block != 64 && block != 128)
    B2Q_FAIL(h, B2Q_ERR_INVALID_ARGUMENT, "MicroScaling block_size must be one of [32, 64, 128], got %d", block);
  if (n <= 0) return B2Q_OK;
  if (n % block != 0) B2Q_FAIL(h, B2Q_ERR_INVALID_DIMENSION, "fp4_block_quantize: n=%lld is not a multiple of block=%d", (long long)n, block);
  if (!x || !packed || !scales || format < 0 || format > 1 || scale_format < 0 || scale_format > 1)
    B2Q_FAIL(h, B2Q_ERR_INVALID_ARGUMENT, "fp4_block_quantize: bad argument");
  if ((reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(packed) & 1))
    B2Q_FAIL(h, B2Q_ERR_INVALID_ARGUMENT, "fp4_block_quantize: x must be 16-byte and packed 2-byte aligned");
  fp4_block_quantize_kernel<<<grid_for(h, n / 4, kThreads), kThreads, 0, h->stream>>>(
      x, n, block, format, scale_format, packed, (float*)scales, (uint8_t*)scales);
  B2Q_LAUNCH_CHECK(h, "fp4_block_quantize_kernel");
  return B2Q_OK;
}

int32_t b2q_fp4_block_dequantize_f32(b2q_handle h, const uint8_t* packed, int64_t n, int block, int format,
                                     int scale_format, const void* scales, float* out) {
  B2Q_REQUIRE_HANDLE(h);
  if (block != 32 && block != 64 && block != 128)
    B2Q_FAIL(h, B2Q_ERR_INVALID_ARGUMENT, "MicroScaling block_size must be one of [32, 64, 128], got %d", block);
  if (n <= 0) return B2Q_OK;
  if (n % block != 0) B2Q_FAIL(h, B2Q_ERR_INVALID_DIMENSION, "fp4_block_dequantize: n=%lld is not a multiple of block=%d", (long long)n, block);
  if (!packed || !scales || !out || format < 0 || format > 1 || scale_format < 0 || scale_format > 1)
    B2Q_FAIL(h, B2Q_ERR_INVALID_ARGUMENT, "fp4_block_dequantize: bad argument");
  if ((reinterpret_cast<uintptr_t>(out) & 15) || (reinterpret_cast<uintptr_t>(packed) & 1))
    B2Q_FAIL(h, B2Q_ERR_INVALID_ARGUMENT, "fp4_block_dequantize: out must be 16-byte and packed 2-byte aligned");
  fp4_block_dequantize_kernel<<<grid_for(h, n / 4, kThreads), kThreads, 0, h->stream>>>(
      packed, n, block, format, scale_format, (const float*)scales, (const uint8_t*)scales, out);
  B2Q_LAUNCH_CHECK(h, "fp4_block_dequantize_kernel");
  return B2Q_OK;
}

int32_t b2q_nf4_decode_f32(b2q_handle h, const uint8_t* packed, int64_t nbytes, int block, const float* absmaxs, float* out) {
  B2Q_REQUIRE_HANDLE(h);
  if (block <= 0 || block % 2 != 0) B2Q_FAIL(h, B2Q_ERR_INVALID_ARGUMENT, "nf4: block must be positive and even");
  if (nbytes <= 0) return B2Q_OK;
  if ((2 * nbytes) % block != 0) B2Q_FAIL(h, B2Q_ERR_DIMENSION_MISMATCH, "nf4_decode: packed length inconsistent with block");
  if (!packed || !absmaxs || !out || (reinterpret_cast<uintptr_t>(out) & 7)) B2Q_FAIL(h, B2Q_ERR_INVALID_ARGUMENT, "nf4_decode: bad pointer");
  nf4_decode_kernel<<<grid_for(h, nbytes, kThreads), kThreads, 0, h->stream>>>(packed, nbytes, block, absmaxs, out);
  B2Q_LAUNCH_CHECK(h, "nf4_decode_kernel");
  return B2Q_OK;
}

int32_t b2q_nf4_encode_f32(b2q_handle h, const float* x, int64_t n, int block, uint8_t* packed, float* absmaxs) {
  B2Q_REQUIRE_HANDLE(h);
  if (n <= 0) B2Q_FAIL(h, B2Q_ERR_EMPTY_INPUT, "Nf4Quantizer::encode: empty input");
  if (block <= 0 || block % 2 != 0) B2Q_FAIL(h, B2Q_ERR_INVALID_ARGUMENT, "nf4: block must be positive and even");
  if (n % block != 0) B2Q_FAIL(h, B2Q_ERR_GROUP_SIZE_MISMATCH, "nf4_encode: len %lld not divisible by group %d", (long long)n, block);
  if (!x || !packed || !absmaxs) B2Q_FAIL(h, B2Q_ERR_INVALID_ARGUMENT, "nf4_encode: null pointer");
  int64_t nblocks = n / block;
  const bool aligned = (reinterpret_cast<uintptr_t>(x) & 15) == 0 && (reinterpret_cast<uintptr_t>(packed) & 3) == 0;
  if (aligned && (block == 32 || block == 64 || block == 128 || block == 256)) {
#define NF4_SUBWARP(G) nf4_encode_subwarp_kernel<G><<<grid_for(h, nblocks, (kThreads / 32) * (32 / G)), kThreads, 0, h->stream>>>(x, nblocks, packed, absmaxs)
    if (block == 32) NF4_SUBWARP(4);
    else if (block == 64) NF4_SUBWARP(8);
    else if (block == 128) NF4_SUBWARP(16);
    else NF4_SUBWARP(32);
#undef NF4_SUBWARP
    B2Q_LAUNCH_CHECK(h, "nf4_encode_subwarp_kernel");
    return B2Q_OK;
  }
  nf4_encode_kernel<<<grid_for(h, nblocks, kThreads / 32), kThreads, 0, h->stream>>>(x, nblocks, block, packed, absmaxs);
  B2Q_LAUNCH_CHECK(h, "nf4_encode_kernel");
  return B2Q_OK;
}

int32_t b2q_int8_quant_f32(b2q_handle h, const float* x, int64_t n, float scale, int8_t* out) {
  B2Q_REQUIRE_HANDLE(h);
  if (n <= 0) return B2Q_OK;
  if (!(scale > 0.0f) || !isfinite(scale)) B2Q_FAIL(h, B2Q_ERR_INVALID_SCALE, "int8_quant: scale %g", (double)scale);
  if (!x || !out) B2Q_FAIL(h, B2Q_ERR_INVALID_ARGUMENT, "int8_quant: null pointer");
  const int vec_ok = ((reinterpret_cast<uintptr_t>(x) & 15) == 0) && ((reinterpret_cast<uintptr_t>(out) & 3) == 0);
  int8_quant_kernel<<<grid_for(h, n, kThreads * 4), kThreads, 0, h->stream>>>(x, n, scale, out, vec_ok);
  B2Q_LAUNCH_CHECK(h, "int8_quant_kernel");
  return B2Q_OK;
}
int32_t b2q_int8_dequant_f32(b2q_handle h, const int8_t* q, int64_t n, float scale, float* out) {
  B2Q_REQUIRE_HANDLE(h);
  if (n <= 0) return B2Q_OK;
  if (!q || !out) B2Q_FAIL(h, B2Q_ERR_INVALID_ARGUMENT, "int8_dequant: null pointer");
  const int vec_ok = ((reinterpret_cast<uintptr_t>(out) & 15) == 0) && ((reinterpret_cast<uintptr_t>(q) & 3) == 0);
  int8_dequant_kernel<<<grid_for(h, n, kThreads * 4), kThreads, 0, h->stream>>>(q, n, scale, out, vec_ok);
  B2Q_LAUNCH_CHECK(h, "int8_dequant_kernel");
  return B2Q_OK;
}

int32_t b2q_distfp8_quantize_block_f32(b2q_handle h, const float* x, int64_t n, int64_t block, uint8_t* q, float* absmaxs) {
  B2Q_REQUIRE_HANDLE(h);
  if (n <= 0) return B2Q_OK;
  if (!x || !q || !absmaxs) B2Q_FAIL(h, B2Q_ERR_INVALID_ARGUMENT, "distfp8_quantize: null pointer");
  if (block < 1) block = 1;
  if (block > n) block = n;
  if (n % block != 0) B2Q_FAIL(h, B2Q_ERR_INVALID_DIMENSION, "distfp8_quantize: device path needs n %% block == 0");
  StatArgs a{kAbsmaxOnly, 0, 0, 0.0f, absmaxs, nullptr, h->d_status, 0};
  int32_t st = launch_row_stats<float>(h, x, n / block, block, a);
  if (st != B2Q_OK) return st;
  const int vec_ok = block % 4 == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0 && (reinterpret_cast<uintptr_t>(q) & 3) == 0;
  distfp8_quantize_kernel<<<grid_for(h, n, kThreads * (vec_ok ? 4 : 1)), kThreads, 0, h->stream>>>(x, n, block, absmaxs, q, vec_ok);
  B2Q_LAUNCH_CHECK(h, "distfp8_quantize_kernel");
  return B2Q_OK;
}
int32_t b2q_distfp8_dequantize_block_f32(b2q_handle h, const uint8_t* q, int64_t n, int64_t block, const float* absmaxs, float* out) {
  B2Q_REQUIRE_HANDLE(h);
  if (n <= 0) return B2Q_OK;
  if (!q || !absmaxs || !out) B2Q_FAIL(h, B2Q_ERR_INVALID_ARGUMENT, "distfp8_dequantize: null pointer");
  if (block < 1) block = 1;
  if (block > n) block = n;
  const int vec_ok = block % 4 == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0 && (reinterpret_cast<uintptr_t>(q) & 3) == 0;
  distfp8_dequantize_kernel<<<grid_for(h, n, kThreads * (vec_ok ? 4 : 1)), kThreads, 0, h->stream>>>(q, n, block, absmaxs, out, vec_ok);
  B2Q_LAUNCH_CHECK(h, "distfp8_dequantize_kernel");
  return B2Q_OK;
}

}  // extern "C"

// ---------------------------------------------------------------------------
// Allocation-free variant of the absmax-scaled FP8 quantizer.
//
// Some callers may not allocate device memory at all: code running under a memory budget it
// does not own (a plugin inside a serving process whose allocator hands out every byte up
// front), code that must not touch the allocator between two points in time (a latency-critical
// region, a region that another component is capturing or replaying), or a host that simply has
// no handle yet.  b2q_create allocates (status word, scratch, later the workspace), so this
// entry point takes no handle: the reduction keys and the status word that the handle's scratch
// normally provides live in the file-scope array below, which every device that loads this
// library carries until the process exits (kNoAllocWords * 4 bytes = 16.25 KiB).
//
// The array's name is only a host-side stand-in for the device object: its device address is
// obtained once per device, with that device current, through cudaGetSymbolAddress.  That set-up
// happens in the first call made on a device, so make the first call outside any stream capture.
// All calls on a device share the array and it keeps the previous call's contents: each call
// re-initialises the keys it is going to use on the stream before using them, and two calls
// whose kernels may overlap on the GPU (different streams, no dependency) race on it.
// ---------------------------------------------------------------------------
namespace {
constexpr int kNoAllocMaxRows = 1024;                         // slices per call
constexpr int kNoAllocWords = 4 * kNoAllocMaxRows + 64;       // 4 keys per slice + the status word (own 256-byte line)
}  // namespace
static __device__ __align__(256) uint32_t g_noalloc_scratch[kNoAllocWords];

namespace {
// per-device set-up record; `ready` is published with release / read with acquire, so a second host thread that sees it
// set also sees ptr and sm_count (two threads racing through the set-up write the same values)
struct NoAllocDevice { uint32_t* ptr; int sm_count; std::atomic<int> ready; };
NoAllocDevice g_noalloc_dev[64];

void noalloc_msg(char* err, size_t err_len, const char* fmt, long long a, long long b) {
  if (err && err_len) snprintf(err, err_len, fmt, a, b);
}
}  // namespace

extern "C" int32_t b2q_fp8_quantize_rows_f32_noalloc(const float* x, int64_t rows, int64_t cols, int fmt, int rounding,
                                                     float* scales, uint8_t* codes, void* stream, int32_t* device_status,
                                                     char* err, size_t err_len) {
  if (err && err_len) err[0] = 0;
  if (rows <= 0 || cols <= 0) { noalloc_msg(err, err_len, "empty input: rows=%lld cols=%lld", rows, cols); return B2Q_ERR_EMPTY_INPUT; }
  if (rows > kNoAllocMaxRows) {
    noalloc_msg(err, err_len, "rows=%lld exceeds the %lld slices the built-in scratch holds; use b2q_fp8_quantize_rows_f32", rows, kNoAllocMaxRows);
    return B2Q_ERR_BUFFER_TOO_SMALL;
  }
  if (!x || !scales || !codes || fmt < 0 || fmt > 1 || rounding < 0 || rounding > 1) {
    noalloc_msg(err, err_len, "null pointer or bad format/rounding (fmt=%lld rounding=%lld)", fmt, rounding);
    return B2Q_ERR_INVALID_ARGUMENT;
  }
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) { noalloc_msg(err, err_len, "no current CUDA device (%lld, %lld)", dev, 0); return B2Q_ERR_CUDA; }
  NoAllocDevice& d = g_noalloc_dev[dev];
  if (!d.ready.load(std::memory_order_acquire)) {             // once per device, with that device current
    void* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
    if (e != cudaSuccess || !p) { noalloc_msg(err, err_len, "cudaGetSymbolAddress failed with CUDA error %lld on device %lld", (int)e, dev); return B2Q_ERR_CUDA; }
    int sms = 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 128;
    d.ptr = (uint32_t*)p;
    d.sm_count = sms;
    d.ready.store(1, std::memory_order_release);
  }
  cudaStream_t st = (cudaStream_t)stream;
  uint32_t* keys = d.ptr;
  int32_t* status = device_status ? device_status : (int32_t*)(d.ptr + 4 * kNoAllocMaxRows);
  // same arithmetic as b2q_fp8_quantize_rows_f32: per-slice absmax through ordered-key atomics, scale, encode
  int64_t bpr = ceil_div64((int64_t)d.sm_count * 8, rows);
  int64_t seg = ceil_div64(cols, bpr);
  seg = ceil_div64(seg, 4 * kThreads) * 4 * kThreads;
  bpr = ceil_div64(cols, seg);
  StatArgs a{kFp8Scale, 0, 0, fp8_fmt(fmt).max_val, scales, nullptr, status, 1};
  stat_keys_init_kernel<<<(int)ceil_div64(rows, 256), 256, 0, st>>>(keys, rows);            // clears what must start clean
  row_stat_split_kernel<float><<<dim3((unsigned)bpr, (unsigned)rows), kThreads, 0, st>>>(x, cols, seg, keys);
  stat_keys_finish_kernel<<<(int)ceil_div64(rows, 256), 256, 0, st>>>(keys, rows, a);
  const int64_t n = rows * cols;
  const int vec_ok = ((reinterpret_cast<uintptr_t>(x) & 15) == 0) && ((reinterpret_cast<uintptr_t>(codes) & 3) == 0);
  int64_t g = ceil_div64(n, (int64_t)kThreads * 4);
  if (g > (int64_t)d.sm_count * 16) g = (int64_t)d.sm_count * 16;
  fp8_encode_kernel<float, true><<<(int)g, kThreads, 0, st>>>(x, n, cols, scales, fmt, rounding, codes, status, vec_ok);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) { noalloc_msg(err, err_len, "kernel launch failed with CUDA error %lld (%lld)", (int)e, 0); return B2Q_ERR_LAUNCH_FAILED; }
  return B2Q_OK;
}

// ---------------------------------------------------------------------------
// SwiGLU + per-token FP8 re-quantization between the column-parallel gate/up projections and the
// row-parallel down projection: h = silu(gate) * up in fp32 (silu(x) = x / (1 + exp(-x))), scale = absmax(h)/max,
// code = encode(h / scale).  One CTA per token row; h is recomputed in the second pass instead of being stored.
// ---------------------------------------------------------------------------
namespace {
__device__ __forceinline__ float swiglu_f32(float g, float u) { return __fdiv_rn(g, 1.0f + expf(-g)) * u; }

// `split` > 1: a thread-block cluster of `split` CTAs shares a row (few rows, long rows: the decode step); each CTA
// takes a contiguous slice of the columns and the slices' maxima are exchanged through distributed shared memory.
// `inter`: gate and up are interleaved per 128 columns in one row of 2 * cols_all elements (hidden unit f: gate at
// column 256 (f / 128) + f % 128, up 128 further; `up` is then gate + 128), the input is the f32 product and h is rounded
// to bf16 before the row maximum and the encoding: the arithmetic of the GEMM epilogue that forms h for many tokens.
template <typename TIn> __device__ __forceinline__ void load8_f32(const TIn* p, float (&v)[8]);
template <> __device__ __forceinline__ void load8_f32<__nv_bfloat16>(const __nv_bfloat16* p, float (&v)[8]) {
  const uint4 q = *reinterpret_cast<const uint4*>(p);
  const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
  for (int j = 0; j < 4; ++j) { v[2 * j] = __uint_as_float(w[j] << 16); v[2 * j + 1] = __uint_as_float(w[j] & 0xFFFF0000u); }
}
template <> __device__ __forceinline__ void load8_f32<float>(const float* p, float (&v)[8]) {
  const float4 a = reinterpret_cast<const float4*>(p)[0], b = reinterpret_cast<const float4*>(p)[1];
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
template <typename TIn> __device__ __forceinline__ float in_as_f32(TIn v);
template <> __device__ __forceinline__ float in_as_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <> __device__ __forceinline__ float in_as_f32<float>(float v) { return v; }

template <typename TIn>
__global__ void __launch_bounds__(1024) swiglu_quantize_rows_kernel(const TIn* __restrict__ gate, const TIn* __restrict__ up, int64_t ld,
                                                                        int64_t cols_all, int fmt, int rounding, float* scales,
                                                                        uint8_t* codes, int split, int inter) {
  b2q_pdl_entry();
  const int64_t r = blockIdx.x / split;
  const int part = (int)(blockIdx.x % split);
  // slices are multiples of 8 columns so that the vector path keeps its alignment
  const int64_t slice = ((cols_all + split - 1) / split + 7) & ~(int64_t)7;
  const int64_t c_begin = min((int64_t)part * slice, cols_all), c_end = min(c_begin + slice, cols_all);
  const int64_t cols = c_end - c_begin;
  const TIn* g = gate + r * ld;
  const TIn* u = up + r * ld;
  auto at = [&](int64_t c) { const int64_t f = c_begin + c; return inter ? ((f >> 7) << 8) + (f & 127) : f; };   // column of unit c_begin + c
  auto hval = [&](float gv, float uv) {
    const float h = swiglu_f32(gv, uv);
    return inter ? __bfloat162float(__float2bfloat16_rn(h)) : h;
  };
  const Fp8Fmt F = fp8_fmt(fmt);
  __shared__ float sh[32];
  const int nthreads = (int)blockDim.x;                      // kThreads, or 1024 when there are few rows
  float amax = 0.0f;
  const bool vec = (cols % 8 == 0) && (cols_all % 8 == 0) && (ld % 8 == 0) &&
                   ((reinterpret_cast<uintptr_t>(gate) | reinterpret_cast<uintptr_t>(up)) & (sizeof(TIn) * 8 - 1)) == 0;
  if (vec) {
    for (int64_t c = (int64_t)threadIdx.x * 8; c < cols; c += (int64_t)nthreads * 8) {
      float gv[8], uv[8];
      load8_f32<TIn>(g + at(c), gv);
      load8_f32<TIn>(u + at(c), uv);
#pragma unroll
      for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(hval(gv[j], uv[j])));
    }
  } else {
    for (int64_t c = threadIdx.x; c < cols; c += nthreads) amax = fmaxf(amax, fabsf(hval(in_as_f32<TIn>(g[at(c)]), in_as_f32<TIn>(u[at(c)]))));
  }
  amax = warp_max(amax);
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = amax;
  __syncthreads();
  amax = sh[0];
  for (int w = 1; w < nthreads / 32; ++w) amax = fmaxf(amax, sh[w]);
  if (split > 1) {
    __shared__ float s_part;
    cg::cluster_group cluster = cg::this_cluster();
    if (threadIdx.x == 0) s_part = amax;
    cluster.sync();
    for (int q = 0; q < split; ++q) amax = fmaxf(amax, *cluster.map_shared_rank(&s_part, q));
    cluster.sync();                                          // peers may still be reading this CTA's maximum
  }
  const float scale = amax > 0.0f ? __fdiv_rn(amax, F.max_val) : 1.0f;
  if (threadIdx.x == 0 && part == 0) scales[r] = scale;
  auto enc = [&](float h) -> uint32_t {
    float v = __fdiv_rn(h, scale);
    v = v < -F.max_val ? -F.max_val : (v > F.max_val ? F.max_val : v);
    return rounding == 0 ? fp8_encode_ref_dev(v, F) : fp8_encode_rne_dev(v, fmt);
  };
  uint8_t* out = codes + r * cols_all + c_begin;
  if (vec) {
    for (int64_t c = (int64_t)threadIdx.x * 8; c < cols; c += (int64_t)nthreads * 8) {
      float gv[8], uv[8];
      load8_f32<TIn>(g + at(c), gv);
      load8_f32<TIn>(u + at(c), uv);
      uint32_t lo = 0, hi = 0;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const uint32_t code = enc(hval(gv[j], uv[j]));
        if (j < 4) lo |= code << (8 * j); else hi |= code << (8 * (j - 4));
      }
      *reinterpret_cast<uint2*>(out + c) = make_uint2(lo, hi);
    }
  } else {
    for (int64_t c = threadIdx.x; c < cols; c += nthreads) out[c] = (uint8_t)enc(hval(in_as_f32<TIn>(g[at(c)]), in_as_f32<TIn>(u[at(c)])));
  }
}
}  // namespace

// gate | up of one GEMM whose weight rows were interleaved per 128 (see b2q_interleave_rows128): gu [rows x 2 cols] f32.
int32_t b2q_swiglu_quantize_rows_interleaved(b2q_handle h, const float* gu, int64_t rows, int64_t cols, int fmt, int rounding, float* scales,
                                             uint8_t* codes);
template <typename TIn>
static int32_t swiglu_quantize_rows_launch(b2q_handle h, const TIn* gate, const TIn* up, int64_t rows, int64_t cols, int64_t ld, int fmt,
                                           int rounding, float* scales, uint8_t* codes, int inter) {
  if (rows <= 0 || cols <= 0) B2Q_FAIL(h, B2Q_ERR_EMPTY_INPUT, "swiglu_quantize_rows: empty input");
  if (!gate || !up || !scales || !codes || ld < cols || fmt < 0 || fmt > 1 || rounding < 0 || rounding > 1)
    B2Q_FAIL(h, B2Q_ERR_INVALID_ARGUMENT, "swiglu_quantize_rows: bad argument");
  if (rows > 0x7FFFFFFF) B2Q_FAIL(h, B2Q_ERR_INVALID_DIMENSION, "swiglu_quantize_rows: too many rows");
  // few rows: 1024 threads per CTA, and for long rows a cluster of 8 CTAs per row
  const int threads = rows <= 2 * h->sm_count ? 1024 : kThreads;
  const int split = (rows * 8 <= h->sm_count && cols >= 8192) ? 8 : 1;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(rows * split));
  cfg.blockDim = dim3((unsigned)threads);
  cfg.stream = h->stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = (unsigned)split;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = h->sw.chain_pdl != 0 ? 2 : 1;
  B2Q_CUDA(h, cudaLaunchKernelEx(&cfg, swiglu_quantize_rows_kernel<TIn>, gate, up, ld, cols, fmt, rounding, scales, codes, split, inter));
  return B2Q_OK;
}

extern "C" int32_t b2q_swiglu_quantize_rows_bf16(b2q_handle h, const void* gate, const void* up, int64_t rows, int64_t cols,
                                                 int64_t ld, int fmt, int rounding, float* scales, uint8_t* codes) {
  B2Q_REQUIRE_HANDLE(h);
  return swiglu_quantize_rows_launch<__nv_bfloat16>(h, (const __nv_bfloat16*)gate, (const __nv_bfloat16*)up, rows, cols, ld, fmt, rounding, scales,
                                                    codes, 0);
}
int32_t b2q_swiglu_quantize_rows_interleaved(b2q_handle h, const float* gu, int64_t rows, int64_t cols, int fmt, int rounding, float* scales,
                                             uint8_t* codes) {
  if (cols % 128 != 0) B2Q_FAIL(h, B2Q_ERR_INVALID_DIMENSION, "swiglu_quantize_rows: the interleaved layout needs a multiple of 128 columns, got %lld", (long long)cols);
  return swiglu_quantize_rows_launch<float>(h, gu, gu ? gu + 128 : nullptr, rows, cols, 2 * cols, fmt, rounding, scales, codes, 1);
}
