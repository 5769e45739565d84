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
// (Rust's saturating `as` casts), so the byte is the low 8 bits of the clamped integer.
__device__ __forceinline__ uint32_t kv_code(float v, KvParams p, int qmin, int qmax) {
  const float q = roundf(__fdiv_rn(__fsub_rn(v, p.zp), p.scale));
  int qi = __float2int_rz(q);          // q is integral; saturates, NaN -> 0
  qi = qi < qmin ? qmin : (qi > qmax ? qmax : qi);
  return (uint32_t)qi & 0xFFu;
}

// ---------------------------------------------------------------------------
// One group per token: a warp per row, statistics and codes in one launch.  The second pass re-reads the row from
// L1/L2 (a row is at most a few KB), so DRAM sees each input byte once.
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
        for (int j = 0; j < 4; ++j) { if (v[j] < mn) mn = v[j]; if (v[j] > mx) mx = v[j]; }
      }
    } else {
      for (int64_t i = lane; i < cols; i += 32) { const float v = ld1<T>(row, i); if (v < mn) mn = v; if (v > mx) mx = v; }
    }
    mn = warp_min(mn);
    mx = warp_max(mx);
    const KvParams p = kv_params(rule, mn, mx, qmin_f, qmax_f);
    if (lane == 0) { scales[r] = p.scale; zps[r] = p.zp; }
    uint8_t* out = codes + r * cols;
    if (VEC) {
      for (int64_t i = (int64_t)lane * 4; i < cols; i += 128) {
        float v[4];
        ld4<T>(row, i, v);
        const uint32_t w = kv_code(v[0], p, qmin, qmax) | (kv_code(v[1], p, qmin, qmax) << 8) | (kv_code(v[2], p, qmin, qmax) << 16) |
                           (kv_code(v[3], p, qmin, qmax) << 24);
        *reinterpret_cast<uint32_t*>(out + i) = w;
      }
    } else {
      for (int64_t i = lane; i < cols; i += 32) out[i] = (uint8_t)kv_code(ld1<T>(row, i), p, qmin, qmax);
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
      for (int j = 0; j < 4; ++j) { if (v[j] < mn) mn = v[j]; if (v[j] > mx) mx = v[j]; }
    }
    for (; r < r1; r += kWarpsPerBlock) { const float v = ld1<T>(x, r * cols + c); if (v < mn) mn = v; if (v > mx) mx = v; }
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

__global__ void kv_channel_params_kernel(const uint32_t* keys, int64_t head_dim, float qmax_f, float* scales, float* zps) {
  const int64_t c = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (c < head_dim) {
    const KvParams p = kv_params(kRuleCache, float_from_order_key(keys[c]), float_from_order_key(keys[head_dim + c]), 0.0f, qmax_f);
    scales[c] = p.scale;
    zps[c] = p.zp;
  }
}

template <typename T, bool VEC>
__global__ void __launch_bounds__(kThreads) kv_quantize_per_channel_kernel(const T* __restrict__ x, int64_t n, int64_t cols, int qmax,
                                                                           const float* __restrict__ scales, const float* __restrict__ zps,
                                                                           uint8_t* __restrict__ codes) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  if (VEC) {   // cols % 4 == 0: four consecutive elements share a row and are four consecutive channels
    for (int64_t i = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 4; i < n; i += stride * 4) {
      const int64_t c = i % cols;
      float v[4];
      ld4<T>(x, i, v);
      const float4 s = *reinterpret_cast<const float4*>(scales + c);
      const float4 z = *reinterpret_cast<const float4*>(zps + c);
      const uint32_t w = kv_code(v[0], KvParams{s.x, z.x}, 0, qmax) | (kv_code(v[1], KvParams{s.y, z.y}, 0, qmax) << 8) |
                         (kv_code(v[2], KvParams{s.z, z.z}, 0, qmax) << 16) | (kv_code(v[3], KvParams{s.w, z.w}, 0, qmax) << 24);
      *reinterpret_cast<uint32_t*>(codes + i) = w;
    }
  } else {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
      const int64_t c = i % cols;
      codes[i] = (uint8_t)kv_code(ld1<T>(x, i), KvParams{scales[c], zps[c]}, 0, qmax);
    }
  }
}

// code * scale + zero point, unfused (kv_cache.rs:224-238, kv_quant.rs:94-100).  axis 0: group = row, 1: group = column.
template <typename T>
__global__ void __launch_bounds__(kThreads) kv_dequantize_kernel(const uint8_t* __restrict__ codes, int64_t n, int64_t cols, int axis,
                                                                 int signed_codes, const float* __restrict__ scales,
                                                                 const float* __restrict__ zps, T* __restrict__ out) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    const int64_t g = axis == 0 ? i / cols : i % cols;
    const uint32_t b = codes[i];
    const float q = signed_codes ? (float)(int)(int8_t)b : (float)b;
    st1<T>(out, i, __fadd_rn(__fmul_rn(q, scales[g]), zps[g]));
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
  const int grid = grid_cap(h, ceil_div64(rows, kWarpsPerBlock));
  if (vec) kv_quantize_per_token_kernel<T, true><<<grid, kThreads, 0, h->stream>>>(x, rows, cols, rule, qmin, qmax, codes, scales, zps);
  else kv_quantize_per_token_kernel<T, false><<<grid, kThreads, 0, h->stream>>>(x, rows, cols, rule, qmin, qmax, codes, scales, zps);
  B2Q_LAUNCH_CHECK(h, "kv_quantize_per_token_kernel");
  return B2Q_OK;
}

template <typename T>
int32_t kv_quantize_channels(b2q_handle h, const T* x, int64_t rows, int64_t cols, int qmax, uint8_t* codes, float* scales, float* zps) {
  if ((size_t)cols * 2 > kScratchWords) B2Q_FAIL(h, B2Q_ERR_UNSUPPORTED, "kv_cache_quantize: per-channel head_dim %lld above %zu", (long long)cols, kScratchWords / 2);
  uint32_t* keys = h->d_scratch;
  kv_channel_keys_init_kernel<<<(unsigned)ceil_div64(cols, kThreads), kThreads, 0, h->stream>>>(keys, cols);
  const int64_t col_blocks = ceil_div64(cols, 32);
  // about 8 blocks per SM over the whole grid, at least 64 rows per block
  int64_t row_blocks = ceil_div64((int64_t)h->sm_count * 8, col_blocks);
  int64_t rows_per_block = ceil_div64(rows, row_blocks);
  if (rows_per_block < 64) rows_per_block = 64;
  row_blocks = ceil_div64(rows, rows_per_block);
  if (row_blocks > 65535) { row_blocks = 65535; rows_per_block = ceil_div64(rows, row_blocks); row_blocks = ceil_div64(rows, rows_per_block); }
  kv_channel_stats_kernel<T><<<dim3((unsigned)col_blocks, (unsigned)row_blocks), kThreads, 0, h->stream>>>(x, rows, cols, rows_per_block, keys);
  kv_channel_params_kernel<<<(unsigned)ceil_div64(cols, kThreads), kThreads, 0, h->stream>>>(keys, cols, (float)qmax, scales, zps);
  const int64_t n = rows * cols;
  const bool vec = cols % 4 == 0 && (reinterpret_cast<uintptr_t>(x) % (4 * sizeof(T))) == 0 && (reinterpret_cast<uintptr_t>(codes) & 3) == 0 &&
                   (reinterpret_cast<uintptr_t>(scales) & 15) == 0 && (reinterpret_cast<uintptr_t>(zps) & 15) == 0;
  if (vec) kv_quantize_per_channel_kernel<T, true><<<grid_cap(h, ceil_div64(n, kThreads * 4)), kThreads, 0, h->stream>>>(x, n, cols, qmax, scales, zps, codes);
  else kv_quantize_per_channel_kernel<T, false><<<grid_cap(h, ceil_div64(n, kThreads)), kThreads, 0, h->stream>>>(x, n, cols, qmax, scales, zps, codes);
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
  kv_dequantize_kernel<T><<<grid_cap(h, ceil_div64(n, kThreads * 4)), kThreads, 0, h->stream>>>(codes, n, head_dim, axis, signed_codes, scales, zps, out);
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
