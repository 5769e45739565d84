// The second public quantize surface of the reference (oxicuda-dnn): per-tensor FP8 E4M3 and INT8 with the scale
// kept on the device, the block-scaled "FP4 proxy" bytes, and the host-side BlockQuantizedInt8 / Fp4BlockQuantizer
// rules, as CUDA kernels.  crates/oxicuda-dnn/src/quantize/{fp8_quantize,int8_quantize,block_scale}.rs; the
// arithmetic follows the statements the reference's GPU tests check bit for bit
// (crates/oxicuda-dnn/src/gpu_tests/quantize.rs:184-325, :503-554): div.rn for every division, round to nearest
// even (cvt.rni) for the integer codes, the E4M3 encoder with ties to even and saturation to 0x7E.
// HBM-bound: 4 bytes read (twice for the per-tensor forms: absmax pass, then the codes) and 1 written per element.
#include "common.cuh"

namespace {

constexpr int kThreads = 256;

enum ScaleRule { kFloorTiny = 0, kOneForZero = 1 };   // max(absmax / m, 1e-12)  |  absmax > 0 ? absmax / m : 1
enum CodeRule { kCodeE4M3 = 0, kCodeInt8Rne = 1, kCodeBlockProxy = 2, kCodeInt8HalfAway = 3 };

__device__ __forceinline__ float group_scale(float absmax, float max_val, int rule) {
  const float s = __fdiv_rn(absmax, max_val);
  return rule == kFloorTiny ? fmaxf(s, 1e-12f) : (absmax > 0.0f ? s : 1.0f);
}

// Groups of up to a few thousand elements: a warp per group (the last group may be short).
__global__ void __launch_bounds__(kThreads) group_scale_warp_kernel(const float* __restrict__ x, int64_t n, int64_t block, float max_val, int rule,
                                                                    float* __restrict__ scales) {
  const int lane = threadIdx.x & 31;
  const int64_t groups = (n + block - 1) / block;
  for (int64_t g = (int64_t)blockIdx.x * (kThreads / 32) + (threadIdx.x >> 5); g < groups; g += (int64_t)gridDim.x * (kThreads / 32)) {
    const int64_t b = g * block, e = b + block < n ? b + block : n;
    float amax = 0.0f;
    if (((reinterpret_cast<uintptr_t>(x + b) & 15) == 0)) {
      const int64_t n4 = (e - b) >> 2;
      for (int64_t i = lane; i < n4; i += 32) {
        const float4 q = reinterpret_cast<const float4*>(x + b)[i];
        amax = fmaxf(fmaxf(amax, fmaxf(fabsf(q.x), fabsf(q.y))), fmaxf(fabsf(q.z), fabsf(q.w)));
      }
      for (int64_t i = b + (n4 << 2) + lane; i < e; i += 32) amax = fmaxf(amax, fabsf(x[i]));
    } else {
      for (int64_t i = b + lane; i < e; i += 32) amax = fmaxf(amax, fabsf(x[i]));
    }
    amax = warp_max(amax);
    if (lane == 0) scales[g] = group_scale(amax, max_val, rule);
  }
}

// One group over the whole tensor: grid-wide absmax through an atomic on the float's bits (non-negative floats order
// like unsigned integers), then the scale.  `key` is one zeroed word of the handle's scratch.
__global__ void tensor_absmax_init_kernel(uint32_t* key) { *key = 0u; }
__global__ void __launch_bounds__(kThreads) tensor_absmax_kernel(const float* __restrict__ x, int64_t n, uint32_t* key) {
  __shared__ float sh[kThreads / 32];
  const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x, nth = (int64_t)gridDim.x * blockDim.x;
  float amax = 0.0f;
  if ((reinterpret_cast<uintptr_t>(x) & 15) == 0) {
    const int64_t n4 = n >> 2;
    for (int64_t i = tid; i < n4; i += nth) {
      const float4 q = reinterpret_cast<const float4*>(x)[i];
      amax = fmaxf(fmaxf(amax, fmaxf(fabsf(q.x), fabsf(q.y))), fmaxf(fabsf(q.z), fabsf(q.w)));
    }
    for (int64_t i = (n4 << 2) + tid; i < n; i += nth) amax = fmaxf(amax, fabsf(x[i]));
  } else {
    for (int64_t i = tid; i < n; i += nth) amax = fmaxf(amax, fabsf(x[i]));
  }
  amax = warp_max(amax);
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = amax;
  __syncthreads();
  if (threadIdx.x < 32) {
    amax = threadIdx.x < kThreads / 32 ? sh[threadIdx.x] : 0.0f;
    amax = warp_max(amax);
    if (threadIdx.x == 0) atomicMax(key, __float_as_uint(amax));
  }
}
__global__ void tensor_scale_kernel(const uint32_t* key, float max_val, int rule, float* scale) {
  *scale = group_scale(__uint_as_float(*key), max_val, rule);
}

// One output byte.  `v` is the element, `s` its group's scale.
__device__ __forceinline__ uint32_t dnn_code(float v, float s, int rule) {
  const float q = __fdiv_rn(v, s);
  if (rule == kCodeE4M3) {
    // clamp to +-448 (NaN stays NaN), then the encoder of the reference's tests (gpu_tests/quantize.rs:64-109): ties to
    // even, flush below 2^-10, 0x7E from 448 up; that is the hardware conversion except that NaN also encodes as 0x7E
    const float c = q < -448.0f ? -448.0f : (q > 448.0f ? 448.0f : q);
    if (c != c) return ((__float_as_uint(c) >> 24) & 0x80u) | 0x7Eu;
    return (uint32_t)__nv_cvt_float_to_fp8(c, __NV_SATFINITE, __NV_E4M3);
  }
  if (rule == kCodeInt8Rne) {          // rne(clamp(x / s, -127, 127)) as i32 as i8   (:216-219)
    const float c = q < -127.0f ? -127.0f : (q > 127.0f ? 127.0f : q);
    return (uint32_t)__float2int_rn(c) & 0xFFu;                     // NaN -> 0
  }
  if (rule == kCodeBlockProxy) {       // clamp(rne(clamp(x / s, -6, 6)) + 6, 0, 255)   (:547-552)
    const float c = q < -6.0f ? -6.0f : (q > 6.0f ? 6.0f : q);
    const int r = __float2int_rn(c) + 6;
    return (uint32_t)(r < 0 ? 0 : (r > 255 ? 255 : r));
  }
  // BlockQuantizedInt8::quantize (int8_quantize.rs:440-443): (x / scale).round().clamp(-128, 127) as i8
  float r = roundf(q);
  r = r < -128.0f ? -128.0f : (r > 127.0f ? 127.0f : r);
  return (uint32_t)__float2int_rz(r) & 0xFFu;                       // NaN -> 0
}

// single != 0: one scale for the whole tensor.  vec != 0: block % 4 == 0 (or single) and aligned pointers.
__global__ void __launch_bounds__(kThreads) dnn_quantize_kernel(const float* __restrict__ x, int64_t n, int64_t block, int single,
                                                                const float* __restrict__ scales, int rule, uint8_t* __restrict__ out, int vec) {
  const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x, nth = (int64_t)gridDim.x * blockDim.x;
  const float s0 = scales[0];
  const int64_t n4 = vec ? n >> 2 : 0;
  for (int64_t i = tid; i < n4; i += nth) {
    const float s = single ? s0 : scales[(4 * i) / block];
    const float4 q = reinterpret_cast<const float4*>(x)[i];
    reinterpret_cast<uint32_t*>(out)[i] = dnn_code(q.x, s, rule) | (dnn_code(q.y, s, rule) << 8) | (dnn_code(q.z, s, rule) << 16) |
                                          (dnn_code(q.w, s, rule) << 24);
  }
  for (int64_t i = (n4 << 2) + tid; i < n; i += nth) out[i] = (uint8_t)dnn_code(x[i], single ? s0 : scales[i / block], rule);
}

// E4M3 decode of the reference's kernel (gpu_tests/quantize.rs:112-125): subnormals m / 512, every other code
// (0x7F included: 480) as the float with exponent field e + 120.
__device__ __forceinline__ float dnn_e4m3_decode(uint32_t b) {
  const uint32_t e = (b >> 3) & 0xFu, m = b & 7u;
  const float mag = e == 0 ? __fmul_rn((float)m, 1.0f / 512.0f) : __uint_as_float(((e + 120u) << 23) | (m << 20));
  return (b & 0x80u) ? -mag : mag;
}
// kind 0: E4M3 bytes, 1: int8.  out = value * scale.
__global__ void __launch_bounds__(kThreads) dnn_dequantize_kernel(const uint8_t* __restrict__ q, int64_t n, int64_t block, int single,
                                                                  const float* __restrict__ scales, int kind, float* __restrict__ out, int vec) {
  const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x, nth = (int64_t)gridDim.x * blockDim.x;
  const float s0 = scales[0];
  auto val = [&](uint32_t b) { return kind == 0 ? dnn_e4m3_decode(b) : (float)(int)(int8_t)b; };
  const int64_t n4 = vec ? n >> 2 : 0;
  for (int64_t i = tid; i < n4; i += nth) {
    const float s = single ? s0 : scales[(4 * i) / block];
    const uint32_t w = reinterpret_cast<const uint32_t*>(q)[i];
    reinterpret_cast<float4*>(out)[i] = make_float4(__fmul_rn(val(w & 0xFF), s), __fmul_rn(val((w >> 8) & 0xFF), s),
                                                    __fmul_rn(val((w >> 16) & 0xFF), s), __fmul_rn(val(w >> 24), s));
  }
  for (int64_t i = (n4 << 2) + tid; i < n; i += nth) out[i] = __fmul_rn(val(q[i]), single ? s0 : scales[i / block]);
}

inline int grid_cap(const b2q_handle h, int64_t blocks) {
  const int64_t cap = (int64_t)h->sm_count * 16;
  return (int)(blocks < 1 ? 1 : (blocks > cap ? cap : blocks));
}

// scales for groups of `block` elements (block >= n: one group), written to `scales`
int32_t launch_scales(b2q_handle h, const float* x, int64_t n, int64_t block, float max_val, int rule, float* scales) {
  if (block >= n && n > (1 << 16)) {
    uint32_t* key = h->d_scratch;
    tensor_absmax_init_kernel<<<1, 1, 0, h->stream>>>(key);
    tensor_absmax_kernel<<<grid_cap(h, ceil_div64(n, kThreads * 16)), kThreads, 0, h->stream>>>(x, n, key);
    tensor_scale_kernel<<<1, 1, 0, h->stream>>>(key, max_val, rule, scales);
  } else {
    const int64_t groups = ceil_div64(n, block);
    group_scale_warp_kernel<<<grid_cap(h, ceil_div64(groups, kThreads / 32)), kThreads, 0, h->stream>>>(x, n, block, max_val, rule, scales);
  }
  B2Q_LAUNCH_CHECK(h, "dnn scale kernels");
  return B2Q_OK;
}

int32_t quantize_common(b2q_handle h, const float* x, int64_t n, int64_t block, float max_val, int scale_rule, int code_rule, uint8_t* out,
                        float* scales, const char* what) {
  if (n == 0) return B2Q_OK;                       // the reference returns Ok(()) for an empty tensor
  if (n < 0 || block <= 0) B2Q_FAIL(h, B2Q_ERR_INVALID_ARGUMENT, "%s: n %lld, block %lld", what, (long long)n, (long long)block);
  if (!x || !out || !scales) B2Q_FAIL(h, B2Q_ERR_BUFFER_TOO_SMALL, "%s: missing buffer", what);
  const int32_t st = launch_scales(h, x, n, block, max_val, scale_rule, scales);
  if (st != B2Q_OK) return st;
  const int single = block >= n;
  const int vec = (single || block % 4 == 0) && (reinterpret_cast<uintptr_t>(x) & 15) == 0 && (reinterpret_cast<uintptr_t>(out) & 3) == 0;
  dnn_quantize_kernel<<<grid_cap(h, ceil_div64(n, kThreads * 4)), kThreads, 0, h->stream>>>(x, n, block, single, scales, code_rule, out, vec);
  B2Q_LAUNCH_CHECK(h, what);
  return B2Q_OK;
}

int32_t dequantize_common(b2q_handle h, const uint8_t* q, const float* scales, int64_t n, int64_t block, int kind, float* out, const char* what) {
  if (n == 0) return B2Q_OK;
  if (n < 0 || block <= 0) B2Q_FAIL(h, B2Q_ERR_INVALID_ARGUMENT, "%s: n %lld, block %lld", what, (long long)n, (long long)block);
  if (!q || !scales || !out) B2Q_FAIL(h, B2Q_ERR_BUFFER_TOO_SMALL, "%s: missing buffer", what);
  const int single = block >= n;
  const int vec = (single || block % 4 == 0) && (reinterpret_cast<uintptr_t>(out) & 15) == 0 && (reinterpret_cast<uintptr_t>(q) & 3) == 0;
  dnn_dequantize_kernel<<<grid_cap(h, ceil_div64(n, kThreads * 4)), kThreads, 0, h->stream>>>(q, n, block, single, scales, kind, out, vec);
  B2Q_LAUNCH_CHECK(h, what);
  return B2Q_OK;
}

}  // namespace

extern "C" {

int32_t b2q_dnn_quantize_to_fp8_f32(b2q_handle h, const float* x, int64_t n, uint8_t* codes, float* scale) {
  B2Q_REQUIRE_HANDLE(h);
  return quantize_common(h, x, n, n > 0 ? n : 1, 448.0f, kFloorTiny, kCodeE4M3, codes, scale, "quantize_to_fp8");
}
int32_t b2q_dnn_dequantize_from_fp8_f32(b2q_handle h, const uint8_t* codes, const float* scale, int64_t n, float* out) {
  B2Q_REQUIRE_HANDLE(h);
  return dequantize_common(h, codes, scale, n, n > 0 ? n : 1, 0, out, "dequantize_from_fp8");
}
int32_t b2q_dnn_quantize_to_int8_f32(b2q_handle h, const float* x, int64_t n, int8_t* q, float* scale) {
  B2Q_REQUIRE_HANDLE(h);
  return quantize_common(h, x, n, n > 0 ? n : 1, 127.0f, kFloorTiny, kCodeInt8Rne, reinterpret_cast<uint8_t*>(q), scale, "quantize_to_int8");
}
int32_t b2q_dnn_dequantize_from_int8_f32(b2q_handle h, const int8_t* q, const float* scale, int64_t n, float* out) {
  B2Q_REQUIRE_HANDLE(h);
  return dequantize_common(h, reinterpret_cast<const uint8_t*>(q), scale, n, n > 0 ? n : 1, 1, out, "dequantize_from_int8");
}
int32_t b2q_dnn_quantize_block_scaled_f32(b2q_handle h, const float* x, int64_t n, uint32_t block_size, uint8_t* out, float* scales) {
  B2Q_REQUIRE_HANDLE(h);
  if (n == 0) return B2Q_OK;
  if (block_size == 0 || (block_size & (block_size - 1)) != 0) B2Q_FAIL(h, B2Q_ERR_INVALID_ARGUMENT, "block_size must be a non-zero power of 2, got %u", block_size);
  if (block_size < 16) B2Q_FAIL(h, B2Q_ERR_INVALID_ARGUMENT, "block_size must be >= 16, got %u", block_size);
  // a block size above n still means one (short) block, never the single-scale shortcut with block >= n semantics changed
  return quantize_common(h, x, n, (int64_t)block_size, 6.0f, kFloorTiny, kCodeBlockProxy, out, scales, "quantize_block_scaled");
}
int32_t b2q_block_int8_quantize_f32(b2q_handle h, const float* x, int64_t n, int64_t block_size, int8_t* q, float* scales) {
  B2Q_REQUIRE_HANDLE(h);
  if (block_size <= 0) B2Q_FAIL(h, B2Q_ERR_INVALID_ARGUMENT, "block_size must be > 0");
  return quantize_common(h, x, n, block_size, 127.0f, kOneForZero, kCodeInt8HalfAway, reinterpret_cast<uint8_t*>(q), scales, "BlockQuantizedInt8::quantize");
}
int32_t b2q_block_int8_dequantize_f32(b2q_handle h, const int8_t* q, const float* scales, int64_t n, int64_t block_size, float* out) {
  B2Q_REQUIRE_HANDLE(h);
  if (block_size <= 0) B2Q_FAIL(h, B2Q_ERR_INVALID_ARGUMENT, "block_size must be > 0");
  return dequantize_common(h, reinterpret_cast<const uint8_t*>(q), scales, n, block_size, 1, out, "BlockQuantizedInt8::dequantize");
}
int32_t b2q_block_absmax_scale_f32(b2q_handle h, const float* x, int64_t n, int64_t block_size, float max_val, float* scales) {
  B2Q_REQUIRE_HANDLE(h);
  if (n == 0) return B2Q_OK;
  if (n < 0 || block_size <= 0 || !(max_val > 0.0f)) B2Q_FAIL(h, B2Q_ERR_INVALID_ARGUMENT, "block_absmax_scale: bad argument");
  if (!x || !scales) B2Q_FAIL(h, B2Q_ERR_BUFFER_TOO_SMALL, "block_absmax_scale: missing buffer");
  return launch_scales(h, x, n, block_size, max_val, kOneForZero, scales);
}

}  // extern "C"
