// GGML block codecs on the GPU: Q8_0, Q4_0, Q4_1 (blocks of 32 weights) and Q4_K (super-blocks of 256), the on-disk
// weight formats of crates/oxicuda-quant/src/scheme/ggml.rs (quantize_* :243-472, dequantize_* :265-506).  Blocks are
// packed little-endian records in the field order of the reference's structs:
//   Q8_0 {d f16, qs i8[32]}                                   34 bytes
//   Q4_0 {d f16, qs u8[16]}   (byte i: code i | code i+16 << 4)   18 bytes
//   Q4_1 {d f16, m f16, qs u8[16]}                             20 bytes
//   Q4_K {d f16, dmin f16, scales u8[8], mins u8[8], qs u8[128]} (byte i: code 2i | code 2i+1 << 4)  148 bytes
// Quantization is bit-exact with the reference's arithmetic: IEEE divisions for the scales, binary16 rounding to nearest
// even (the hardware conversion), w * (1 / dq) with roundf (half away from zero) and a clamp.  One warp owns a block of
// 32 (lane = element) or a super-block of 256 (lane = element of each of the 8 sub-blocks); records have odd sizes, so
// they are written and read bytewise or as 16-bit pieces.  HBM-bound byte work: 4 B read + 0.56-1.06 B written per
// weight when quantizing, the reverse when dequantizing.
#include "common.cuh"
#include <cuda_fp16.h>

namespace ggml {

constexpr int kThreads = 256;
__device__ __forceinline__ float f16_round(float x) { return __half2float(__float2half_rn(x)); }
__device__ __forceinline__ uint16_t f16_bits(float x) { const __half h = __float2half_rn(x); return *reinterpret_cast<const uint16_t*>(&h); }
__device__ __forceinline__ float f16_from_bits(uint16_t b) { return __half2float(*reinterpret_cast<const __half*>(&b)); }
__device__ __forceinline__ float clampf(float v, float lo, float hi) { return v < lo ? lo : (v > hi ? hi : v); }
__device__ __forceinline__ float wmax(float v) { for (int o = 16; o; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o)); return v; }
__device__ __forceinline__ float wmin(float v) { for (int o = 16; o; o >>= 1) v = fminf(v, __shfl_xor_sync(0xffffffffu, v, o)); return v; }
__device__ __forceinline__ void put16(uint8_t* p, uint16_t v) { p[0] = (uint8_t)(v & 0xFF); p[1] = (uint8_t)(v >> 8); }
__device__ __forceinline__ uint16_t get16(const uint8_t* p) { return (uint16_t)(p[0] | (p[1] << 8)); }

// Blocks of 32: TYPE 0 Q8_0, 1 Q4_0, 2 Q4_1.
template <int TYPE>
__global__ void __launch_bounds__(kThreads) quantize32_kernel(const float* __restrict__ w, int64_t nblocks, uint8_t* __restrict__ out) {
  constexpr int BB = TYPE == 0 ? 34 : (TYPE == 1 ? 18 : 20);
  const int lane = threadIdx.x & 31;
  const int64_t warp = (int64_t)blockIdx.x * (kThreads / 32) + (threadIdx.x >> 5), nwarps = (int64_t)gridDim.x * (kThreads / 32);
  for (int64_t b = warp; b < nblocks; b += nwarps) {
    const float v = w[b * 32 + lane];
    uint8_t* o = out + b * BB;
    if constexpr (TYPE == 0) {
      const float amax = wmax(fabsf(v));
      const float d = __fdiv_rn(amax, 127.0f), dq = f16_round(d), inv = dq > 0.0f ? __fdiv_rn(1.0f, dq) : 0.0f;
      if (lane == 0) put16(o, f16_bits(d));
      o[2 + lane] = (uint8_t)(int8_t)clampf(roundf(__fmul_rn(v, inv)), -127.0f, 127.0f);
    } else if constexpr (TYPE == 1) {
      // the signed value of the FIRST element with the largest magnitude (strict > in the reference's scan)
      const float a = fabsf(v), amax = wmax(a);
      const unsigned first = __ffs(__ballot_sync(0xffffffffu, a == amax)) - 1;
      const float mx = amax > 0.0f ? __shfl_sync(0xffffffffu, v, first) : 0.0f;
      const float d = __fdiv_rn(mx, -8.0f), dq = f16_round(d), inv = dq != 0.0f ? __fdiv_rn(1.0f, dq) : 0.0f;
      const uint32_t code = (uint32_t)clampf(__fadd_rn(roundf(__fmul_rn(v, inv)), 8.0f), 0.0f, 15.0f);
      const uint32_t hi = __shfl_down_sync(0xffffffffu, code, 16);
      if (lane == 0) put16(o, f16_bits(d));
      if (lane < 16) o[2 + lane] = (uint8_t)(code | (hi << 4));
    } else {
      const float mn = wmin(v), mx = wmax(v);
      const float d = __fdiv_rn(__fsub_rn(mx, mn), 15.0f), dq = f16_round(d), mq = f16_round(mn), inv = dq > 0.0f ? __fdiv_rn(1.0f, dq) : 0.0f;
      const uint32_t code = (uint32_t)clampf(roundf(__fmul_rn(__fsub_rn(v, mq), inv)), 0.0f, 15.0f);
      const uint32_t hi = __shfl_down_sync(0xffffffffu, code, 16);
      if (lane == 0) { put16(o, f16_bits(d)); put16(o + 2, f16_bits(mn)); }
      if (lane < 16) o[4 + lane] = (uint8_t)(code | (hi << 4));
    }
  }
}

// Q4_K: one warp per super-block; lane l holds element l of each of the 8 sub-blocks.
__global__ void __launch_bounds__(kThreads) quantize_q4k_kernel(const float* __restrict__ w, int64_t nblocks, uint8_t* __restrict__ out) {
  const int lane = threadIdx.x & 31;
  const int64_t warp = (int64_t)blockIdx.x * (kThreads / 32) + (threadIdx.x >> 5), nwarps = (int64_t)gridDim.x * (kThreads / 32);
  for (int64_t b = warp; b < nblocks; b += nwarps) {
    float v[8], sub_scale[8], sub_min[8];
    float max_scale = 0.0f, max_min = 0.0f;
#pragma unroll
    for (int sb = 0; sb < 8; ++sb) {
      v[sb] = w[b * 256 + sb * 32 + lane];
      const float mn = fminf(wmin(v[sb]), 0.0f), mx = wmax(v[sb]);
      sub_scale[sb] = __fdiv_rn(__fsub_rn(mx, mn), 15.0f);
      sub_min[sb] = -mn;
      max_scale = fmaxf(max_scale, sub_scale[sb]);
      max_min = fmaxf(max_min, sub_min[sb]);
    }
    max_min = __fadd_rn(max_min, 0.0f);        // a zero maximum of -0.0 entries: +0 (the reference's f32::max leaves the sign open)
    const float d = __fdiv_rn(max_scale, 63.0f), dmin = __fdiv_rn(max_min, 63.0f), dq = f16_round(d), dminq = f16_round(dmin);
    const float inv_d = dq > 0.0f ? __fdiv_rn(1.0f, dq) : 0.0f, inv_dmin = dminq > 0.0f ? __fdiv_rn(1.0f, dminq) : 0.0f;
    uint8_t* o = out + b * 148;
    if (lane == 0) { put16(o, f16_bits(d)); put16(o + 2, f16_bits(dmin)); }
#pragma unroll
    for (int sb = 0; sb < 8; ++sb) {
      const float qs = clampf(roundf(__fmul_rn(sub_scale[sb], inv_d)), 0.0f, 63.0f), qm = clampf(roundf(__fmul_rn(sub_min[sb], inv_dmin)), 0.0f, 63.0f);
      if (lane == 0) { o[4 + sb] = (uint8_t)qs; o[12 + sb] = (uint8_t)qm; }
      const float sc = __fmul_rn(dq, qs), mn = __fmul_rn(dminq, qm), inv_sc = sc > 0.0f ? __fdiv_rn(1.0f, sc) : 0.0f;
      const uint32_t code = (uint32_t)clampf(roundf(__fmul_rn(__fadd_rn(v[sb], mn), inv_sc)), 0.0f, 15.0f);
      const uint32_t nxt = __shfl_down_sync(0xffffffffu, code, 1);            // code 2i + 1 sits in the next lane
      if ((lane & 1) == 0) o[20 + sb * 16 + (lane >> 1)] = (uint8_t)(code | (nxt << 4));
    }
  }
}

template <typename TOut> __device__ __forceinline__ void store_out(TOut* p, float v);
template <> __device__ __forceinline__ void store_out<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void store_out<__nv_bfloat16>(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }

// One thread per weight (grid-stride): the record bytes of a block are shared by its 32 / 256 threads through L1.
template <int TYPE, typename TOut>
__global__ void __launch_bounds__(kThreads) dequantize_kernel(const uint8_t* __restrict__ blocks, int64_t n, TOut* __restrict__ out) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    float v;
    if constexpr (TYPE == 0) {
      const uint8_t* p = blocks + (i >> 5) * 34;
      v = __fmul_rn((float)(int8_t)p[2 + (i & 31)], f16_from_bits(get16(p)));
    } else if constexpr (TYPE == 1) {
      const uint8_t* p = blocks + (i >> 5) * 18;
      const int k = (int)(i & 31);
      const int q = k < 16 ? (p[2 + k] & 0x0F) : (p[2 + k - 16] >> 4);
      v = __fmul_rn((float)(q - 8), f16_from_bits(get16(p)));
    } else if constexpr (TYPE == 2) {
      const uint8_t* p = blocks + (i >> 5) * 20;
      const int k = (int)(i & 31);
      const int q = k < 16 ? (p[4 + k] & 0x0F) : (p[4 + k - 16] >> 4);
      v = __fadd_rn(__fmul_rn((float)q, f16_from_bits(get16(p))), f16_from_bits(get16(p + 2)));
    } else {
      const uint8_t* p = blocks + (i >> 8) * 148;
      const int k = (int)(i & 255), sb = k >> 5;
      const float sc = __fmul_rn(f16_from_bits(get16(p)), (float)p[4 + sb]), mn = __fmul_rn(f16_from_bits(get16(p + 2)), (float)p[12 + sb]);
      const int q = (k & 1) ? (p[20 + (k >> 1)] >> 4) : (p[20 + (k >> 1)] & 0x0F);
      v = __fsub_rn(__fmul_rn(sc, (float)q), mn);
    }
    store_out<TOut>(out + i, v);
  }
}

static inline int block_size(int type) { return type == B2Q_GGML_Q4_K ? 256 : 32; }

}  // namespace ggml

extern "C" {

int64_t b2q_ggml_block_bytes(int type) {
  return type == B2Q_GGML_Q8_0 ? 34 : type == B2Q_GGML_Q4_0 ? 18 : type == B2Q_GGML_Q4_1 ? 20 : type == B2Q_GGML_Q4_K ? 148 : -1;
}
int64_t b2q_ggml_block_size(int type) { return type < 0 || type > 3 ? -1 : ggml::block_size(type); }

int32_t b2q_ggml_quantize_f32(b2q_handle h, int type, const float* w, int64_t n, uint8_t* blocks) {
  B2Q_REQUIRE_HANDLE(h);
  if (type < 0 || type > 3) B2Q_FAIL(h, B2Q_ERR_INVALID_ARGUMENT, "ggml_quantize: unknown block type %d", type);
  if (n <= 0) B2Q_FAIL(h, B2Q_ERR_EMPTY_INPUT, "ggml quantize: empty input");
  const int bs = ggml::block_size(type);
  if (n % bs != 0) B2Q_FAIL(h, B2Q_ERR_GROUP_SIZE_MISMATCH, "ggml quantize: len %lld not divisible by group %d", (long long)n, bs);
  if (!w || !blocks) B2Q_FAIL(h, B2Q_ERR_INVALID_ARGUMENT, "ggml_quantize: null pointer");
  const int64_t nb = n / bs;
  int64_t g = ceil_div64(nb, ggml::kThreads / 32);
  if (g > (int64_t)h->sm_count * 16) g = (int64_t)h->sm_count * 16;
  if (type == B2Q_GGML_Q8_0) ggml::quantize32_kernel<0><<<(int)g, ggml::kThreads, 0, h->stream>>>(w, nb, blocks);
  else if (type == B2Q_GGML_Q4_0) ggml::quantize32_kernel<1><<<(int)g, ggml::kThreads, 0, h->stream>>>(w, nb, blocks);
  else if (type == B2Q_GGML_Q4_1) ggml::quantize32_kernel<2><<<(int)g, ggml::kThreads, 0, h->stream>>>(w, nb, blocks);
  else ggml::quantize_q4k_kernel<<<(int)g, ggml::kThreads, 0, h->stream>>>(w, nb, blocks);
  B2Q_LAUNCH_CHECK(h, "ggml quantize kernel");
  return B2Q_OK;
}

int32_t b2q_ggml_dequantize(b2q_handle h, int type, const uint8_t* blocks, int64_t n, void* out, int out_type) {
  B2Q_REQUIRE_HANDLE(h);
  if (type < 0 || type > 3) B2Q_FAIL(h, B2Q_ERR_INVALID_ARGUMENT, "ggml_dequantize: unknown block type %d", type);
  if (n <= 0) return B2Q_OK;                                 // the reference returns an empty vector for no blocks
  const int bs = ggml::block_size(type);
  if (n % bs != 0) B2Q_FAIL(h, B2Q_ERR_GROUP_SIZE_MISMATCH, "ggml dequantize: len %lld not divisible by group %d", (long long)n, bs);
  if (!blocks || !out || out_type < 0 || out_type > 1) B2Q_FAIL(h, B2Q_ERR_INVALID_ARGUMENT, "ggml_dequantize: bad argument");
  int64_t g = ceil_div64(n, ggml::kThreads);
  if (g > (int64_t)h->sm_count * 32) g = (int64_t)h->sm_count * 32;
#define GGML_DEQ(T)                                                                                                              \
  do {                                                                                                                           \
    if (out_type == B2Q_OUT_BF16) ggml::dequantize_kernel<T, __nv_bfloat16><<<(int)g, ggml::kThreads, 0, h->stream>>>(blocks, n, (__nv_bfloat16*)out); \
    else ggml::dequantize_kernel<T, float><<<(int)g, ggml::kThreads, 0, h->stream>>>(blocks, n, (float*)out);                     \
  } while (0)
  if (type == B2Q_GGML_Q8_0) GGML_DEQ(0);
  else if (type == B2Q_GGML_Q4_0) GGML_DEQ(1);
  else if (type == B2Q_GGML_Q4_1) GGML_DEQ(2);
  else GGML_DEQ(3);
#undef GGML_DEQ
  B2Q_LAUNCH_CHECK(h, "ggml dequantize kernel");
  return B2Q_OK;
}

}  // extern "C"
