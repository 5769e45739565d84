// Weight-only block-scaled FP4 GEMM for prefill-sized token counts:
//   out[t, n] = sum_k x[t, k] * decode(codes[n, k]) * scale[n, k / block]
// Fp4GemmConfig / generate_fp4_gemm_ptx (crates/oxicuda-blas/src/precision/fp4_fp6_ops.rs:337-395, :1237-1362) with the
// defined semantics dequantize_fp4 (:879-897) followed by a matmul.  The weights are expanded once per call to bf16 in
// the handle's workspace (E2M1 times a power-of-two scale is exact in bf16; an f32 scale rounds to 8 bits) and the
// product runs on tcgen05 (kind::f16, fp32 accumulation in TMEM).  Token counts of 32 and below take the decode GEMV.
#include "common.cuh"

int32_t b2q_gemm_bf16_tc(b2q_handle h, const void* a, const void* w, int64_t M, int64_t N, int64_t K, void* out, int out_type);

namespace {

// 16 codes (8 bytes) per thread -> 16 bf16 (32 bytes)
__global__ void __launch_bounds__(256) fp4_expand_bf16_kernel(const uint2* __restrict__ packed, int64_t n16, int block, int format,
                                                              const float* __restrict__ sf, const uint8_t* __restrict__ se,
                                                              uint4* __restrict__ out) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n16; i += (int64_t)gridDim.x * blockDim.x) {
    const uint2 w = packed[i];
    const int64_t b = (i * 16) / block;
    const float scale = sf ? sf[b] : e8m0_to_f32_dev(se[b]);
    uint32_t o[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const uint32_t byte = ((j < 4 ? w.x : w.y) >> (8 * (j & 3))) & 0xFF;
      const float lo = (format == 0 ? e2m1_decode_dev(byte & 0xF) : int4_decode_dev(byte & 0xF)) * scale;
      const float hi = (format == 0 ? e2m1_decode_dev(byte >> 4) : int4_decode_dev(byte >> 4)) * scale;
      __nv_bfloat162 h2 = __floats2bfloat162_rn(lo, hi);
      o[j] = *reinterpret_cast<uint32_t*>(&h2);
    }
    out[2 * i] = make_uint4(o[0], o[1], o[2], o[3]);
    out[2 * i + 1] = make_uint4(o[4], o[5], o[6], o[7]);
  }
}

}  // namespace

extern "C" int32_t b2q_gemm_fp4_wo(b2q_handle h, const uint8_t* codes, const void* scales, int scale_format, int block, int format,
                                   const void* x_bf16, int64_t tokens, int64_t N, int64_t K, void* out, int out_type) {
  B2Q_REQUIRE_HANDLE(h);
  if (tokens <= 0 || N <= 0 || K <= 0)
    B2Q_FAIL(h, B2Q_ERR_INVALID_DIMENSION, "FP4 GEMM dimensions must be non-zero: m=%lld, n=%lld, k=%lld", (long long)N, (long long)tokens, (long long)K);
  if (K % 2 != 0) B2Q_FAIL(h, B2Q_ERR_INVALID_DIMENSION, "FP4 GEMM K dimension must be even for packing, got k=%lld", (long long)K);
  if (block != 32 && block != 64 && block != 128)
    B2Q_FAIL(h, B2Q_ERR_INVALID_ARGUMENT, "MicroScaling block_size must be one of [32, 64, 128], got %d", block);
  if (!codes || !scales || !x_bf16 || !out || scale_format < 0 || scale_format > 1 || format < 0 || format > 1 || out_type < 0 || out_type > 1)
    B2Q_FAIL(h, B2Q_ERR_INVALID_ARGUMENT, "gemm_fp4_wo: bad argument");
  if (tokens <= 32 && block == 32 && format == 0 && K % 128 == 0)
    return b2q_gemv_fp4_wo(h, codes, scales, scale_format, block, x_bf16, tokens, N, K, out, out_type);
  if (scale_format == B2Q_SCALE_E8M0 && block == 32 && format == 0 && K % 128 == 0 && (reinterpret_cast<uintptr_t>(codes) & 31) == 0 &&
      (reinterpret_cast<uintptr_t>(scales) & 3) == 0 && (reinterpret_cast<uintptr_t>(x_bf16) & 15) == 0)
    return b2q_gemm_fp4_blockscaled(h, codes, (const uint8_t*)scales, x_bf16, tokens, N, K, B2Q_FP4_ACT_SPLIT, out, out_type);
  if (K % block != 0 || K % 16 != 0) B2Q_FAIL(h, B2Q_ERR_INVALID_DIMENSION, "gemm_fp4_wo: K must be a multiple of the block size and of 16, got %lld", (long long)K);
  if (((reinterpret_cast<uintptr_t>(codes) & 7) | (reinterpret_cast<uintptr_t>(x_bf16) & 15)) != 0)
    B2Q_FAIL(h, B2Q_ERR_INVALID_ARGUMENT, "gemm_fp4_wo: codes must be 8-byte and activations 16-byte aligned");
  void* ws = nullptr;
  int32_t st = b2q_workspace(h, (size_t)N * (size_t)K * 2, &ws);
  if (st != B2Q_OK) return st;
  const int64_t n16 = N * K / 16;
  int64_t g = ceil_div64(n16, 256);
  if (g > (int64_t)h->sm_count * 16) g = (int64_t)h->sm_count * 16;
  fp4_expand_bf16_kernel<<<(int)g, 256, 0, h->stream>>>((const uint2*)codes, n16, block, format,
                                                        scale_format == B2Q_SCALE_F32 ? (const float*)scales : nullptr,
                                                        scale_format == B2Q_SCALE_E8M0 ? (const uint8_t*)scales : nullptr, (uint4*)ws);
  B2Q_LAUNCH_CHECK(h, "fp4_expand_bf16_kernel");
  st = b2q_gemm_bf16_tc(h, x_bf16, ws, tokens, N, K, out, out_type);
  if (st == B2Q_ERR_UNSUPPORTED) B2Q_FAIL(h, B2Q_ERR_UNSUPPORTED, "gemm_fp4_wo: shape or alignment not supported by the tensor-core path");
  return st;
}
