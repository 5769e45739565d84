// FP8 GEMM, checker arithmetic on the GPU: software decode of the codes (reference
// codec or IEEE), k-ascending fp32 FMA per output element, then the scale and the
// bf16/f32 store.  This is the arithmetic order of the reference's only complete
// GEMM kernel (one thread per C element, fma.rn.f32 over ascending k).  It serves
// decode-sized shapes and row pitches TMA cannot take, and is the exact-order
// comparison for the tensor-core path.
#include "common.cuh"

namespace {

constexpr int T = 16;   // 16x16 outputs per CTA, K staged 64 at a time through a decode LUT

__global__ void __launch_bounds__(T * T) gemm_fp8_simt_kernel(const uint8_t* __restrict__ a, const uint8_t* __restrict__ w,
                                                              int64_t M, int64_t N, int64_t K, int fmt, int decode_mode,
                                                              const float* sa, int sa_rows, const float* sw, int sw_rows,
                                                              void* out, int out_type) {
  __shared__ float lut[256];
  __shared__ float As[T][65];
  __shared__ float Ws[T][65];
  const Fp8Fmt F = fp8_fmt(fmt);
  const int tid = threadIdx.y * T + threadIdx.x;
  lut[tid] = decode_mode == 0 ? fp8_decode_ref_dev((uint32_t)tid, F) : fp8_decode_ieee_dev((uint32_t)tid, F);
  __syncthreads();
  const int64_t m = (int64_t)blockIdx.y * T + threadIdx.y;
  const int64_t n = (int64_t)blockIdx.x * T + threadIdx.x;
  float acc = 0.0f;
  for (int64_t k0 = 0; k0 < K; k0 += 64) {
    for (int i = tid; i < T * 64; i += T * T) {
      int r = i >> 6, kk = i & 63;
      int64_t k = k0 + kk;
      int64_t am = (int64_t)blockIdx.y * T + r, wn = (int64_t)blockIdx.x * T + r;
      As[r][kk] = (am < M && k < K) ? lut[a[am * K + k]] : 0.0f;
      Ws[r][kk] = (wn < N && k < K) ? lut[w[wn * K + k]] : 0.0f;
    }
    __syncthreads();
    const int kmax = (int)((K - k0) < 64 ? (K - k0) : 64);
    for (int kk = 0; kk < kmax; ++kk) acc = __fmaf_rn(As[threadIdx.y][kk], Ws[threadIdx.x][kk], acc);
    __syncthreads();
  }
  if (m < M && n < N) {
    float s = __fmul_rn(sa_rows ? sa[m] : sa[0], sw_rows ? sw[n] : sw[0]);
    float v = __fmul_rn(acc, s);
    if (out_type == B2Q_OUT_BF16) reinterpret_cast<__nv_bfloat16*>(out)[m * N + n] = __float2bfloat16_rn(v);
    else reinterpret_cast<float*>(out)[m * N + n] = v;
  }
}

}  // namespace

// out_cols: the columns of out when they are not N (the SwiGLU-pair epilogue writes N / 2); 0 = N.
int32_t b2q_validate_gemm_fp8(b2q_handle h, const uint8_t* a, const uint8_t* w, int64_t M, int64_t N, int64_t K, int fmt,
                              const float* scale_a, int ka, const float* scale_w, int kw, void* out, int out_type, int64_t out_cols) {
  // Order follows the reference's gemm_impl: dimensions first, then argument checks, then overlap.
  if (M <= 0 || N <= 0 || K <= 0)
    B2Q_FAIL(h, B2Q_ERR_INVALID_DIMENSION, "FP8 GEMM dimensions must be non-zero: m=%lld, n=%lld, k=%lld", (long long)M, (long long)N, (long long)K);
  if (!a || !w || !out || !scale_a || !scale_w) B2Q_FAIL(h, B2Q_ERR_INVALID_ARGUMENT, "gemm_fp8: null pointer");
  if (fmt < 0 || fmt > 1 || ka < 0 || ka > 1 || kw < 0 || kw > 1 || out_type < 0 || out_type > 1)
    B2Q_FAIL(h, B2Q_ERR_INVALID_ARGUMENT, "gemm_fp8: bad enum value");
  const uintptr_t c0 = reinterpret_cast<uintptr_t>(out), c1 = c0 + (size_t)(M * (out_cols > 0 ? out_cols : N)) * (out_type == B2Q_OUT_BF16 ? 2 : 4);
  const uintptr_t a0 = reinterpret_cast<uintptr_t>(a), a1 = a0 + (size_t)(M * K);
  const uintptr_t w0 = reinterpret_cast<uintptr_t>(w), w1 = w0 + (size_t)(N * K);
  if ((c0 < a1 && a0 < c1) || (c0 < w1 && w0 < c1))
    B2Q_FAIL(h, B2Q_ERR_INVALID_ARGUMENT, "gemm_fp8: output buffer overlaps an input");
  return B2Q_OK;
}

extern "C" int32_t b2q_gemm_fp8_simt(b2q_handle h, const uint8_t* a, const uint8_t* w, int64_t M, int64_t N, int64_t K, int fmt,
                                     int decode_mode, const float* scale_a, int scale_a_kind, const float* scale_w,
                                     int scale_w_kind, void* out, int out_type) {
  B2Q_REQUIRE_HANDLE(h);
  int32_t st = b2q_validate_gemm_fp8(h, a, w, M, N, K, fmt, scale_a, scale_a_kind, scale_w, scale_w_kind, out, out_type, 0);
  if (st != B2Q_OK) return st;
  if (decode_mode < 0 || decode_mode > 1) B2Q_FAIL(h, B2Q_ERR_INVALID_ARGUMENT, "gemm_fp8_simt: bad decode mode");
  dim3 grid((unsigned)ceil_div64(N, T), (unsigned)ceil_div64(M, T));
  gemm_fp8_simt_kernel<<<grid, dim3(T, T), 0, h->stream>>>(a, w, M, N, K, fmt, decode_mode, scale_a, scale_a_kind, scale_w,
                                                           scale_w_kind, out, out_type);
  B2Q_LAUNCH_CHECK(h, "gemm_fp8_simt_kernel");
  return B2Q_OK;
}
