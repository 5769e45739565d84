// INT8 paths: the LLM.int8 W8A8 linear (quantize both operands on the fly, exact
// integer accumulation, fp32 outlier side path) and the pre-quantized INT8 GEMM
// with exact s32 accumulation.  Decode-sized problems (few activation rows) are
// HBM/launch bound: one warp per weight row, 128-bit loads, dp4a, shuffle reduce.
#include "common.cuh"

namespace {

constexpr int kThreads = 256;

// Column outlier mask: is_out[c] = max_r |x[r,c]| >= threshold; n_out counts them.
__global__ void outlier_mask_kernel(const float* x, int64_t samples, int64_t cols, float threshold,
                                    uint8_t* is_out, int32_t* n_out) {
  int64_t c = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  int flag = 0;
  if (c < cols) {
    float m = 0.0f;
    for (int64_t r = 0; r < samples; ++r) {
      float a = fabsf(x[r * cols + c]);
      if (a > m) m = a;
    }
    flag = m >= threshold;
    is_out[c] = (uint8_t)flag;
  }
  unsigned b = __ballot_sync(0xffffffffu, flag);
  if ((threadIdx.x & 31) == 0 && b) atomicAdd(n_out, __popc(b));
}

// Global masked absmax (per-tensor activation scale), key in *amax_bits.
__global__ void masked_absmax_kernel(const float* x, int64_t n, int64_t cols, const uint8_t* is_out, uint32_t* amax_bits) {
  float m = 0.0f;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
    if (!is_out[i % cols]) m = fmaxf(m, fabsf(x[i]));
  m = warp_max(m);
  if ((threadIdx.x & 31) == 0) atomicMax(amax_bits, __float_as_uint(m));
}

// One block per row: scale = amax/127 over the regular columns (1.0 when amax == 0),
// code = clamp(round(v * (1/scale)), +-127) (round half away from zero), outlier
// columns get code 0.  `global_amax_bits` (optional) replaces the per-row absmax.
__global__ void __launch_bounds__(kThreads) int8_row_quant_kernel(const float* x, int64_t cols, int64_t ld, const uint8_t* is_out,
                                                                  const uint32_t* global_amax_bits, int8_t* q, float* scales) {
  const int64_t r = blockIdx.x;
  const float* row = x + r * cols;
  __shared__ float sh[kThreads / 32];
  __shared__ float s_scale;
  float m = 0.0f;
  if (global_amax_bits) {
    m = __uint_as_float(*global_amax_bits);
  } else {
    for (int64_t c = threadIdx.x; c < cols; c += kThreads)
      if (!is_out[c]) m = fmaxf(m, fabsf(row[c]));
    m = warp_max(m);
    if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = m;
    __syncthreads();
    if (threadIdx.x == 0) {
      for (int w = 1; w < kThreads / 32; ++w) m = fmaxf(m, sh[w]);
      sh[0] = m;
    }
    __syncthreads();
    m = sh[0];
  }
  if (threadIdx.x == 0) {
    float sc = m > 0.0f ? __fdiv_rn(m, 127.0f) : 1.0f;
    s_scale = sc;
    scales[r] = sc;
  }
  __syncthreads();
  const float inv = __fdiv_rn(1.0f, s_scale);
  for (int64_t c = threadIdx.x; c < cols; c += kThreads) {
    int8_t code = 0;
    if (!is_out[c]) {
      float t = roundf(__fmul_rn(row[c], inv));
      t = t < -127.0f ? -127.0f : (t > 127.0f ? 127.0f : t);
      code = isnan(t) ? (int8_t)0 : (int8_t)(int)t;
    }
    q[r * ld + c] = code;
  }
  for (int64_t c = cols + threadIdx.x; c < ld; c += kThreads) q[r * ld + c] = 0;   // padding columns contribute nothing
}

// Small-M INT8 GEMM: C[m,n] = sum_k A[m,k] * B[n,k].  A (all M rows) is staged in
// shared memory; each warp owns one weight row n at a time and streams it with
// 128-bit loads.  MT = rows of A handled per pass (compile-time for unrolling).
// Epilogue: optional s32 store, optional f32 = f32(acc) * (sa[m]*sb[n]) [+ fp32 side term].
template <int MT>
__global__ void __launch_bounds__(kThreads) gemm_i8_small_m_kernel(
    const int8_t* __restrict__ a, const int8_t* __restrict__ b, int M, int64_t N, int64_t K, int32_t* c_s32,
    float* c_f32, const float* sa, const float* sb,
    // outlier side path (LLM.int8): fp32 operands and the mask; all null/0 when unused
    const float* xf, const float* wf, const uint8_t* is_out, const int32_t* n_out, int64_t Kf) {
  extern __shared__ __align__(16) int8_t sa_tile[];          // [M][K]
  const int64_t total = (int64_t)M * K;
  for (int64_t i = (int64_t)threadIdx.x * 16; i < total; i += (int64_t)kThreads * 16)
    *reinterpret_cast<int4*>(sa_tile + i) = *reinterpret_cast<const int4*>(a + i);
  __syncthreads();
  const int lane = threadIdx.x & 31;
  const int64_t warp = (int64_t)blockIdx.x * (kThreads / 32) + (threadIdx.x >> 5);
  const int64_t nwarps = (int64_t)gridDim.x * (kThreads / 32);
  const bool side = n_out != nullptr && *n_out > 0;
  for (int64_t n = warp; n < N; n += nwarps) {
    const int8_t* brow = b + n * K;
    for (int m0 = 0; m0 < M; m0 += MT) {
      int32_t acc[MT];
#pragma unroll
      for (int t = 0; t < MT; ++t) acc[t] = 0;
      for (int64_t k = (int64_t)lane * 16; k < K; k += 32 * 16) {
        int4 w = *reinterpret_cast<const int4*>(brow + k);
#pragma unroll
        for (int t = 0; t < MT; ++t) {
          if (m0 + t < M) {
            int4 v = *reinterpret_cast<const int4*>(sa_tile + (int64_t)(m0 + t) * K + k);
            acc[t] = __dp4a(v.x, w.x, acc[t]);
            acc[t] = __dp4a(v.y, w.y, acc[t]);
            acc[t] = __dp4a(v.z, w.z, acc[t]);
            acc[t] = __dp4a(v.w, w.w, acc[t]);
          }
        }
      }
#pragma unroll
      for (int t = 0; t < MT; ++t) {
        int32_t v = acc[t];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
        acc[t] = v;
      }
      if (lane < MT && m0 + lane < M) {
        const int m = m0 + lane;
        int32_t v = 0;
#pragma unroll
        for (int t = 0; t < MT; ++t) if (t == lane) v = acc[t];
        if (c_s32) c_s32[(int64_t)m * N + n] = v;
        if (c_f32) {
          float o = __int2float_rn(v);
          if (sa && sb) o = __fmul_rn(o, __fmul_rn(sa[m], sb[n]));
          if (side) {
            // acc_fp += x[m,c]*w[n,c] over outlier columns in ascending order, unfused
            float fp = 0.0f;
            for (int64_t c = 0; c < Kf; ++c)
              if (is_out[c]) fp = __fadd_rn(fp, __fmul_rn(xf[(int64_t)m * Kf + c], wf[n * Kf + c]));
            o = __fadd_rn(o, fp);
          }
          c_f32[(int64_t)m * N + n] = o;
        }
      }
    }
  }
}

// General exact INT8 GEMM (any M): 64x64 CTA tile, K staged 64 at a time, dp4a.
// Kept simple: the tensor-core INT8 path (tcgen05 kind::i8) serves the prefill
// shapes; this kernel covers everything the fast paths do not take.
constexpr int TB = 64, TK = 64;
__global__ void __launch_bounds__(256) gemm_i8_tiled_kernel(const int8_t* __restrict__ a, const int8_t* __restrict__ b,
                                                            int64_t M, int64_t N, int64_t K, int32_t* c_s32, float* c_f32,
                                                            const float* sa, const float* sb) {
  __shared__ __align__(16) int32_t As[TB][TK / 4 + 1];
  __shared__ __align__(16) int32_t Bs[TB][TK / 4 + 1];
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;     // 16 x 16 threads, 4x4 outputs each
  const int64_t m0 = (int64_t)blockIdx.y * TB, n0 = (int64_t)blockIdx.x * TB;
  int32_t acc[4][4] = {};
  for (int64_t k0 = 0; k0 < K; k0 += TK) {
    for (int i = threadIdx.x; i < TB * (TK / 4); i += 256) {
      int r = i / (TK / 4), kq = i % (TK / 4);
      int64_t k = k0 + kq * 4;
      int32_t va = 0, vb = 0;
      if (k < K) {                                            // K % 4 == 0: a word is all in or all out
        if (m0 + r < M) va = *reinterpret_cast<const int32_t*>(a + (m0 + r) * K + k);
        if (n0 + r < N) vb = *reinterpret_cast<const int32_t*>(b + (n0 + r) * K + k);
      }
      As[r][kq] = va;
      Bs[r][kq] = vb;
    }
    __syncthreads();
#pragma unroll
    for (int kq = 0; kq < TK / 4; ++kq) {
      int32_t av[4], bv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) { av[i] = As[ty * 4 + i][kq]; bv[i] = Bs[tx * 4 + i][kq]; }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = __dp4a(av[i], bv[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      int64_t m = m0 + ty * 4 + i, n = n0 + tx * 4 + j;
      if (m < M && n < N) {
        if (c_s32) c_s32[m * N + n] = acc[i][j];
        if (c_f32) {
          float o = __int2float_rn(acc[i][j]);
          if (sa && sb) o = __fmul_rn(o, __fmul_rn(sa[m], sb[n]));
          c_f32[m * N + n] = o;
        }
      }
    }
}

// Adds the fp32 outlier side term after a tiled GEMM (rare path: large M with outliers).
__global__ void outlier_side_kernel(const float* xf, const float* wf, const uint8_t* is_out, const int32_t* n_out,
                                    int64_t M, int64_t N, int64_t K, float* out) {
  if (*n_out <= 0) return;
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= M * N) return;
  int64_t m = i / N, n = i % N;
  float fp = 0.0f;
  for (int64_t c = 0; c < K; ++c)
    if (is_out[c]) fp = __fadd_rn(fp, __fmul_rn(xf[m * K + c], wf[n * K + c]));
  out[i] = __fadd_rn(out[i], fp);
}

int32_t launch_gemm_i8(b2q_handle h, const int8_t* a, const int8_t* b, int64_t M, int64_t N, int64_t K, int32_t* c_s32,
                       float* c_f32, const float* sa, const float* sb, const float* xf, const float* wf,
                       const uint8_t* is_out, const int32_t* n_out, int64_t Kf) {
  const bool aligned = ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b)) & 15) == 0 && K % 16 == 0;
  const size_t smem = (size_t)M * K;
  if (aligned && M <= 64 && smem <= 96 * 1024) {
    int grid = (int)ceil_div64(N, kThreads / 32);
    if (grid > h->sm_count * 8) grid = h->sm_count * 8;
    auto kern = M <= 8 ? gemm_i8_small_m_kernel<8> : gemm_i8_small_m_kernel<4>;
    if (smem > 48 * 1024)
      B2Q_CUDA(h, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    kern<<<grid, kThreads, smem, h->stream>>>(a, b, (int)M, N, K, c_s32, c_f32, sa, sb, xf, wf, is_out, n_out, Kf);
    B2Q_LAUNCH_CHECK(h, "gemm_i8_small_m_kernel");
    return B2Q_OK;
  }
  dim3 grid((unsigned)ceil_div64(N, TB), (unsigned)ceil_div64(M, TB));
  gemm_i8_tiled_kernel<<<grid, 256, 0, h->stream>>>(a, b, M, N, K, c_s32, c_f32, sa, sb);
  B2Q_LAUNCH_CHECK(h, "gemm_i8_tiled_kernel");
  if (c_f32 && n_out) {
    outlier_side_kernel<<<(int)ceil_div64(M * N, 256), 256, 0, h->stream>>>(xf, wf, is_out, n_out, M, N, Kf, c_f32);
    B2Q_LAUNCH_CHECK(h, "outlier_side_kernel");
  }
  return B2Q_OK;
}

}  // namespace

// tcgen05 kind::i8 path for prefill-sized INT8 GEMMs (defined in gemm_tc.cu);
// returns B2Q_ERR_UNSUPPORTED when the shape does not qualify.
int32_t b2q_gemm_i8_tc(b2q_handle h, const int8_t* a, const int8_t* b, int64_t M, int64_t N, int64_t K, int32_t* c_s32,
                       float* c_f32, const float* sa, const float* sb);

extern "C" {

int32_t b2q_gemm_i8(b2q_handle h, const int8_t* a, const int8_t* b, int64_t M, int64_t N, int64_t K, int32_t* c_s32,
                    float* c_f32, const float* scale_a, const float* scale_b) {
  B2Q_REQUIRE_HANDLE(h);
  if (M <= 0 || N <= 0 || K <= 0)
    B2Q_FAIL(h, B2Q_ERR_INVALID_DIMENSION, "INT8 GEMM dimensions must be non-zero: m=%lld, n=%lld, k=%lld", (long long)M, (long long)N, (long long)K);
  if (K % 4 != 0) B2Q_FAIL(h, B2Q_ERR_INVALID_DIMENSION, "INT8 GEMM K must be a multiple of 4, got k=%lld", (long long)K);
  if (!a || !b || (!c_s32 && !c_f32)) B2Q_FAIL(h, B2Q_ERR_INVALID_ARGUMENT, "gemm_i8: null pointer");
  if ((scale_a == nullptr) != (scale_b == nullptr)) B2Q_FAIL(h, B2Q_ERR_INVALID_ARGUMENT, "gemm_i8: give both scales or neither");
  if (((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b)) & 3) != 0)
    B2Q_FAIL(h, B2Q_ERR_INVALID_ARGUMENT, "gemm_i8: operands must be 4-byte aligned");
  if (M >= 128) {
    int32_t st = b2q_gemm_i8_tc(h, a, b, M, N, K, c_s32, c_f32, scale_a, scale_b);
    if (st != B2Q_ERR_UNSUPPORTED) return st;
    h->err[0] = 0;
  }
  return launch_gemm_i8(h, a, b, M, N, K, c_s32, c_f32, scale_a, scale_b, nullptr, nullptr, nullptr, nullptr, K);
}

int32_t b2q_llm_int8_linear_f32(b2q_handle h, const float* x, const float* w, int64_t samples, int64_t rows, int64_t cols,
                                float threshold, int row_wise, float* out, int8_t* wq, float* sw, int8_t* xq, float* sx,
                                int32_t* acc, int32_t* n_outliers) {
  B2Q_REQUIRE_HANDLE(h);
  if (samples <= 0 || rows <= 0 || cols <= 0) B2Q_FAIL(h, B2Q_ERR_EMPTY_INPUT, "LlmInt8::matmul: empty input");
  if (!isfinite(threshold) || threshold <= 0.0f)
    B2Q_FAIL(h, B2Q_ERR_INVALID_CONFIG, "LLM.int8 threshold must be finite and positive, got %g", (double)threshold);
  if (!x || !w || !out) B2Q_FAIL(h, B2Q_ERR_INVALID_ARGUMENT, "llm_int8_linear: null pointer");
  // Codes are kept with the row length padded to 16 so that every row starts 16-byte aligned; the padding is zero.
  // Caller-provided dumps are used in place when no padding is needed, otherwise filled by a strided copy.
  const int64_t ld = (cols + 15) & ~(int64_t)15;
  const bool padded = ld != cols;
  int8_t* wq_user = wq; int8_t* xq_user = xq;
  auto al = [](size_t v) { return (v + 255) & ~(size_t)255; };
  const size_t need_wq = (wq && !padded) ? 0 : (size_t)(rows * ld), need_xq = (xq && !padded) ? 0 : (size_t)(samples * ld);
  const size_t need_sw = sw ? 0 : sizeof(float) * (size_t)rows, need_sx = sx ? 0 : sizeof(float) * (size_t)samples;
  const size_t total = al(need_wq) + al(need_xq) + al(need_sw) + al(need_sx) + al((size_t)cols) + 256;
  uint8_t* p = nullptr;
  int32_t wst = b2q_workspace(h, total, (void**)&p);
  if (wst != B2Q_OK) return wst;
  if (need_wq) { wq = (int8_t*)p; p += al(need_wq); }
  if (need_xq) { xq = (int8_t*)p; p += al(need_xq); }
  if (!sw) { sw = (float*)p; p += al(need_sw); }
  if (!sx) { sx = (float*)p; p += al(need_sx); }
  uint8_t* is_out = p; p += al((size_t)cols);
  int32_t* n_out = (int32_t*)p;            // [0] count, [1] global absmax bits
  uint32_t* gmax = (uint32_t*)(n_out + 1);
  B2Q_CUDA(h, cudaMemsetAsync(n_out, 0, 8, h->stream));

  outlier_mask_kernel<<<(int)ceil_div64(cols, 256), 256, 0, h->stream>>>(x, samples, cols, threshold, is_out, n_out);
  int8_row_quant_kernel<<<(int)rows, kThreads, 0, h->stream>>>(w, cols, ld, is_out, nullptr, wq, sw);
  if (!row_wise) {
    int g = (int)ceil_div64(samples * cols, 256);
    if (g > h->sm_count * 8) g = h->sm_count * 8;
    masked_absmax_kernel<<<g, 256, 0, h->stream>>>(x, samples * cols, cols, is_out, gmax);
  }
  int8_row_quant_kernel<<<(int)samples, kThreads, 0, h->stream>>>(x, cols, ld, is_out, row_wise ? nullptr : gmax, xq, sx);
  B2Q_LAUNCH_CHECK(h, "llm_int8 quantize kernels");
  int32_t st = launch_gemm_i8(h, xq, wq, samples, rows, ld, acc, out, sx, sw, x, w, is_out, n_out, cols);
  if (padded && wq_user) B2Q_CUDA(h, cudaMemcpy2DAsync(wq_user, (size_t)cols, wq, (size_t)ld, (size_t)cols, (size_t)rows, cudaMemcpyDeviceToDevice, h->stream));
  if (padded && xq_user) B2Q_CUDA(h, cudaMemcpy2DAsync(xq_user, (size_t)cols, xq, (size_t)ld, (size_t)cols, (size_t)samples, cudaMemcpyDeviceToDevice, h->stream));
  if (n_outliers) B2Q_CUDA(h, cudaMemcpyAsync(n_outliers, n_out, sizeof(int32_t), cudaMemcpyDeviceToDevice, h->stream));
  return st;
}

}  // extern "C"
