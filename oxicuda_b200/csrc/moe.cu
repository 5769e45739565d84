// Mixture-of-experts plumbing on the quantized-linear path: token scatter into per-expert buffers, the
// weighted gather that combines the expert outputs, and the grouped FP8 GEMM over per-expert problems.
// Replaces ep_token_scatter / ep_token_gather (crates/oxicuda-dist-infer/src/ptx_kernels.rs:46-469),
// ExpertDispatcher::{scatter,gather} (crates/oxicuda-dist-infer/src/expert_parallel/dispatch.rs:99-219) and
// grouped_gemm (crates/oxicuda-blas/src/batched/grouped_gemm.rs:46-78).
#include "common.cuh"

int32_t b2q_validate_gemm_fp8(b2q_handle h, const uint8_t* a, const uint8_t* w, int64_t M, int64_t N, int64_t K, int fmt,
                              const float* scale_a, int ka, const float* scale_w, int kw, void* out, int out_type);

namespace {

// expert_buf[slot[i]] = in[token[i]] for every routed (token, expert) pair i; one warp per pair, 16-byte copies.
__global__ void __launch_bounds__(256) token_scatter_kernel(const uint4* __restrict__ in, const int32_t* __restrict__ token,
                                                            const int32_t* __restrict__ slot, int64_t pairs, int64_t row_vec,
                                                            uint4* __restrict__ out) {
  const int lane = threadIdx.x & 31;
  const int64_t warp = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
  const int64_t nwarps = (int64_t)gridDim.x * 8;
  for (int64_t i = warp; i < pairs; i += nwarps) {
    const uint4* src = in + (int64_t)token[i] * row_vec;
    uint4* dst = out + (int64_t)slot[i] * row_vec;
    for (int64_t v = lane; v < row_vec; v += 32) dst[v] = src[v];
  }
}

// out[t] = sum_j weight[t*k + j] * expert_out[slot[t*k + j]] in fp32, j ascending (the order of the routing plan),
// stored as bf16.  One warp per token.
__global__ void __launch_bounds__(256) token_gather_kernel(const __nv_bfloat16* __restrict__ expert_out, const int32_t* __restrict__ slot,
                                                           const float* __restrict__ weight, int64_t tokens, int top_k, int64_t hidden,
                                                           __nv_bfloat16* __restrict__ out) {
  const int lane = threadIdx.x & 31;
  const int64_t warp = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
  const int64_t nwarps = (int64_t)gridDim.x * 8;
  for (int64_t t = warp; t < tokens; t += nwarps) {
    for (int64_t c = (int64_t)lane * 2; c < hidden; c += 64) {
      float a0 = 0.0f, a1 = 0.0f;
      for (int j = 0; j < top_k; ++j) {
        const int32_t s = slot[t * top_k + j];
        if (s < 0) continue;                                  // pair routed to an expert of another rank
        const float wgt = weight[t * top_k + j];
        const __nv_bfloat162 v = *reinterpret_cast<const __nv_bfloat162*>(expert_out + (int64_t)s * hidden + c);
        a0 = __fadd_rn(a0, __fmul_rn(wgt, __low2float(v)));
        a1 = __fadd_rn(a1, __fmul_rn(wgt, __high2float(v)));
      }
      *reinterpret_cast<__nv_bfloat162*>(out + t * hidden + c) = __floats2bfloat162_rn(a0, a1);
    }
  }
}

}  // namespace

extern "C" {

int32_t b2q_ep_token_scatter(b2q_handle h, const void* in, const int32_t* token, const int32_t* slot, int64_t pairs,
                             int64_t row_bytes, void* expert_buf) {
  B2Q_REQUIRE_HANDLE(h);
  if (pairs == 0) return B2Q_OK;
  if (pairs < 0 || row_bytes <= 0 || !in || !token || !slot || !expert_buf) B2Q_FAIL(h, B2Q_ERR_INVALID_ARGUMENT, "ep_token_scatter: bad argument");
  if (row_bytes % 16 != 0 || ((reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(expert_buf)) & 15) != 0)
    B2Q_FAIL(h, B2Q_ERR_INVALID_ARGUMENT, "ep_token_scatter: rows must be 16-byte multiples and 16-byte aligned");
  int64_t g = ceil_div64(pairs, 8);
  if (g > (int64_t)h->sm_count * 16) g = (int64_t)h->sm_count * 16;
  token_scatter_kernel<<<(int)g, 256, 0, h->stream>>>((const uint4*)in, token, slot, pairs, row_bytes / 16, (uint4*)expert_buf);
  B2Q_LAUNCH_CHECK(h, "token_scatter_kernel");
  return B2Q_OK;
}

int32_t b2q_ep_token_gather_bf16(b2q_handle h, const void* expert_out, const int32_t* slot, const float* weight, int64_t tokens,
                                 int top_k, int64_t hidden, void* out) {
  B2Q_REQUIRE_HANDLE(h);
  if (tokens == 0) return B2Q_OK;
  if (tokens < 0 || top_k <= 0 || hidden <= 0 || !expert_out || !slot || !weight || !out)
    B2Q_FAIL(h, B2Q_ERR_INVALID_ARGUMENT, "ep_token_gather: bad argument");
  if (hidden % 2 != 0) B2Q_FAIL(h, B2Q_ERR_INVALID_DIMENSION, "ep_token_gather: hidden must be even, got %lld", (long long)hidden);
  int64_t g = ceil_div64(tokens, 8);
  if (g > (int64_t)h->sm_count * 16) g = (int64_t)h->sm_count * 16;
  token_gather_kernel<<<(int)g, 256, 0, h->stream>>>((const __nv_bfloat16*)expert_out, slot, weight, tokens, top_k, hidden,
                                                     (__nv_bfloat16*)out);
  B2Q_LAUNCH_CHECK(h, "token_gather_kernel");
  return B2Q_OK;
}

int32_t b2q_grouped_gemm_fp8(b2q_handle h, const b2q_gemm_fp8_problem* problems, int count, int fmt, int out_type) {
  B2Q_REQUIRE_HANDLE(h);
  if (count < 0 || (count > 0 && !problems)) B2Q_FAIL(h, B2Q_ERR_INVALID_ARGUMENT, "grouped_gemm_fp8: bad problem table");
  for (int i = 0; i < count; ++i) {
    const b2q_gemm_fp8_problem& p = problems[i];
    if (p.m == 0) continue;                                   // an expert that received no token
    int32_t st = b2q_gemm_fp8(h, p.a, p.w, p.m, p.n, p.k, fmt, p.scale_a, p.scale_a_kind, p.scale_w, p.scale_w_kind, p.out, out_type);
    if (st != B2Q_OK) return st;
  }
  return B2Q_OK;
}

}  // extern "C"
