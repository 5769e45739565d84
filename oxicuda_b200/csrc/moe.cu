// Mixture-of-experts plumbing on the quantized-linear path: token scatter into per-expert buffers, the
// weighted gather that combines the expert outputs, and the grouped FP8 GEMM over per-expert problems.
// Replaces ep_token_scatter / ep_token_gather (crates/oxicuda-dist-infer/src/ptx_kernels.rs:46-469),
// ExpertDispatcher::{scatter,gather} (crates/oxicuda-dist-infer/src/expert_parallel/dispatch.rs:99-219) and
// grouped_gemm (crates/oxicuda-blas/src/batched/grouped_gemm.rs:46-78).
#include "common.cuh"

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


// TopKRouter::route (crates/oxicuda-dist-infer/src/expert_parallel/router.rs:94-140): per token the top_k experts by
// descending logit (a stable sort: equal logits keep index order) and the softmax of those k logits.  One thread per token.
constexpr int kMaxExperts = 64, kMaxTopK = 8;
__global__ void __launch_bounds__(128) moe_route_topk_kernel(const float* __restrict__ logits, int64_t tokens, int n_experts, int top_k,
                                                             int32_t* __restrict__ expert_idx, float* __restrict__ weight) {
  const int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= tokens) return;
  const float* lg = logits + t * n_experts;
  uint64_t taken = 0;
  float top[kMaxTopK];
  for (int j = 0; j < top_k; ++j) {
    int best = -1;
    float bv = 0.0f;
    for (int e = 0; e < n_experts; ++e) {
      if ((taken >> e) & 1ull) continue;
      const float v = lg[e];
      if (best < 0 || v > bv) { best = e; bv = v; }          // strict: the first of equal logits wins, as a stable descending sort gives
    }
    taken |= 1ull << best;
    top[j] = bv;
    expert_idx[t * top_k + j] = best;
  }
  float ex[kMaxTopK], sum = 0.0f;
  for (int j = 0; j < top_k; ++j) { ex[j] = expf(top[j] - top[0]); sum += ex[j]; }
  const float denom = sum > 0.0f ? sum : 1.0f;
  for (int j = 0; j < top_k; ++j) weight[t * top_k + j] = __fdiv_rn(ex[j], denom);
}

// Slots for the routed (token, expert) pairs of this rank's experts, without the host: one CTA counts the pairs per
// local expert, lays the experts out at row offsets padded to multiples of 256 (the tile height of the grouped GEMM)
// and hands every pair a row.  slot_of_pair is -1 for pairs served by another rank.  Rows inside an expert's range are
// handed out in arrival order; a pair's result does not depend on its row.
__global__ void __launch_bounds__(1024) moe_slot_kernel(const int32_t* __restrict__ expert_idx, int64_t pairs, int first_local, int n_local,
                                                        int32_t* __restrict__ counts, int32_t* __restrict__ offsets,
                                                        int32_t* __restrict__ slot_of_pair) {
  __shared__ int s_cnt[kMaxExperts], s_off[kMaxExperts + 1], s_cur[kMaxExperts];
  for (int e = threadIdx.x; e < kMaxExperts; e += blockDim.x) { s_cnt[e] = 0; s_cur[e] = 0; }
  __syncthreads();
  for (int64_t i = threadIdx.x; i < pairs; i += blockDim.x) {
    const int e = expert_idx[i] - first_local;
    if (e >= 0 && e < n_local) atomicAdd(&s_cnt[e], 1);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int off = 0;
    for (int e = 0; e < n_local; ++e) {
      s_off[e] = off;
      counts[e] = s_cnt[e];
      offsets[e] = off;
      off += (s_cnt[e] + 255) / 256 * 256;
    }
    s_off[n_local] = off;
    offsets[n_local] = off;
  }
  __syncthreads();
  for (int64_t i = threadIdx.x; i < pairs; i += blockDim.x) {
    const int e = expert_idx[i] - first_local;
    slot_of_pair[i] = (e >= 0 && e < n_local) ? s_off[e] + atomicAdd(&s_cur[e], 1) : -1;
  }
}

// expert_buf[slot_of_pair[i]] = x[i / top_k] for every pair with a slot; one warp per pair, 16-byte copies.
__global__ void __launch_bounds__(256) moe_scatter_kernel(const uint4* __restrict__ x, const int32_t* __restrict__ slot_of_pair, int64_t pairs,
                                                          int top_k, int64_t row_vec, uint4* __restrict__ out) {
  const int lane = threadIdx.x & 31;
  const int64_t warp = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
  const int64_t nwarps = (int64_t)gridDim.x * 8;
  for (int64_t i = warp; i < pairs; i += nwarps) {
    const int32_t sl = slot_of_pair[i];
    if (sl < 0) continue;
    const uint4* src = x + (i / top_k) * row_vec;
    uint4* dst = out + (int64_t)sl * row_vec;
    for (int64_t v = lane; v < row_vec; v += 32) dst[v] = src[v];
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

extern "C" {

int32_t b2q_moe_route_topk(b2q_handle h, const float* logits, int64_t tokens, int n_experts, int top_k, int32_t* expert_idx, float* weight) {
  B2Q_REQUIRE_HANDLE(h);
  if (tokens <= 0) return B2Q_OK;
  if (!logits || !expert_idx || !weight) B2Q_FAIL(h, B2Q_ERR_INVALID_ARGUMENT, "moe_route_topk: null operand");
  if (n_experts < 1 || n_experts > kMaxExperts) B2Q_FAIL(h, B2Q_ERR_UNSUPPORTED, "moe_route_topk: 1 to %d experts, got %d", kMaxExperts, n_experts);
  if (top_k < 1 || top_k > n_experts || top_k > kMaxTopK)
    B2Q_FAIL(h, B2Q_ERR_INVALID_ARGUMENT, "top_k %d must be in [1, %d]", top_k, n_experts < kMaxTopK ? n_experts : kMaxTopK);
  moe_route_topk_kernel<<<(unsigned)ceil_div64(tokens, 128), 128, 0, h->stream>>>(logits, tokens, n_experts, top_k, expert_idx, weight);
  B2Q_LAUNCH_CHECK(h, "moe_route_topk_kernel");
  return B2Q_OK;
}

int32_t b2q_moe_assign_slots(b2q_handle h, const int32_t* expert_idx, int64_t pairs, int first_local, int n_local, int32_t* counts,
                             int32_t* offsets, int32_t* slot_of_pair) {
  B2Q_REQUIRE_HANDLE(h);
  if (pairs <= 0 || n_local < 1 || n_local > kMaxExperts || !expert_idx || !counts || !offsets || !slot_of_pair)
    B2Q_FAIL(h, B2Q_ERR_INVALID_ARGUMENT, "moe_assign_slots: bad argument");
  moe_slot_kernel<<<1, 1024, 0, h->stream>>>(expert_idx, pairs, first_local, n_local, counts, offsets, slot_of_pair);
  B2Q_LAUNCH_CHECK(h, "moe_slot_kernel");
  return B2Q_OK;
}

int32_t b2q_moe_scatter(b2q_handle h, const void* x, const int32_t* slot_of_pair, int64_t pairs, int top_k, int64_t row_bytes, void* expert_buf) {
  B2Q_REQUIRE_HANDLE(h);
  if (pairs <= 0) return B2Q_OK;
  if (top_k < 1 || row_bytes <= 0 || !x || !slot_of_pair || !expert_buf) B2Q_FAIL(h, B2Q_ERR_INVALID_ARGUMENT, "moe_scatter: bad argument");
  if (row_bytes % 16 != 0 || ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(expert_buf)) & 15) != 0)
    B2Q_FAIL(h, B2Q_ERR_INVALID_ARGUMENT, "moe_scatter: rows must be 16-byte multiples and 16-byte aligned");
  int64_t g = ceil_div64(pairs, 8);
  if (g > (int64_t)h->sm_count * 16) g = (int64_t)h->sm_count * 16;
  moe_scatter_kernel<<<(int)g, 256, 0, h->stream>>>((const uint4*)x, slot_of_pair, pairs, top_k, row_bytes / 16, (uint4*)expert_buf);
  B2Q_LAUNCH_CHECK(h, "moe_scatter_kernel");
  return B2Q_OK;
}

}  // extern "C"
