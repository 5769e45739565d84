// FP8 (W8A8) decode GEMV, tokens <= 32 (HBM-bound): out[t, n] = (sum_k x[t,k] * w[n,k]) * sx[t] * sw[n]
// with x [tokens x K] and w [N x K] as E4M3/E5M2 codes.  The decode-sized branch of the FP8 GEMM dispatch
// (the reference's Skinny category, crates/oxicuda-blas/src/level3/gemm/dispatch.rs:493-534, and its
// level-2 gemv, crates/oxicuda-blas/src/level2/gemv.rs:63-143).
//
//   * a CTA owns 16 weight rows; its WK warps split K into contiguous slices, walked in 256-byte chunks;
//   * a lane loads 16 bytes of row g and 16 bytes of row g+8 per 64-wide step (a warp instruction covers
//     8 rows x 64 contiguous bytes); the codes ARE the A fragments of mma.sync.m16n8k32 (no conversion);
//   * activations are codes too: B fragments are 16-byte loads straight from global memory (the activation
//     matrix is a few KiB and stays in L1/L2), predicated off for token rows that do not exist;
//   * the next chunk's weights are prefetched into a second register set; fp32 accumulation in the MMA;
//   * one __syncthreads to add the WK partial sums, scales applied once per output.
#include "common.cuh"

namespace gemv8 {

constexpr int KC = 256;    // K bytes per chunk (4 steps of 64)

__device__ __forceinline__ uint4 ld_stream_v4(const void* p) {
  uint4 r;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(p));
  return r;
}
template <bool E5>
__device__ __forceinline__ void mma_fp8(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  if constexpr (E5) {
    asm("mma.sync.aligned.m16n8k32.row.col.f32.e5m2.e5m2.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
  } else {
    asm("mma.sync.aligned.m16n8k32.row.col.f32.e4m3.e4m3.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
  }
}

struct Chunk { uint4 wa[4], wb[4]; };

__device__ __forceinline__ void load_chunk(Chunk& r, const uint8_t* w0, const uint8_t* w1, int steps) {
#pragma unroll
  for (int s = 0; s < 4; ++s) {
    if (s < steps) {
      r.wa[s] = ld_stream_v4(w0 + s * 64);
      r.wb[s] = ld_stream_v4(w1 + s * 64);
    } else {
      r.wa[s] = make_uint4(0, 0, 0, 0);
      r.wb[s] = make_uint4(0, 0, 0, 0);
    }
  }
}

// xk: this lane's 16 bytes inside the chunk's first step of token row g (token tiles are 8 rows apart)
template <int MT, bool E5>
__device__ __forceinline__ void mul_chunk(const Chunk& r, const uint8_t* xk, int64_t K, int g, int tokens, int steps, float (&acc)[MT][4]) {
#pragma unroll
  for (int s = 0; s < 4; ++s) {
    if (s < steps) {
#pragma unroll
      for (int t = 0; t < MT; ++t) {
        uint4 xv = make_uint4(0, 0, 0, 0);
        if (t * 8 + g < tokens) xv = __ldg(reinterpret_cast<const uint4*>(xk + (int64_t)(t * 8) * K + s * 64));
        mma_fp8<E5>(acc[t], r.wa[s].x, r.wb[s].x, r.wa[s].y, r.wb[s].y, xv.x, xv.y);
        mma_fp8<E5>(acc[t], r.wa[s].z, r.wb[s].z, r.wa[s].w, r.wb[s].w, xv.z, xv.w);
      }
    }
  }
}

template <int MT, int WK, bool E5>
__global__ void __launch_bounds__(WK * 32) gemv_fp8_kernel(const uint8_t* __restrict__ x, const uint8_t* __restrict__ w, int tokens,
                                                           int64_t N, int64_t K, const float* __restrict__ sx, int sx_rows,
                                                           const float* __restrict__ sw, int sw_rows, void* out, int out_type) {
  constexpr int MPAD = 8 * MT;
  __shared__ float red[WK][16][MPAD];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, tig = lane & 3;
  const int64_t n0 = (int64_t)blockIdx.x * 16;
  const int64_t r0 = min(n0 + g, N - 1), r1 = min(n0 + g + 8, N - 1);

  const int total_steps = (int)(K >> 6);
  const int chunks_total = (total_steps + 3) >> 2;
  const int cpw = (chunks_total + WK - 1) / WK;
  int c = warp * cpw;
  const int c_end = min(c + cpw, chunks_total);

  const uint8_t* w0 = w + r0 * K + tig * 16 + (int64_t)c * KC;
  const uint8_t* w1 = w + r1 * K + tig * 16 + (int64_t)c * KC;
  const uint8_t* xk = x + (int64_t)min(g, tokens - 1) * K + tig * 16 + (int64_t)c * KC;

  float acc[MT][4];
#pragma unroll
  for (int t = 0; t < MT; ++t) { acc[t][0] = acc[t][1] = acc[t][2] = acc[t][3] = 0.0f; }

  Chunk A, B;
  if (c < c_end) load_chunk(A, w0, w1, min(4, total_steps - c * 4));
  while (c < c_end) {
    if (c + 1 < c_end) load_chunk(B, w0 + KC, w1 + KC, min(4, total_steps - (c + 1) * 4));
    mul_chunk<MT, E5>(A, xk, K, g, tokens, min(4, total_steps - c * 4), acc);
    ++c; w0 += KC; w1 += KC; xk += KC;
    if (c >= c_end) break;
    if (c + 1 < c_end) load_chunk(A, w0 + KC, w1 + KC, min(4, total_steps - (c + 1) * 4));
    mul_chunk<MT, E5>(B, xk, K, g, tokens, min(4, total_steps - c * 4), acc);
    ++c; w0 += KC; w1 += KC; xk += KC;
  }

  // acc[t][0],[1]: row g, tokens 8t + 2*tig, +1;  acc[t][2],[3]: row g+8
#pragma unroll
  for (int t = 0; t < MT; ++t) {
    red[warp][g][t * 8 + tig * 2 + 0] = acc[t][0];
    red[warp][g][t * 8 + tig * 2 + 1] = acc[t][1];
    red[warp][g + 8][t * 8 + tig * 2 + 0] = acc[t][2];
    red[warp][g + 8][t * 8 + tig * 2 + 1] = acc[t][3];
  }
  __syncthreads();
  for (int e = threadIdx.x; e < 16 * tokens; e += WK * 32) {
    const int tok = e >> 4, row = e & 15;                 // consecutive threads -> consecutive output rows
    float v = 0.0f;
#pragma unroll
    for (int q = 0; q < WK; ++q) v += red[q][row][tok];
    const int64_t n = n0 + row;
    if (n < N) {
      v *= (sx_rows ? sx[tok] : sx[0]) * (sw_rows ? sw[n] : sw[0]);
      if (out_type == B2Q_OUT_BF16) reinterpret_cast<__nv_bfloat16*>(out)[(int64_t)tok * N + n] = __float2bfloat16_rn(v);
      else reinterpret_cast<float*>(out)[(int64_t)tok * N + n] = v;
    }
  }
}

template <int MT, int WK>
int32_t launch(b2q_handle h, const uint8_t* x, const uint8_t* w, int tokens, int64_t N, int64_t K, int fmt, const float* sx,
               int sx_rows, const float* sw, int sw_rows, void* out, int out_type) {
  const unsigned grid = (unsigned)ceil_div64(N, 16);
  if (fmt == B2Q_FP8_E5M2)
    gemv_fp8_kernel<MT, WK, true><<<grid, WK * 32, 0, h->stream>>>(x, w, tokens, N, K, sx, sx_rows, sw, sw_rows, out, out_type);
  else
    gemv_fp8_kernel<MT, WK, false><<<grid, WK * 32, 0, h->stream>>>(x, w, tokens, N, K, sx, sx_rows, sw, sw_rows, out, out_type);
  B2Q_LAUNCH_CHECK(h, "gemv_fp8_kernel");
  return B2Q_OK;
}

}  // namespace gemv8

// Decode-sized FP8 GEMM (M <= 32, K % 64 == 0, 16-byte aligned operands); B2Q_ERR_UNSUPPORTED otherwise.
int32_t b2q_gemv_fp8_dispatch(b2q_handle h, const uint8_t* a, const uint8_t* w, int64_t M, int64_t N, int64_t K, int fmt,
                              const float* scale_a, int ka, const float* scale_w, int kw, void* out, int out_type) {
  if (M > 32 || K % 64 != 0 || ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(w)) & 15) != 0)
    return B2Q_ERR_UNSUPPORTED;
  const int t = (int)M;
  const bool deep = K >= 8192;
#define B2Q_GEMV8(MT) (deep ? gemv8::launch<MT, 8>(h, a, w, t, N, K, fmt, scale_a, ka, scale_w, kw, out, out_type) \
                            : gemv8::launch<MT, 4>(h, a, w, t, N, K, fmt, scale_a, ka, scale_w, kw, out, out_type))
  if (t <= 8) return B2Q_GEMV8(1);
  if (t <= 16) return B2Q_GEMV8(2);
  return B2Q_GEMV8(4);
#undef B2Q_GEMV8
}
