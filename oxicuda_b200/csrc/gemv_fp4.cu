// Block-scaled FP4 (E2M1) weight-only decode GEMV, tokens <= 32 (HBM-bound):
//   out[t, n] = sum_k x[t, k] * decode(codes[n, k]) * scale[n, k / 32]
//
// Work decomposition
//   * a CTA owns R = 16 * WARPS consecutive weight rows and one K slice; a thread-block
//     cluster of `split_k` CTAs covers the whole K of those rows and reduces the
//     partial sums through distributed shared memory (no global scratch, no atomics);
//   * a warp owns 16 weight rows and walks K in steps of 128 (four scale blocks).  For
//     each block the four lanes of a quad load 4 bytes each of row g and of row g+8, so
//     one warp instruction covers 8 rows x 16 contiguous bytes and the four instructions
//     of a step cover 64 contiguous bytes per row (both 32-byte sectors fully used);
//   * codes are expanded in registers with cvt.rn.f16x2.e2m1x2 (one instruction per
//     byte, exact) and are directly the A fragments of mma.sync.m16n8k16: every MMA spans
//     16 codes of ONE scale block, so the block scale is applied to the fp32 result of
//     the two MMAs of a block (exact for f32 and for E8M0 scales alike);
//   * activations are converted bf16 -> f16 once per 512-wide K chunk and staged in
//     shared memory in fragment order, so B fragments are conflict-free 128-bit loads;
//   * fp32 accumulation; bf16 (RNE) or f32 store.
// f16 operands are used because E2M1 -> f16x2 is a single hardware conversion and every
// E2M1 value is exact in f16; activations beyond +-65504 saturate.
#include "common.cuh"
#include <cooperative_groups.h>
#include <stdlib.h>

namespace cg = cooperative_groups;

namespace gemv {

constexpr int KC = 512;   // K elements per staged activation chunk (4 steps of 128)

__device__ __forceinline__ uint32_t ld_stream_u32(const void* p) {
  uint32_t r;
  asm volatile("ld.global.nc.u32 %0, [%1];" : "=r"(r) : "l"(p));
  return r;
}

// Four bytes (eight E2M1 codes) -> four f16x2 registers; low nibble is the low half.
// (Plain asm, not volatile: these are pure functions, and the scheduler must be free to interleave the
// conversions, MMAs and FMAs of different scale blocks — in program order the chain cvt -> mma -> mma -> fma
// leaves the pipes idle.)
__device__ __forceinline__ void cvt_e2m1x8(uint32_t w, uint32_t (&h)[4]) {
  asm(
      "{\n\t.reg .b8 b0, b1, b2, b3;\n\t"
      "mov.b32 {b0, b1, b2, b3}, %4;\n\t"
      "cvt.rn.f16x2.e2m1x2 %0, b0;\n\t"
      "cvt.rn.f16x2.e2m1x2 %1, b1;\n\t"
      "cvt.rn.f16x2.e2m1x2 %2, b2;\n\t"
      "cvt.rn.f16x2.e2m1x2 %3, b3;\n\t}"
      : "=r"(h[0]), "=r"(h[1]), "=r"(h[2]), "=r"(h[3]) : "r"(w));
}
// d = a * b (+ 0): first MMA of a scale block
__device__ __forceinline__ void mma_f16_zero(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%10, %10, %10, %10};"
      : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.0f));
}
__device__ __forceinline__ void mma_f16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t bf16x2_to_f16x2_sat(uint32_t v) {
  float lo = __uint_as_float(v << 16), hi = __uint_as_float(v & 0xFFFF0000u);
  lo = fminf(fmaxf(lo, -65504.0f), 65504.0f);
  hi = fminf(fmaxf(hi, -65504.0f), 65504.0f);
  __half2 h = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}

// Scales of the four blocks of one 128-wide step of one row, kept as loaded (E8M0: one word,
// f32: four floats) and decoded at the point of use.
template <bool E8> struct Scales4;
template <> struct Scales4<true> {
  uint32_t w;
  __device__ __forceinline__ void load(const void* base, int64_t idx) {            // idx is a multiple of 4
    w = __ldg(reinterpret_cast<const uint32_t*>(reinterpret_cast<const uint8_t*>(base) + idx));
  }
  __device__ __forceinline__ void clear() { w = 0; }
  __device__ __forceinline__ float get(int j) const { return e8m0_to_f32_dev((w >> (8 * j)) & 0xFF); }
};
template <> struct Scales4<false> {
  float4 v;
  __device__ __forceinline__ void load(const void* base, int64_t idx) {
    v = __ldg(reinterpret_cast<const float4*>(reinterpret_cast<const float*>(base) + idx));
  }
  __device__ __forceinline__ void clear() { v = make_float4(0.f, 0.f, 0.f, 0.f); }
  __device__ __forceinline__ float get(int j) const { return j == 0 ? v.x : j == 1 ? v.y : j == 2 ? v.z : v.w; }
};

// MT: token tiles of 8 (tokens padded to 8*MT).  WARPS: warps per CTA (16 rows each).
template <int MT, int WARPS, bool E8>
__global__ void __launch_bounds__(WARPS * 32) gemv_fp4_kernel(const uint8_t* __restrict__ codes, const void* __restrict__ scales,
                                                              const __nv_bfloat16* __restrict__ x, int tokens, int64_t N, int64_t K,
                                                              void* out, int out_type, int split_k) {
  constexpr int MPAD = 8 * MT;
  constexpr int R = 16 * WARPS;
  constexpr int NT = WARPS * 32;
  extern __shared__ __align__(16) uint8_t smem[];        // activation chunk, later the partial sums
  uint4* xs = reinterpret_cast<uint4*>(smem);            // [block-of-32 (16 per chunk)][MPAD][quad lane 4] x 16 bytes
  float* red = reinterpret_cast<float*>(smem);           // [MPAD][R]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, tig = lane & 3;
  const int ks = blockIdx.x % split_k;
  const int64_t row_tile = blockIdx.x / split_k;
  const int64_t n0 = row_tile * R + warp * 16;
  // clamp so that loads stay in bounds; rows >= N are dropped at the store
  const int64_t r0 = min(n0 + g, N - 1), r1 = min(n0 + g + 8, N - 1);
  const int64_t kblocks = K >> 5;                        // scale blocks per row
  const uint8_t* w0 = codes + r0 * (K >> 1) + tig * 4;   // this lane's 4 bytes inside every 16-byte block
  const uint8_t* w1 = codes + r1 * (K >> 1) + tig * 4;

  const int chunks_total = (int)((K + KC - 1) / KC);
  const int cpc = (chunks_total + split_k - 1) / split_k;
  const int c_begin = ks * cpc, c_end = min(c_begin + cpc, chunks_total);

  float acc[MT][4];
#pragma unroll
  for (int t = 0; t < MT; ++t) { acc[t][0] = acc[t][1] = acc[t][2] = acc[t][3] = 0.0f; }

  for (int c = c_begin; c < c_end; ++c) {
    const int64_t k0 = (int64_t)c * KC;
    // ---- issue this chunk's weight and scale loads first (they are the long-latency HBM stream) ----
    uint32_t wa[4][4], wb[4][4];
    Scales4<E8> sa[4], sb[4];
#pragma unroll
    for (int s = 0; s < 4; ++s) {
      const int64_t k = k0 + s * 128;
      if (k < K) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          wa[s][j] = ld_stream_u32(w0 + ((k + j * 32) >> 1));
          wb[s][j] = ld_stream_u32(w1 + ((k + j * 32) >> 1));
        }
        sa[s].load(scales, r0 * kblocks + (k >> 5));
        sb[s].load(scales, r1 * kblocks + (k >> 5));
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j) { wa[s][j] = 0; wb[s][j] = 0; }
        sa[s].clear();
        sb[s].clear();
      }
    }
    // ---- stage activations of this chunk: bf16 -> f16, fragment order ----
    __syncthreads();                                     // previous chunk's readers are done
    for (int i = threadIdx.x; i < 64 * MPAD; i += NT) {
      const int ttig = i & 3, tok = (i >> 2) % MPAD, blk = i / (4 * MPAD);
      const int64_t k = k0 + blk * 32 + ttig * 8;
      uint4 v = make_uint4(0, 0, 0, 0);
      if (tok < tokens && k < K) v = __ldg(reinterpret_cast<const uint4*>(x + (int64_t)tok * K + k));
      uint4 h;
      h.x = bf16x2_to_f16x2_sat(v.x); h.y = bf16x2_to_f16x2_sat(v.y);
      h.z = bf16x2_to_f16x2_sat(v.z); h.w = bf16x2_to_f16x2_sat(v.w);
      xs[i] = h;                                         // == xs[(blk * MPAD + tok) * 4 + ttig]
    }
    __syncthreads();
    // ---- expand codes, multiply, scale in fp32 ----
#pragma unroll
    for (int s = 0; s < 4; ++s) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {                      // one scale block: 8 codes per lane and row, two MMA k-steps
        uint32_t ha[4], hb[4];
        cvt_e2m1x8(wa[s][j], ha);
        cvt_e2m1x8(wb[s][j], hb);
        const float fa = sa[s].get(j), fb = sb[s].get(j);
#pragma unroll
        for (int t = 0; t < MT; ++t) {
          const uint4 xv = xs[((s * 4 + j) * MPAD + (t * 8 + g)) * 4 + tig];
          float d[4];
          mma_f16_zero(d, ha[0], hb[0], ha[1], hb[1], xv.x, xv.y);
          mma_f16(d, ha[2], hb[2], ha[3], hb[3], xv.z, xv.w);
          acc[t][0] = fmaf(fa, d[0], acc[t][0]);
          acc[t][1] = fmaf(fa, d[1], acc[t][1]);
          acc[t][2] = fmaf(fb, d[2], acc[t][2]);
          acc[t][3] = fmaf(fb, d[3], acc[t][3]);
        }
      }
    }
  }

  // ---- partial sums to shared memory: red[token][row within the CTA] ----
  __syncthreads();
#pragma unroll
  for (int t = 0; t < MT; ++t) {
    const int tok = t * 8 + tig * 2;
    red[(tok + 0) * R + warp * 16 + g] = acc[t][0];
    red[(tok + 1) * R + warp * 16 + g] = acc[t][1];
    red[(tok + 0) * R + warp * 16 + g + 8] = acc[t][2];
    red[(tok + 1) * R + warp * 16 + g + 8] = acc[t][3];
  }
  cg::cluster_group cluster = cg::this_cluster();
  if (split_k > 1) cluster.sync(); else __syncthreads();
  // ---- each CTA of the cluster reduces and stores its share of the [MPAD x R] tile ----
  const int E = MPAD * R;
  const int per = (E + split_k - 1) / split_k;
  const int e_begin = ks * per, e_end = min(e_begin + per, E);
  for (int e = e_begin + threadIdx.x; e < e_end; e += NT) {
    float v = 0.0f;
    if (split_k > 1) {
      for (int pr = 0; pr < split_k; ++pr) v += cluster.map_shared_rank(red, pr)[e];
    } else {
      v = red[e];
    }
    const int tok = e / R;
    const int64_t n = row_tile * R + (e % R);
    if (tok < tokens && n < N) {
      if (out_type == B2Q_OUT_BF16) reinterpret_cast<__nv_bfloat16*>(out)[(int64_t)tok * N + n] = __float2bfloat16_rn(v);
      else reinterpret_cast<float*>(out)[(int64_t)tok * N + n] = v;
    }
  }
  if (split_k > 1) cluster.sync();                       // peers may still be reading this CTA's partials
}

template <int MT, int WARPS, bool E8>
int32_t launch_fmt(b2q_handle h, const uint8_t* codes, const void* scales, const void* x, int tokens, int64_t N, int64_t K,
                   void* out, int out_type) {
  constexpr int R = 16 * WARPS;
  const int64_t row_tiles = ceil_div64(N, R);
  const int chunks = (int)ceil_div64(K, KC);
  // K split = cluster size (<= 8, a divisor of the chunk count): the smallest one that gives about 1.5 CTAs
  // per SM, else the largest available.
  int split = 1;
  for (int s = 1; s <= 8 && s <= chunks; ++s) {
    if (chunks % s != 0) continue;
    split = s;
    if (row_tiles * s >= (3 * (int64_t)h->sm_count) / 2) break;
  }
  const size_t smem = (size_t)1024 * 8 * MT > (size_t)8 * MT * R * 4 ? (size_t)1024 * 8 * MT : (size_t)8 * MT * R * 4;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(row_tiles * split));
  cfg.blockDim = dim3(WARPS * 32);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = h->stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = (unsigned)split;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  B2Q_CUDA(h, cudaLaunchKernelEx(&cfg, gemv_fp4_kernel<MT, WARPS, E8>, codes, scales, (const __nv_bfloat16*)x, tokens, N, K, out,
                                 out_type, split));
  return B2Q_OK;
}

template <int MT, int WARPS>
int32_t launch(b2q_handle h, const uint8_t* codes, const void* scales, int scale_format, const void* x, int tokens, int64_t N,
               int64_t K, void* out, int out_type) {
  return scale_format == B2Q_SCALE_E8M0 ? launch_fmt<MT, WARPS, true>(h, codes, scales, x, tokens, N, K, out, out_type)
                                        : launch_fmt<MT, WARPS, false>(h, codes, scales, x, tokens, N, K, out, out_type);
}

// ---------------------------------------------------------------------------
// Decode kernel for tokens <= 8 (the bandwidth-bound regime).  The kernel is bound by instruction issue
// long before HBM, so the inner loop is kept to the conversions, two MMAs and four FMAs per scale block:
//   * a CTA owns 16 weight rows; its WK warps split K into contiguous slices of 512-wide chunks;
//   * a warp prefetches the codes and scales of its NEXT chunk into a second register set before it
//     multiplies the current one, so HBM loads stay in flight while the tensor core works;
//   * each warp stages only its own slice of the activations (warp-private shared memory, __syncwarp),
//     TOK = 1, 2, 4 or 8 token rows so that all index arithmetic is shifts;
//   * one __syncthreads at the end to add the WK partial sums.
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t bf16x2_to_f16x2_satfinite(uint32_t v) {
  uint32_t r;
  asm("cvt.rn.satfinite.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(__uint_as_float(v & 0xFFFF0000u)), "f"(__uint_as_float(v << 16)));
  return r;
}

// E8M0 byte j of a packed word -> 2^(b-127) as fp32 bits (b == 0, i.e. 2^-127, reads as 0)
__device__ __forceinline__ float e8m0_word_get(uint32_t w, int j) {
  return __uint_as_float(j == 3 ? ((w >> 1) & 0x7F800000u) : ((w << (23 - 8 * j)) & 0x7F800000u));
}

template <bool E8> struct StepScales;
template <> struct StepScales<true> {
  uint32_t w;
  __device__ __forceinline__ void load(const void* base, int64_t idx) {
    w = __ldg(reinterpret_cast<const uint32_t*>(reinterpret_cast<const uint8_t*>(base) + idx));
  }
  __device__ __forceinline__ void clear() { w = 0; }
  __device__ __forceinline__ float get(int j) const { return e8m0_word_get(w, j); }
};
template <> struct StepScales<false> {
  float4 v;
  __device__ __forceinline__ void load(const void* base, int64_t idx) {
    v = __ldg(reinterpret_cast<const float4*>(reinterpret_cast<const float*>(base) + idx));
  }
  __device__ __forceinline__ void clear() { v = make_float4(0.f, 0.f, 0.f, 0.f); }
  __device__ __forceinline__ float get(int j) const { return j == 0 ? v.x : j == 1 ? v.y : j == 2 ? v.z : v.w; }
};

template <bool E8> struct ChunkRegs {
  uint32_t wa[4][4], wb[4][4];
  StepScales<E8> sa[4], sb[4];
};

// w0/w1: this lane's byte inside the chunk's first block of row g / g+8; s0/s1: scale index of that block
template <bool E8>
__device__ __forceinline__ void load_chunk(ChunkRegs<E8>& r, const uint8_t* w0, const uint8_t* w1, const void* scales,
                                           int64_t s0, int64_t s1, int steps) {
#pragma unroll
  for (int s = 0; s < 4; ++s) {
    if (s < steps) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        r.wa[s][j] = ld_stream_u32(w0 + s * 64 + j * 16);
        r.wb[s][j] = ld_stream_u32(w1 + s * 64 + j * 16);
      }
      r.sa[s].load(scales, s0 + s * 4);
      r.sb[s].load(scales, s1 + s * 4);
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j) { r.wa[s][j] = 0; r.wb[s][j] = 0; }
      r.sa[s].clear();
      r.sb[s].clear();
    }
  }
}

template <bool E8>
__device__ __forceinline__ void mul_chunk(const ChunkRegs<E8>& r, const uint4* xs_lane, float (&acc)[4]) {
#pragma unroll
  for (int s = 0; s < 4; ++s) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      uint32_t ha[4], hb[4];
      cvt_e2m1x8(r.wa[s][j], ha);
      cvt_e2m1x8(r.wb[s][j], hb);
      const uint4 xv = xs_lane[(s * 4 + j) * 32];          // [block][8 token rows][4 quad lanes]
      float d[4];
      mma_f16_zero(d, ha[0], hb[0], ha[1], hb[1], xv.x, xv.y);
      mma_f16(d, ha[2], hb[2], ha[3], hb[3], xv.z, xv.w);
      const float fa = r.sa[s].get(j), fb = r.sb[s].get(j);
      acc[0] = fmaf(fa, d[0], acc[0]);
      acc[1] = fmaf(fa, d[1], acc[1]);
      acc[2] = fmaf(fb, d[2], acc[2]);
      acc[3] = fmaf(fb, d[3], acc[3]);
    }
  }
}

// Stages activations [tokens x 512] of one chunk into this warp's buffer (f16, fragment order).
// TOK (power of two >= tokens) rows are written; rows TOK..7 of the buffer stay zero.
template <int TOK>
__device__ __forceinline__ void stage_x_warp(uint4* xs, const __nv_bfloat16* xk, int tokens, int64_t K, int k_left, int lane) {
  __syncwarp();                                          // the previous chunk's fragment reads are done
#pragma unroll
  for (int i = 0; i < 2 * TOK; ++i) {
    const int p = lane + 32 * i;                         // 64 * TOK pieces of 8 activations
    const int ttig = p & 3, tok = (p >> 2) & (TOK - 1), blk = p / (4 * TOK);
    const int k = blk * 32 + ttig * 8;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (tok < tokens && k < k_left) v = __ldg(reinterpret_cast<const uint4*>(xk + (int64_t)tok * K + k));
    uint4 h;
    h.x = bf16x2_to_f16x2_satfinite(v.x); h.y = bf16x2_to_f16x2_satfinite(v.y);
    h.z = bf16x2_to_f16x2_satfinite(v.z); h.w = bf16x2_to_f16x2_satfinite(v.w);
    xs[(blk * 8 + tok) * 4 + ttig] = h;
  }
  __syncwarp();
}

template <bool E8, int WK, int TOK>
__global__ void __launch_bounds__(WK * 32, 512 / (WK * 32)) gemv_fp4_small_kernel(const uint8_t* __restrict__ codes, const void* __restrict__ scales,
                                                                 const __nv_bfloat16* __restrict__ x, int tokens, int64_t N, int64_t K,
                                                                 void* out, int out_type) {
  extern __shared__ __align__(16) uint8_t smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, tig = lane & 3;
  uint4* xs = reinterpret_cast<uint4*>(smem) + warp * 512;        // [16 blocks][8 tokens][4] x 16 bytes = 8 KiB per warp
  float* red = reinterpret_cast<float*>(smem);                    // [WK][16 rows][8 tokens], reused after the main loop

  const int64_t n0 = (int64_t)blockIdx.x * 16;
  const int64_t r0 = min(n0 + g, N - 1), r1 = min(n0 + g + 8, N - 1);
  const int64_t kblocks = K >> 5;

  const int chunks_total = (int)((K + KC - 1) / KC);
  const int cpw = (chunks_total + WK - 1) / WK;
  int c = warp * cpw;
  const int c_end = min(c + cpw, chunks_total);
  const int total_steps = (int)(K >> 7);                          // 128-wide steps in a row

  const uint8_t* w0 = codes + r0 * (K >> 1) + tig * 4 + (int64_t)c * (KC / 2);
  const uint8_t* w1 = codes + r1 * (K >> 1) + tig * 4 + (int64_t)c * (KC / 2);
  int64_t s0 = r0 * kblocks + (int64_t)c * (KC / 32), s1 = r1 * kblocks + (int64_t)c * (KC / 32);
  const __nv_bfloat16* xk = x + (int64_t)c * KC;

  ChunkRegs<E8> A, B;
  if (c < c_end) load_chunk<E8>(A, w0, w1, scales, s0, s1, min(4, total_steps - c * 4));
  // rows of the fragment buffer that belong to no token stay zero for the whole kernel
#pragma unroll
  for (int i = 0; i < 16; ++i) xs[lane + 32 * i] = make_uint4(0, 0, 0, 0);
  const uint4* xs_lane = xs + g * 4 + tig;

  float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
  while (c < c_end) {
    if (c + 1 < c_end) load_chunk<E8>(B, w0 + KC / 2, w1 + KC / 2, scales, s0 + KC / 32, s1 + KC / 32, min(4, total_steps - (c + 1) * 4));
    stage_x_warp<TOK>(xs, xk, tokens, K, (int)min((int64_t)KC, K - (int64_t)c * KC), lane);
    mul_chunk<E8>(A, xs_lane, acc);
    ++c; w0 += KC / 2; w1 += KC / 2; s0 += KC / 32; s1 += KC / 32; xk += KC;
    if (c >= c_end) break;
    if (c + 1 < c_end) load_chunk<E8>(A, w0 + KC / 2, w1 + KC / 2, scales, s0 + KC / 32, s1 + KC / 32, min(4, total_steps - (c + 1) * 4));
    stage_x_warp<TOK>(xs, xk, tokens, K, (int)min((int64_t)KC, K - (int64_t)c * KC), lane);
    mul_chunk<E8>(B, xs_lane, acc);
    ++c; w0 += KC / 2; w1 += KC / 2; s0 += KC / 32; s1 += KC / 32; xk += KC;
  }

  __syncthreads();                                       // every warp is done with its activation buffer
  // acc[0],acc[1]: row g, tokens 2*tig, 2*tig+1;  acc[2],acc[3]: row g+8
  red[(warp * 16 + g) * 8 + tig * 2 + 0] = acc[0];
  red[(warp * 16 + g) * 8 + tig * 2 + 1] = acc[1];
  red[(warp * 16 + g + 8) * 8 + tig * 2 + 0] = acc[2];
  red[(warp * 16 + g + 8) * 8 + tig * 2 + 1] = acc[3];
  __syncthreads();
  for (int e = threadIdx.x; e < 16 * tokens; e += WK * 32) {
    const int tok = e >> 4, row = e & 15;               // consecutive threads -> consecutive output rows
    float v = 0.0f;
#pragma unroll
    for (int w = 0; w < WK; ++w) v += red[(w * 16 + row) * 8 + tok];
    const int64_t n = n0 + row;
    if (n < N) {
      if (out_type == B2Q_OUT_BF16) reinterpret_cast<__nv_bfloat16*>(out)[(int64_t)tok * N + n] = __float2bfloat16_rn(v);
      else reinterpret_cast<float*>(out)[(int64_t)tok * N + n] = v;
    }
  }
}

template <bool E8, int WK, int TOK>
int32_t launch_small_t(b2q_handle h, const uint8_t* codes, const void* scales, const void* x, int tokens, int64_t N, int64_t K,
                       void* out, int out_type) {
  const unsigned grid = (unsigned)ceil_div64(N, 16);
  const size_t smem = (size_t)WK * 8192;
  if (smem > 48 * 1024) {
    B2Q_SMEM_ATTR(h, (gemv_fp4_small_kernel<E8, WK, TOK>), (int)smem);
  }
  gemv_fp4_small_kernel<E8, WK, TOK><<<grid, WK * 32, smem, h->stream>>>(codes, scales, (const __nv_bfloat16*)x, tokens, N, K, out, out_type);
  B2Q_LAUNCH_CHECK(h, "gemv_fp4_small_kernel");
  return B2Q_OK;
}

// ---------------------------------------------------------------------------
// E8M0 decode kernel for tokens <= 8: 128-bit weight loads.
// The exact kernel above needs four 4-byte loads per row and 128-wide step so that one MMA stays inside
// one scale block; each of those warp instructions touches 8 cache lines, and the L1 wavefront rate
// (measured 84 % of peak) bounds it.  With power-of-two scales the block scale can instead be multiplied
// into the f16 codes before the MMA without rounding (code * 2^e is exact in f16 for -23 <= e <= 13), so a
// lane may own a whole 32-code block: ONE 16-byte load per row and step, a quarter of the wavefronts.
// Exponents below -23 lose at most 2^-24 per code (flushed towards zero in f16).  An exponent above 13 would
// overflow f16: a warp that meets one in a 512-wide chunk computes that chunk with exact_chunk_e8 instead
// (fp32 scale, fp32 FMA, k ascending), so every legal E8M0 tensor gives the defined result.
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint4 ld_stream_v4(const void* p) {
  uint4 r;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(p));
  return r;
}
__device__ __forceinline__ uint32_t hmul2_u32(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}
// E8M0 byte -> 2^(b-127) as f16x2 (both halves); subnormal f16 below 2^-14, zero below 2^-24.
__device__ __forceinline__ uint32_t e8m0_to_h2(uint32_t b) {
  const int ee = (int)b - 112;                           // f16 exponent field
  const uint32_t h = ee > 0 ? ((uint32_t)min(ee, 30) << 10) : (ee > -10 ? (0x0400u >> (1 - ee)) : 0u);
  return h * 0x00010001u;
}

struct ChunkRegsE8 {
  uint4 wa[4], wb[4];      // one 32-code block per step for row g and row g+8
  uint4 sa, sb;            // the 16 scale bytes of the chunk for both rows
};

__device__ __forceinline__ void load_chunk_e8(ChunkRegsE8& r, const uint8_t* w0, const uint8_t* w1, const uint8_t* s0,
                                              const uint8_t* s1, int steps) {
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
  if (steps == 4 && ((reinterpret_cast<uintptr_t>(s0) | reinterpret_cast<uintptr_t>(s1)) & 15) == 0) {
    r.sa = __ldg(reinterpret_cast<const uint4*>(s0));
    r.sb = __ldg(reinterpret_cast<const uint4*>(s1));
  } else {                                               // ragged tail or K % 512 != 0: word loads stay aligned and inside the row
    // steps past the end of the row get scale 2^0 (their codes are zero), which keeps the range check quiet
    uint32_t a[4] = {0x7F7F7F7Fu, 0x7F7F7F7Fu, 0x7F7F7F7Fu, 0x7F7F7F7Fu}, b[4] = {0x7F7F7F7Fu, 0x7F7F7F7Fu, 0x7F7F7F7Fu, 0x7F7F7F7Fu};
    for (int s = 0; s < steps; ++s) {
      a[s] = __ldg(reinterpret_cast<const uint32_t*>(s0) + s);
      b[s] = __ldg(reinterpret_cast<const uint32_t*>(s1) + s);
    }
    r.sa = make_uint4(a[0], a[1], a[2], a[3]);
    r.sb = make_uint4(b[0], b[1], b[2], b[3]);
  }
}

// True when one of this lane's scale bytes of the chunk is an exponent above 13 (byte > 140).
__device__ __forceinline__ bool chunk_overflows_f16(const ChunkRegsE8& r, int tig) {
  const uint32_t w[8] = {r.sa.x, r.sa.y, r.sa.z, r.sa.w, r.sb.x, r.sb.y, r.sb.z, r.sb.w};
  bool bad = false;
#pragma unroll
  for (int i = 0; i < 8; ++i) bad |= ((w[i] >> (8 * tig)) & 0xFFu) > 140u;
  return bad;
}

// The defined arithmetic (dequantize_fp4, then an fp32 dot product with k ascending) for one chunk of `klen` K
// values starting at k0 and the four outputs a lane holds in one MMA accumulator: rows ra, rb x tokens t0, t0 + 1.
// Reads global memory directly; only runs for chunks that hold a block exponent f16 cannot carry.
__device__ __noinline__ void exact_chunk_e8(const uint8_t* __restrict__ codes, const uint8_t* __restrict__ scales,
                                            const __nv_bfloat16* __restrict__ x, int64_t K, int64_t ra, int64_t rb, int64_t k0,
                                            int klen, int t0, int tokens, float (&add)[4]) {
  for (int ri = 0; ri < 2; ++ri) {
    const int64_t row = ri ? rb : ra;
    const uint8_t* cw = codes + row * (K >> 1) + (k0 >> 1);
    const uint8_t* sc = scales + row * (K >> 5) + (k0 >> 5);
    float s0 = 0.0f, s1 = 0.0f;
    for (int b = 0; b < (klen >> 5); ++b) {
      const float scale = e8m0_to_f32_dev(sc[b]);
      for (int i = 0; i < 16; ++i) {
        const uint32_t byte = cw[b * 16 + i];
        const float wl = e2m1_decode_dev(byte & 15u) * scale, wh = e2m1_decode_dev(byte >> 4) * scale;
        const int64_t k = k0 + b * 32 + 2 * i;
        if (t0 < tokens) {
          s0 = fmaf(wl, __bfloat162float(x[(int64_t)t0 * K + k]), s0);
          s0 = fmaf(wh, __bfloat162float(x[(int64_t)t0 * K + k + 1]), s0);
        }
        if (t0 + 1 < tokens) {
          s1 = fmaf(wl, __bfloat162float(x[(int64_t)(t0 + 1) * K + k]), s1);
          s1 = fmaf(wh, __bfloat162float(x[(int64_t)(t0 + 1) * K + k + 1]), s1);
        }
      }
    }
    add[2 * ri] += s0;
    add[2 * ri + 1] += s1;
  }
}

__device__ __forceinline__ void mul_chunk_e8(const ChunkRegsE8& r, const uint4* xs_lane, int tig, float (&acc0)[4],
                                             float (&acc1)[4]) {
  const uint32_t saw[4] = {r.sa.x, r.sa.y, r.sa.z, r.sa.w};
  const uint32_t sbw[4] = {r.sb.x, r.sb.y, r.sb.z, r.sb.w};
#pragma unroll
  for (int s = 0; s < 4; ++s) {
    const uint32_t ha2 = e8m0_to_h2((saw[s] >> (8 * tig)) & 0xFFu);
    const uint32_t hb2 = e8m0_to_h2((sbw[s] >> (8 * tig)) & 0xFFu);
    const uint32_t wav[4] = {r.wa[s].x, r.wa[s].y, r.wa[s].z, r.wa[s].w};
    const uint32_t wbv[4] = {r.wb[s].x, r.wb[s].y, r.wb[s].z, r.wb[s].w};
#pragma unroll
    for (int jj = 0; jj < 4; ++jj) {                     // 8 codes per row: two MMA k-steps
      uint32_t ha[4], hb[4];
      cvt_e2m1x8(wav[jj], ha);
      cvt_e2m1x8(wbv[jj], hb);
#pragma unroll
      for (int i = 0; i < 4; ++i) { ha[i] = hmul2_u32(ha[i], ha2); hb[i] = hmul2_u32(hb[i], hb2); }
      const uint4 xv = xs_lane[(s * 4 + jj) * 32];        // [step][jj][8 token rows][4 quad lanes]
      mma_f16(acc0, ha[0], hb[0], ha[1], hb[1], xv.x, xv.y);
      mma_f16(acc1, ha[2], hb[2], ha[3], hb[3], xv.z, xv.w);
    }
  }
}

// Activations of one chunk for the block-per-lane mapping: piece (step, jj, token, quad lane) holds
// x[token][step*128 + lane*32 + jj*8 .. +8).
template <int TOK>
__device__ __forceinline__ void stage_x_warp_e8(uint4* xs, const __nv_bfloat16* xk, int tokens, int64_t K, int k_left, int lane) {
  __syncwarp();
#pragma unroll
  for (int i = 0; i < 2 * TOK; ++i) {
    const int p = lane + 32 * i;
    const int ttig = p & 3, tok = (p >> 2) & (TOK - 1), sjj = p / (4 * TOK);
    const int k = (sjj >> 2) * 128 + ttig * 32 + (sjj & 3) * 8;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (tok < tokens && k < k_left) v = __ldg(reinterpret_cast<const uint4*>(xk + (int64_t)tok * K + k));
    uint4 h;
    h.x = bf16x2_to_f16x2_satfinite(v.x); h.y = bf16x2_to_f16x2_satfinite(v.y);
    h.z = bf16x2_to_f16x2_satfinite(v.z); h.w = bf16x2_to_f16x2_satfinite(v.w);
    xs[(sjj * 8 + tok) * 4 + ttig] = h;
  }
  __syncwarp();
}

template <int WK, int TOK>
__global__ void __launch_bounds__(WK * 32, 512 / (WK * 32)) gemv_fp4_e8_kernel(const uint8_t* __restrict__ codes, const uint8_t* __restrict__ scales,
                                                                               const __nv_bfloat16* __restrict__ x, int tokens, int64_t N, int64_t K,
                                                                               void* out, int out_type, int32_t* status) {
  extern __shared__ __align__(16) uint8_t smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, tig = lane & 3;
  uint4* xs = reinterpret_cast<uint4*>(smem) + warp * 512;
  float* red = reinterpret_cast<float*>(smem);

  const int64_t n0 = (int64_t)blockIdx.x * 16;
  const int64_t r0 = min(n0 + g, N - 1), r1 = min(n0 + g + 8, N - 1);
  const int64_t kblocks = K >> 5;
  const int chunks_total = (int)((K + KC - 1) / KC);
  const int cpw = (chunks_total + WK - 1) / WK;
  int c = warp * cpw;
  const int c_end = min(c + cpw, chunks_total);
  const int total_steps = (int)(K >> 7);

  const uint8_t* w0 = codes + r0 * (K >> 1) + tig * 16 + (int64_t)c * (KC / 2);     // this lane's block inside each step
  const uint8_t* w1 = codes + r1 * (K >> 1) + tig * 16 + (int64_t)c * (KC / 2);
  const uint8_t* s0 = scales + r0 * kblocks + (int64_t)c * (KC / 32);
  const uint8_t* s1 = scales + r1 * kblocks + (int64_t)c * (KC / 32);
  const __nv_bfloat16* xk = x + (int64_t)c * KC;

  ChunkRegsE8 A, B;
  if (c < c_end) load_chunk_e8(A, w0, w1, s0, s1, min(4, total_steps - c * 4));
#pragma unroll
  for (int i = 0; i < 16; ++i) xs[lane + 32 * i] = make_uint4(0, 0, 0, 0);
  const uint4* xs_lane = xs + g * 4 + tig;

  float acc0[4] = {0.0f, 0.0f, 0.0f, 0.0f}, acc1[4] = {0.0f, 0.0f, 0.0f, 0.0f};
  auto consume = [&](const ChunkRegsE8& R) {
    const int klen = (int)min((int64_t)KC, K - (int64_t)c * KC);
    if (__any_sync(0xFFFFFFFFu, chunk_overflows_f16(R, tig))) {      // warp-uniform; never taken for ordinary weights
      exact_chunk_e8(codes, scales, x, K, r0, r1, (int64_t)c * KC, klen, 2 * tig, tokens, acc0);
    } else {
      stage_x_warp_e8<TOK>(xs, xk, tokens, K, klen, lane);
      mul_chunk_e8(R, xs_lane, tig, acc0, acc1);
    }
    ++c; w0 += KC / 2; w1 += KC / 2; s0 += KC / 32; s1 += KC / 32; xk += KC;
  };
  while (c < c_end) {
    if (c + 1 < c_end) load_chunk_e8(B, w0 + KC / 2, w1 + KC / 2, s0 + KC / 32, s1 + KC / 32, min(4, total_steps - (c + 1) * 4));
    consume(A);
    if (c >= c_end) break;
    if (c + 1 < c_end) load_chunk_e8(A, w0 + KC / 2, w1 + KC / 2, s0 + KC / 32, s1 + KC / 32, min(4, total_steps - (c + 1) * 4));
    consume(B);
  }

  __syncthreads();
  red[(warp * 16 + g) * 8 + tig * 2 + 0] = acc0[0] + acc1[0];
  red[(warp * 16 + g) * 8 + tig * 2 + 1] = acc0[1] + acc1[1];
  red[(warp * 16 + g + 8) * 8 + tig * 2 + 0] = acc0[2] + acc1[2];
  red[(warp * 16 + g + 8) * 8 + tig * 2 + 1] = acc0[3] + acc1[3];
  __syncthreads();
  for (int e = threadIdx.x; e < 16 * tokens; e += WK * 32) {
    const int tok = e >> 4, row = e & 15;
    float v = 0.0f;
#pragma unroll
    for (int w = 0; w < WK; ++w) v += red[(w * 16 + row) * 8 + tok];
    const int64_t n = n0 + row;
    if (n < N) {
      if (out_type == B2Q_OUT_BF16) reinterpret_cast<__nv_bfloat16*>(out)[(int64_t)tok * N + n] = __float2bfloat16_rn(v);
      else reinterpret_cast<float*>(out)[(int64_t)tok * N + n] = v;
    }
  }
}

template <int WK, int TOK>
int32_t launch_e8_t(b2q_handle h, const uint8_t* codes, const void* scales, const void* x, int tokens, int64_t N, int64_t K,
                    void* out, int out_type) {
  const unsigned grid = (unsigned)ceil_div64(N, 16);
  const size_t smem = (size_t)WK * 8192;
  if (smem > 48 * 1024) {
    B2Q_SMEM_ATTR(h, (gemv_fp4_e8_kernel<WK, TOK>), (int)smem);
  }
  gemv_fp4_e8_kernel<WK, TOK><<<grid, WK * 32, smem, h->stream>>>(codes, (const uint8_t*)scales, (const __nv_bfloat16*)x, tokens, N, K,
                                                                   out, out_type, h->d_status);
  B2Q_LAUNCH_CHECK(h, "gemv_fp4_e8_kernel");
  return B2Q_OK;
}

template <int WK>
int32_t launch_e8(b2q_handle h, const uint8_t* codes, const void* scales, const void* x, int tokens, int64_t N, int64_t K, void* out,
                  int out_type) {
  return tokens == 1 ? launch_e8_t<WK, 1>(h, codes, scales, x, tokens, N, K, out, out_type)
       : tokens == 2 ? launch_e8_t<WK, 2>(h, codes, scales, x, tokens, N, K, out, out_type)
       : tokens <= 4 ? launch_e8_t<WK, 4>(h, codes, scales, x, tokens, N, K, out, out_type)
                     : launch_e8_t<WK, 8>(h, codes, scales, x, tokens, N, K, out, out_type);
}

// ---------------------------------------------------------------------------
// E8M0 kernel for 9..32 tokens: the 128-bit-load inner loop above over MT token tiles.  The activation
// chunk (8*MT tokens x 512 K values as f16) is too large to stage per warp, so the CTA's WARPS warps own
// 16 rows each and share one staged chunk; K is split across the CTAs of a cluster and the partial sums
// are added through distributed shared memory, as in gemv_fp4_kernel.
// ---------------------------------------------------------------------------
template <int MT>
__device__ __forceinline__ void mul_chunk_e8c(const ChunkRegsE8& r, const uint4* xs_lane, int tig, float (&acc0)[MT][4],
                                              float (&acc1)[MT][4]) {
  constexpr int MPAD = 8 * MT;
  const uint32_t saw[4] = {r.sa.x, r.sa.y, r.sa.z, r.sa.w};
  const uint32_t sbw[4] = {r.sb.x, r.sb.y, r.sb.z, r.sb.w};
#pragma unroll
  for (int s = 0; s < 4; ++s) {
    const uint32_t ha2 = e8m0_to_h2((saw[s] >> (8 * tig)) & 0xFFu);
    const uint32_t hb2 = e8m0_to_h2((sbw[s] >> (8 * tig)) & 0xFFu);
    const uint32_t wav[4] = {r.wa[s].x, r.wa[s].y, r.wa[s].z, r.wa[s].w};
    const uint32_t wbv[4] = {r.wb[s].x, r.wb[s].y, r.wb[s].z, r.wb[s].w};
#pragma unroll
    for (int jj = 0; jj < 4; ++jj) {
      uint32_t ha[4], hb[4];
      cvt_e2m1x8(wav[jj], ha);
      cvt_e2m1x8(wbv[jj], hb);
#pragma unroll
      for (int i = 0; i < 4; ++i) { ha[i] = hmul2_u32(ha[i], ha2); hb[i] = hmul2_u32(hb[i], hb2); }
#pragma unroll
      for (int t = 0; t < MT; ++t) {
        const uint4 xv = xs_lane[((s * 4 + jj) * MPAD + t * 8) * 4];   // [step][jj][token][quad lane]
        mma_f16(acc0[t], ha[0], hb[0], ha[1], hb[1], xv.x, xv.y);
        mma_f16(acc1[t], ha[2], hb[2], ha[3], hb[3], xv.z, xv.w);
      }
    }
  }
}

template <int MT, int WARPS, bool DB>
__global__ void __launch_bounds__(WARPS * 32, DB ? 1 : 512 / (WARPS * 32)) gemv_fp4_e8c_kernel(const uint8_t* __restrict__ codes, const uint8_t* __restrict__ scales,
                                                                  const __nv_bfloat16* __restrict__ x, int tokens, int64_t N, int64_t K,
                                                                  void* out, int out_type, int split_k, int32_t* status) {
  constexpr int MPAD = 8 * MT;
  constexpr int R = 16 * WARPS;
  constexpr int NT = WARPS * 32;
  extern __shared__ __align__(16) uint8_t smem[];        // activation chunk, later the partial sums
  uint4* xs = reinterpret_cast<uint4*>(smem);            // [step 4][jj 4][MPAD][quad lane 4] x 16 bytes
  float* red = reinterpret_cast<float*>(smem);           // [MPAD][R]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, tig = lane & 3;
  const int ks = blockIdx.x % split_k;
  const int64_t row_tile = blockIdx.x / split_k;
  const int64_t n0 = row_tile * R + warp * 16;
  const int64_t r0 = min(n0 + g, N - 1), r1 = min(n0 + g + 8, N - 1);
  const int64_t kblocks = K >> 5;
  const int chunks_total = (int)((K + KC - 1) / KC);
  const int cpc = (chunks_total + split_k - 1) / split_k;
  int c = ks * cpc;
  const int c_end = min(c + cpc, chunks_total);
  const int total_steps = (int)(K >> 7);

  const uint8_t* w0 = codes + r0 * (K >> 1) + tig * 16 + (int64_t)c * (KC / 2);
  const uint8_t* w1 = codes + r1 * (K >> 1) + tig * 16 + (int64_t)c * (KC / 2);
  const uint8_t* s0 = scales + r0 * kblocks + (int64_t)c * (KC / 32);
  const uint8_t* s1 = scales + r1 * kblocks + (int64_t)c * (KC / 32);
  const uint4* xs_lane = xs + g * 4 + tig;

  float acc0[MT][4], acc1[MT][4];
#pragma unroll
  for (int t = 0; t < MT; ++t) {
#pragma unroll
    for (int i = 0; i < 4; ++i) { acc0[t][i] = 0.0f; acc1[t][i] = 0.0f; }
  }
  // one chunk of this warp's rows: tensor-core path, or the exact fp32 statement when a block exponent exceeds f16
  auto consume = [&](const ChunkRegsE8& R, int cc) {
    if (__any_sync(0xFFFFFFFFu, chunk_overflows_f16(R, tig))) {
      const int klen = (int)min((int64_t)KC, K - (int64_t)cc * KC);
#pragma unroll
      for (int t = 0; t < MT; ++t) exact_chunk_e8(codes, scales, x, K, r0, r1, (int64_t)cc * KC, klen, t * 8 + 2 * tig, tokens, acc0[t]);
    } else {
      mul_chunk_e8c<MT>(R, xs_lane, tig, acc0, acc1);
    }
  };

  // activations of chunk cc for the whole CTA: piece (step, jj, token, quad lane) = x[token][step*128 + lane*32 + jj*8 .. +8)
  auto stage = [&](int cc) {
    const int64_t k0 = (int64_t)cc * KC;
    __syncthreads();                                     // the previous chunk's readers are done
    for (int i = threadIdx.x; i < 64 * MPAD; i += NT) {
      const int ttig = i & 3, tok = (i >> 2) % MPAD, sjj = i / (4 * MPAD);
      const int64_t k = k0 + (sjj >> 2) * 128 + ttig * 32 + (sjj & 3) * 8;
      uint4 v = make_uint4(0, 0, 0, 0);
      if (tok < tokens && k < K) v = __ldg(reinterpret_cast<const uint4*>(x + (int64_t)tok * K + k));
      uint4 hv;
      hv.x = bf16x2_to_f16x2_satfinite(v.x); hv.y = bf16x2_to_f16x2_satfinite(v.y);
      hv.z = bf16x2_to_f16x2_satfinite(v.z); hv.w = bf16x2_to_f16x2_satfinite(v.w);
      xs[i] = hv;                                        // == xs[(sjj * MPAD + tok) * 4 + ttig]
    }
    __syncthreads();
  };

  // every warp of the CTA walks the same chunks, so the barriers inside stage() are uniform
  if constexpr (DB) {                                    // next chunk's weights in a second register set; one CTA per SM
    ChunkRegsE8 A, B;
    if (c < c_end) load_chunk_e8(A, w0, w1, s0, s1, min(4, total_steps - c * 4));
    while (c < c_end) {
      if (c + 1 < c_end) load_chunk_e8(B, w0 + KC / 2, w1 + KC / 2, s0 + KC / 32, s1 + KC / 32, min(4, total_steps - (c + 1) * 4));
      stage(c);
      consume(A, c);
      ++c; w0 += KC / 2; w1 += KC / 2; s0 += KC / 32; s1 += KC / 32;
      if (c >= c_end) break;
      if (c + 1 < c_end) load_chunk_e8(A, w0 + KC / 2, w1 + KC / 2, s0 + KC / 32, s1 + KC / 32, min(4, total_steps - (c + 1) * 4));
      stage(c);
      consume(B, c);
      ++c; w0 += KC / 2; w1 += KC / 2; s0 += KC / 32; s1 += KC / 32;
    }
  } else {                                               // one register set, two CTAs per SM hide the load latency
    for (; c < c_end; ++c) {
      ChunkRegsE8 A;
      load_chunk_e8(A, w0, w1, s0, s1, min(4, total_steps - c * 4));
      stage(c);
      consume(A, c);
      w0 += KC / 2; w1 += KC / 2; s0 += KC / 32; s1 += KC / 32;
    }
  }

  // ---- partial sums to shared memory: red[token][row within the CTA] ----
  __syncthreads();
#pragma unroll
  for (int t = 0; t < MT; ++t) {
    const int tok = t * 8 + tig * 2;
    red[(tok + 0) * R + warp * 16 + g] = acc0[t][0] + acc1[t][0];
    red[(tok + 1) * R + warp * 16 + g] = acc0[t][1] + acc1[t][1];
    red[(tok + 0) * R + warp * 16 + g + 8] = acc0[t][2] + acc1[t][2];
    red[(tok + 1) * R + warp * 16 + g + 8] = acc0[t][3] + acc1[t][3];
  }
  cg::cluster_group cluster = cg::this_cluster();
  if (split_k > 1) cluster.sync(); else __syncthreads();
  const int E = MPAD * R;
  const int per = (E + split_k - 1) / split_k;
  const int e_begin = ks * per, e_end = min(e_begin + per, E);
  for (int e = e_begin + threadIdx.x; e < e_end; e += NT) {
    float v = 0.0f;
    if (split_k > 1) {
      for (int pr = 0; pr < split_k; ++pr) v += cluster.map_shared_rank(red, pr)[e];
    } else {
      v = red[e];
    }
    const int tok = e / R;
    const int64_t n = row_tile * R + (e % R);
    if (tok < tokens && n < N) {
      if (out_type == B2Q_OUT_BF16) reinterpret_cast<__nv_bfloat16*>(out)[(int64_t)tok * N + n] = __float2bfloat16_rn(v);
      else reinterpret_cast<float*>(out)[(int64_t)tok * N + n] = v;
    }
  }
  if (split_k > 1) cluster.sync();                       // peers may still be reading this CTA's partials
}

template <int MT, int WARPS, bool DB>
int32_t launch_e8c_t(b2q_handle h, const uint8_t* codes, const void* scales, const void* x, int tokens, int64_t N, int64_t K,
                   void* out, int out_type) {
  constexpr int R = 16 * WARPS;
  const int64_t row_tiles = ceil_div64(N, R);
  const int chunks = (int)ceil_div64(K, KC);
  int split = 1;                                         // cluster size: smallest divisor of the chunk count giving ~2 CTAs per SM
  for (int s = 1; s <= 8 && s <= chunks; ++s) {
    if (chunks % s != 0) continue;
    split = s;
    if (row_tiles * s >= 2 * (int64_t)h->sm_count) break;
  }
  const size_t smem = (size_t)1024 * 8 * MT > (size_t)8 * MT * R * 4 ? (size_t)1024 * 8 * MT : (size_t)8 * MT * R * 4;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(row_tiles * split));
  cfg.blockDim = dim3(WARPS * 32);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = h->stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = (unsigned)split;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  B2Q_CUDA(h, cudaLaunchKernelEx(&cfg, gemv_fp4_e8c_kernel<MT, WARPS, DB>, codes, (const uint8_t*)scales, (const __nv_bfloat16*)x, tokens,
                                 N, K, out, out_type, split, h->d_status));
  return B2Q_OK;
}

template <int MT, int WARPS>
int32_t launch_e8c(b2q_handle h, const uint8_t* codes, const void* scales, const void* x, int tokens, int64_t N, int64_t K,
                   void* out, int out_type) {
  if (h->sw.e8c_db == 1)                                // experiment switch: double-buffered weights, one CTA per SM
    return launch_e8c_t<MT, WARPS, true>(h, codes, scales, x, tokens, N, K, out, out_type);
  return launch_e8c_t<MT, WARPS, false>(h, codes, scales, x, tokens, N, K, out, out_type);
}

template <int WK>
int32_t launch_small(b2q_handle h, const uint8_t* codes, const void* scales, int scale_format, const void* x, int tokens, int64_t N,
                     int64_t K, void* out, int out_type) {
#define B2Q_SMALL(E8, TOK) launch_small_t<E8, WK, TOK>(h, codes, scales, x, tokens, N, K, out, out_type)
  if (scale_format == B2Q_SCALE_E8M0)
    return tokens == 1 ? B2Q_SMALL(true, 1) : tokens == 2 ? B2Q_SMALL(true, 2) : tokens <= 4 ? B2Q_SMALL(true, 4) : B2Q_SMALL(true, 8);
  return tokens == 1 ? B2Q_SMALL(false, 1) : tokens == 2 ? B2Q_SMALL(false, 2) : tokens <= 4 ? B2Q_SMALL(false, 4) : B2Q_SMALL(false, 8);
#undef B2Q_SMALL
}

}  // namespace gemv

int32_t b2q_gemv_fp4_mx_dispatch(b2q_handle h, const uint8_t* codes, const void* scales, const void* x, int tokens, int64_t N, int64_t K,
                                 void* out, int out_type);
int32_t b2q_gemv_fp4_mxf4_dispatch(b2q_handle h, const uint8_t* codes, const void* scales, const void* x, int tokens, int64_t N, int64_t K,
                                   void* out, int out_type);

extern "C" int32_t b2q_gemv_fp4_wo(b2q_handle h, const uint8_t* codes, const void* scales, int scale_format, int block,
                                   const void* x_bf16, int64_t tokens, int64_t N, int64_t K, void* out, int out_type) {
  B2Q_REQUIRE_HANDLE(h);
  if (tokens <= 0 || N <= 0 || K <= 0)
    B2Q_FAIL(h, B2Q_ERR_INVALID_DIMENSION, "FP4 GEMM dimensions must be non-zero: m=%lld, n=%lld, k=%lld", (long long)N, (long long)tokens, (long long)K);
  if (K % 2 != 0) B2Q_FAIL(h, B2Q_ERR_INVALID_DIMENSION, "FP4 GEMM K dimension must be even for packing, got k=%lld", (long long)K);
  if (block != 32 && block != 64 && block != 128)
    B2Q_FAIL(h, B2Q_ERR_INVALID_ARGUMENT, "MicroScaling block_size must be one of [32, 64, 128], got %d", block);
  if (block != 32) B2Q_FAIL(h, B2Q_ERR_UNSUPPORTED, "gemv_fp4_wo: only 32-element scale blocks are implemented");
  if (tokens > 32) B2Q_FAIL(h, B2Q_ERR_UNSUPPORTED, "gemv_fp4_wo: decode path takes at most 32 tokens, got %lld", (long long)tokens);
  if (K % 128 != 0) B2Q_FAIL(h, B2Q_ERR_INVALID_DIMENSION, "gemv_fp4_wo: K must be a multiple of 128, got %lld", (long long)K);
  if (!codes || !scales || !x_bf16 || !out || scale_format < 0 || scale_format > 1 || out_type < 0 || out_type > 1)
    B2Q_FAIL(h, B2Q_ERR_INVALID_ARGUMENT, "gemv_fp4_wo: bad argument");
  if (((reinterpret_cast<uintptr_t>(codes) | reinterpret_cast<uintptr_t>(x_bf16)) & 15) != 0)
    B2Q_FAIL(h, B2Q_ERR_INVALID_ARGUMENT, "gemv_fp4_wo: codes and activations must be 16-byte aligned");
  if ((reinterpret_cast<uintptr_t>(scales) & (scale_format == B2Q_SCALE_E8M0 ? 3 : 15)) != 0)
    B2Q_FAIL(h, B2Q_ERR_INVALID_ARGUMENT, "gemv_fp4_wo: scales must be 4-byte (E8M0) or 16-byte (f32) aligned");
  const int t = (int)tokens;
  const bool small_n = N <= 2048;
  {
    // E8M0 scales, up to 16 tokens, matrices with a 256-row tile for (nearly) every SM and 64 MiB of codes or more: the
    // dense-format kernel (tcgen05 kind::mxf4, twice the bytes in flight; measured 27.9 against 29.8 us on 8192 x 28672).
    // Below that its fixed cost per call (seven-term activation split, six scale copies per stage, partial-sum exchange)
    // loses to the kernels below.  B2Q_GEMV_STREAM=2 / 0 forces it on (wherever it applies) / off.
    const bool pays = N >= 256 * 104 && N * (K / 2) >= ((int64_t)64 << 20);
    if (scale_format == B2Q_SCALE_E8M0 && t <= 16 && (h->sw.gemv_stream >= 0 ? h->sw.gemv_stream == 2 : pays)) {
      const int32_t st = b2q_gemv_fp4_mxf4_dispatch(h, codes, scales, x_bf16, t, N, K, out, out_type);
      if (st != B2Q_ERR_UNSUPPORTED) return st;
    }
  }
  {
    // E8M0 scales: the tcgen05 block-scaled kernel (weights never touch a CUDA core) where its fixed cost pays:
    // from 16 MiB of codes with 4 tokens or more or with enough rows for one tile per SM (no partial sums to
    // exchange), from 40 MiB otherwise.  B2Q_GEMV_MX=1 / 0 forces it on / off.
    const int64_t code_bytes = N * (K / 2);
    const bool mx_pays = code_bytes >= ((int64_t)40 << 20) || (code_bytes >= ((int64_t)16 << 20) && (t >= 4 || N >= 13312));
    if (scale_format == B2Q_SCALE_E8M0 && (h->sw.gemv_mx >= 0 ? h->sw.gemv_mx == 1 : mx_pays)) {
      const int32_t st = b2q_gemv_fp4_mx_dispatch(h, codes, scales, x_bf16, t, N, K, out, out_type);
      if (st != B2Q_ERR_UNSUPPORTED) return st;
    }
  }
  if (t <= 8) {
    // experiment switch: B2Q_GEMV_CLUSTER=1 takes the cluster split-K kernel for small token counts too
    if (h->sw.gemv_cluster == 1)
      return small_n ? gemv::launch<1, 4>(h, codes, scales, scale_format, x_bf16, t, N, K, out, out_type)
                     : gemv::launch<1, 8>(h, codes, scales, scale_format, x_bf16, t, N, K, out, out_type);
    // E8M0 scales: 128-bit-load kernel (scale folded into the f16 codes, exact for powers of two) unless
    // B2Q_GEMV_EXACT=1 asks for the fp32-scaled kernel; f32 scales always take the fp32-scaled kernel.
    const bool scales16 = (reinterpret_cast<uintptr_t>(scales) & 15) == 0;
    if (scale_format == B2Q_SCALE_E8M0 && scales16 && h->sw.gemv_exact != 1)
      return K >= 8192 ? gemv::launch_e8<8>(h, codes, scales, x_bf16, t, N, K, out, out_type)
                       : gemv::launch_e8<4>(h, codes, scales, x_bf16, t, N, K, out, out_type);
    return K >= 8192 ? gemv::launch_small<8>(h, codes, scales, scale_format, x_bf16, t, N, K, out, out_type)
                     : gemv::launch_small<4>(h, codes, scales, scale_format, x_bf16, t, N, K, out, out_type);
  }
  {
    if (scale_format == B2Q_SCALE_E8M0 && h->sw.gemv_exact != 1) {
      if (t <= 16) return small_n ? gemv::launch_e8c<2, 4>(h, codes, scales, x_bf16, t, N, K, out, out_type)
                                  : gemv::launch_e8c<2, 8>(h, codes, scales, x_bf16, t, N, K, out, out_type);
      return small_n ? gemv::launch_e8c<4, 4>(h, codes, scales, x_bf16, t, N, K, out, out_type)
                     : gemv::launch_e8c<4, 8>(h, codes, scales, x_bf16, t, N, K, out, out_type);
    }
  }
  if (t <= 16) return small_n ? gemv::launch<2, 4>(h, codes, scales, scale_format, x_bf16, t, N, K, out, out_type)
                              : gemv::launch<2, 8>(h, codes, scales, scale_format, x_bf16, t, N, K, out, out_type);
  return small_n ? gemv::launch<4, 4>(h, codes, scales, scale_format, x_bf16, t, N, K, out, out_type)
                 : gemv::launch<4, 8>(h, codes, scales, scale_format, x_bf16, t, N, K, out, out_type);
}
