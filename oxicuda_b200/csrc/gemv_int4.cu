// INT4 group-scaled weight-only linear (GPTQ / AWQ style): eight two's-complement nibbles per u32, one f16 scale per
// `group_size` weights along K.  crates/oxicuda-blas/src/precision/int_ops.rs:196-429 (Int4GemmConfig, pack_int4,
// unpack_int4), :602-757 (the kernel the reference generates).
//   * gemm_int4_ref_order_kernel: the reference kernel's arithmetic element for element (f32 activations [K x N],
//     k-ascending fma of float(int4) * scale) — bit-exact against the CPU oracle, any valid shape;
//   * gemv_int4_kernel: the decode path (up to 32 tokens, bf16 activations [tokens x K], K % 128 == 0), HBM-bound:
//     0.5 byte per weight plus 2 bytes per group.  Weights go from nibbles to f16 pairs with one logic operation and
//     one half2 subtraction per pair, straight into mma.sync.m16n8k16 A fragments; every MMA stays inside one block of 32
//     weights, so the group scale is applied to its fp32 result.
#include "common.cuh"
#include <cooperative_groups.h>
#include <stdlib.h>

namespace cg = cooperative_groups;

namespace i4w {

constexpr int KC = 512;   // K elements per staged activation chunk (4 steps of 128)

__device__ __forceinline__ uint32_t ld_stream_u32(const void* p) {
  uint32_t r;
  asm volatile("ld.global.nc.u32 %0, [%1];" : "=r"(r) : "l"(p));
  return r;
}

// ---------------------------------------------------------------------------
// pack_int4 on the device: one thread per output word; a value outside [-8, 7] records B2Q_ERR_INVALID_ARGUMENT.
// ---------------------------------------------------------------------------
__global__ void pack_int4_kernel(const int8_t* __restrict__ values, int64_t words, uint32_t* __restrict__ packed, int32_t* status) {
  for (int64_t w = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; w < words; w += (int64_t)gridDim.x * blockDim.x) {
    const uint2 v = *reinterpret_cast<const uint2*>(values + w * 8);
    uint32_t p = 0;
    bool bad = false;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int val = (int)(int8_t)(((j < 4 ? v.x : v.y) >> (8 * (j & 3))) & 0xFF);
      bad |= val < -8 || val > 7;
      p |= ((uint32_t)val & 0xFu) << (4 * j);
    }
    if (bad) atomicCAS(status, 0, (int)B2Q_ERR_INVALID_ARGUMENT);
    packed[w] = p;
  }
}
__global__ void unpack_int4_kernel(const uint32_t* __restrict__ packed, int64_t words, int8_t* __restrict__ out) {
  for (int64_t w = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; w < words; w += (int64_t)gridDim.x * blockDim.x) {
    const uint32_t p = packed[w];
    uint32_t lo = 0, hi = 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const uint32_t nib = (p >> (4 * j)) & 0xFu;
      const uint32_t b = (nib & 8u) ? (nib | 0xF0u) : nib;
      if (j < 4) lo |= b << (8 * j); else hi |= b << (8 * (j - 4));
    }
    *reinterpret_cast<uint2*>(out + w * 8) = make_uint2(lo, hi);
  }
}

// ---------------------------------------------------------------------------
// The reference kernel, one thread per element of C (column index fastest, as in the reference's launch).
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256) gemm_int4_ref_order_kernel(const uint32_t* __restrict__ a_packed, const __half* __restrict__ scales,
                                                                  const float* __restrict__ b, float* __restrict__ c, int64_t M, int64_t N,
                                                                  int64_t K, int64_t group) {
  const int64_t col = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t row = (int64_t)blockIdx.y * blockDim.y + threadIdx.y;
  if (row >= M || col >= N) return;
  const int64_t groups = K / group, kw = K >> 3;
  float acc = 0.0f;
  for (int64_t k = 0; k < K; k += 8) {
    const float scale = __half2float(scales[row * groups + k / group]);
    const uint32_t w = a_packed[row * kw + (k >> 3)];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const uint32_t nib = (w >> (4 * j)) & 0xFu;
      const int v = (nib & 8u) ? (int)(nib | 0xFFFFFFF0u) : (int)nib;
      acc = __fmaf_rn(__fmul_rn((float)v, scale), b[(k + j) * N + col], acc);
    }
  }
  c[row * N + col] = acc;
}

// ---------------------------------------------------------------------------
// Decode kernel
// ---------------------------------------------------------------------------
// Eight nibbles n0..n7 of a word -> f16 pairs (s0, s4), (s1, s5), (s2, s6), (s3, s7), s = two's-complement value.
// w ^ 0x88888888 turns every nibble into u = s + 8; (u | 0x6400) is the f16 1024 + u, (u << 4 | 0x6400) is 1024 + 16 u;
// one subtraction or one fused multiply-add per pair brings both back to s exactly.
__device__ __forceinline__ void cvt_int4x8(uint32_t w, uint32_t (&h)[4]) {
  const uint32_t x = w ^ 0x88888888u, y = x >> 8;
  const uint32_t lo0 = (x & 0x000F000Fu) | 0x64006400u, hi0 = (x & 0x00F000F0u) | 0x64006400u;
  const uint32_t lo1 = (y & 0x000F000Fu) | 0x64006400u, hi1 = (y & 0x00F000F0u) | 0x64006400u;
  const uint32_t k1032 = 0x64086408u, k16th = 0x2C002C00u, km72 = 0xD480D480u;   // 1032, 1/16, -72 as f16 pairs
  asm("sub.f16x2 %0, %1, %2;" : "=r"(h[0]) : "r"(lo0), "r"(k1032));
  asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(h[1]) : "r"(hi0), "r"(k16th), "r"(km72));
  asm("sub.f16x2 %0, %1, %2;" : "=r"(h[2]) : "r"(lo1), "r"(k1032));
  asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(h[3]) : "r"(hi1), "r"(k16th), "r"(km72));
}
__device__ __forceinline__ void mma_f16_zero(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%10, %10, %10, %10};"
      : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.0f));
}
__device__ __forceinline__ void mma_f16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float bf16_lo(uint32_t v) { return fminf(fmaxf(__uint_as_float(v << 16), -65504.0f), 65504.0f); }
__device__ __forceinline__ float bf16_hi(uint32_t v) { return fminf(fmaxf(__uint_as_float(v & 0xFFFF0000u), -65504.0f), 65504.0f); }
__device__ __forceinline__ uint32_t pack_f16x2(float lo, float hi) {
  const __half2 h = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&h);
}

// The f16 scales of the four blocks of 32 of one 128-wide step of one row: 4, 2 or 1 distinct values for a group size
// of 32, 64 or >= 128 (gsh = log2 of the group size).
template <bool WIDE> struct StepScales;          // WIDE: group size 32 (four scales per step); else 64 and up (two or one)
template <> struct StepScales<true> {
  uint32_t a, b;
  __device__ __forceinline__ void load(const __half* row_scales, int64_t k, int) {
    const uint2 v = __ldg(reinterpret_cast<const uint2*>(row_scales + (k >> 5)));
    a = v.x; b = v.y;
  }
  __device__ __forceinline__ void clear() { a = b = 0; }
  __device__ __forceinline__ float get(int j, int) const {
    return __half2float(__ushort_as_half((unsigned short)(((j < 2 ? a : b) >> (16 * (j & 1))) & 0xFFFFu)));
  }
};
template <> struct StepScales<false> {
  uint32_t a;
  __device__ __forceinline__ void load(const __half* row_scales, int64_t k, int gsh) {
    const __half* p = row_scales + (k >> gsh);
    a = gsh == 6 ? __ldg(reinterpret_cast<const uint32_t*>(p)) : (uint32_t)__ldg(reinterpret_cast<const unsigned short*>(p));
  }
  __device__ __forceinline__ void clear() { a = 0; }
  __device__ __forceinline__ float get(int j, int gsh) const {
    return __half2float(__ushort_as_half((unsigned short)((gsh == 6 && j >= 2 ? a >> 16 : a) & 0xFFFFu)));
  }
};

// MT: token tiles of 8.  WARPS: warps per CTA, 16 weight rows each.  A cluster of split_k CTAs covers K and adds
// the partial sums through distributed shared memory.
template <int MT, int WARPS, bool WIDE>
__global__ void __launch_bounds__(WARPS * 32) gemv_int4_kernel(const uint32_t* __restrict__ packed, const __half* __restrict__ scales, int gsh,
                                                               const __nv_bfloat16* __restrict__ x, int tokens, int64_t N, int64_t K,
                                                               void* out, int out_type, int split_k) {
  constexpr int MPAD = 8 * MT, R = 16 * WARPS, NT = WARPS * 32;
  extern __shared__ __align__(16) uint8_t smem[];
  uint4* xs = reinterpret_cast<uint4*>(smem);            // [block of 32 (16 per chunk)][MPAD][quad lane] x 16 bytes
  float* red = reinterpret_cast<float*>(smem);           // [MPAD][R]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, tig = lane & 3;
  const int ks = blockIdx.x % split_k;
  const int64_t row_tile = blockIdx.x / split_k, n0 = row_tile * R + warp * 16;
  const int64_t r0 = min(n0 + g, N - 1), r1 = min(n0 + g + 8, N - 1);   // clamped loads; rows >= N are dropped at the store
  const int64_t groups = K >> gsh;
  const uint8_t* w0 = reinterpret_cast<const uint8_t*>(packed) + r0 * (K >> 1) + tig * 4;   // this lane's word of every block of 32
  const uint8_t* w1 = reinterpret_cast<const uint8_t*>(packed) + r1 * (K >> 1) + tig * 4;
  const __half* s0 = scales + r0 * groups;
  const __half* s1 = scales + r1 * groups;
  const int chunks_total = (int)((K + KC - 1) / KC), cpc = (chunks_total + split_k - 1) / split_k;
  const int c_begin = ks * cpc, c_end = min(c_begin + cpc, chunks_total);
  float acc[MT][4];
#pragma unroll
  for (int t = 0; t < MT; ++t) acc[t][0] = acc[t][1] = acc[t][2] = acc[t][3] = 0.0f;

  for (int c = c_begin; c < c_end; ++c) {
    const int64_t k0 = (int64_t)c * KC;
    uint32_t wa[4][4], wb[4][4];
    StepScales<WIDE> sa[4], sb[4];
#pragma unroll
    for (int s = 0; s < 4; ++s) {                        // the HBM stream first
      const int64_t k = k0 + s * 128;
      if (k < K) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          wa[s][j] = ld_stream_u32(w0 + ((k + j * 32) >> 1));
          wb[s][j] = ld_stream_u32(w1 + ((k + j * 32) >> 1));
        }
        sa[s].load(s0, k, gsh);
        sb[s].load(s1, k, gsh);
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j) { wa[s][j] = 0; wb[s][j] = 0; }   // nibble 0 is the value 0
        sa[s].clear();
        sb[s].clear();
      }
    }
    __syncthreads();                                     // previous chunk's readers are done
    for (int i = threadIdx.x; i < 64 * MPAD; i += NT) {  // activations: bf16 -> f16 in the pair order of cvt_int4x8
      const int ttig = i & 3, tok = (i >> 2) % MPAD, blk = i / (4 * MPAD);
      const int64_t k = k0 + blk * 32 + ttig * 8;
      uint4 v = make_uint4(0, 0, 0, 0);
      if (tok < tokens && k < K) v = __ldg(reinterpret_cast<const uint4*>(x + (int64_t)tok * K + k));
      uint4 h;
      h.x = pack_f16x2(bf16_lo(v.x), bf16_lo(v.z));      // (k0, k4)
      h.y = pack_f16x2(bf16_hi(v.x), bf16_hi(v.z));      // (k1, k5)
      h.z = pack_f16x2(bf16_lo(v.y), bf16_lo(v.w));      // (k2, k6)
      h.w = pack_f16x2(bf16_hi(v.y), bf16_hi(v.w));      // (k3, k7)
      xs[i] = h;
    }
    __syncthreads();
#pragma unroll
    for (int s = 0; s < 4; ++s) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {                      // one block of 32: 8 weights per lane and row, two MMA k-steps
        uint32_t ha[4], hb[4];
        cvt_int4x8(wa[s][j], ha);
        cvt_int4x8(wb[s][j], hb);
        const float fa = sa[s].get(j, gsh), fb = sb[s].get(j, gsh);
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
  const int E = MPAD * R, per = (E + split_k - 1) / split_k;
  const int e_begin = ks * per, e_end = min(e_begin + per, E);
  for (int e = e_begin + threadIdx.x; e < e_end; e += NT) {
    float v = 0.0f;
    if (split_k > 1) { for (int pr = 0; pr < split_k; ++pr) v += cluster.map_shared_rank(red, pr)[e]; }
    else v = red[e];
    const int tok = e / R;
    const int64_t n = row_tile * R + (e % R);
    if (tok < tokens && n < N) {
      if (out_type == B2Q_OUT_BF16) reinterpret_cast<__nv_bfloat16*>(out)[(int64_t)tok * N + n] = __float2bfloat16_rn(v);
      else reinterpret_cast<float*>(out)[(int64_t)tok * N + n] = v;
    }
  }
  if (split_k > 1) cluster.sync();                       // peers may still be reading this CTA's partial sums
}

// ---------------------------------------------------------------------------
// Decode kernel for up to 8 tokens.  Instruction issue binds long before HBM, so: a CTA owns 16 weight rows and its WK
// warps split K into contiguous slices of 512-wide chunks; a warp loads the words and scales of its NEXT chunk into a
// second register set before it multiplies the current one (HBM loads stay in flight under the MMAs); every warp stages
// only its own slice of the activations (warp-private shared memory, __syncwarp); one __syncthreads at the end adds the
// WK partial sums.
// ---------------------------------------------------------------------------
template <bool WIDE> struct ChunkRegs {
  uint32_t wa[4][4], wb[4][4];
  StepScales<WIDE> sa[4], sb[4];
};
// w0 / w1: this lane's word of the chunk's first block of row g / g + 8; k: first K index of the chunk
template <bool WIDE>
__device__ __forceinline__ void load_chunk(ChunkRegs<WIDE>& r, const uint8_t* w0, const uint8_t* w1, const __half* s0, const __half* s1, int64_t k,
                                           int gsh, int steps) {
#pragma unroll
  for (int s = 0; s < 4; ++s) {
    if (s < steps) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        r.wa[s][j] = ld_stream_u32(w0 + s * 64 + j * 16);
        r.wb[s][j] = ld_stream_u32(w1 + s * 64 + j * 16);
      }
      r.sa[s].load(s0, k + s * 128, gsh);
      r.sb[s].load(s1, k + s * 128, gsh);
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j) { r.wa[s][j] = 0; r.wb[s][j] = 0; }
      r.sa[s].clear();
      r.sb[s].clear();
    }
  }
}
template <bool WIDE>
__device__ __forceinline__ void mul_chunk(const ChunkRegs<WIDE>& r, const uint4* xs_lane, int gsh, float (&acc)[4]) {
#pragma unroll
  for (int s = 0; s < 4; ++s) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      uint32_t ha[4], hb[4];
      cvt_int4x8(r.wa[s][j], ha);
      cvt_int4x8(r.wb[s][j], hb);
      const uint4 xv = xs_lane[(s * 4 + j) * 32];          // [block][8 token rows][4 quad lanes]
      float d[4];
      mma_f16_zero(d, ha[0], hb[0], ha[1], hb[1], xv.x, xv.y);
      mma_f16(d, ha[2], hb[2], ha[3], hb[3], xv.z, xv.w);
      const float fa = r.sa[s].get(j, gsh), fb = r.sb[s].get(j, gsh);
      acc[0] = fmaf(fa, d[0], acc[0]);
      acc[1] = fmaf(fa, d[1], acc[1]);
      acc[2] = fmaf(fb, d[2], acc[2]);
      acc[3] = fmaf(fb, d[3], acc[3]);
    }
  }
}
// Activations [tokens x 512] of one chunk into this warp's buffer: f16, in the pair order of cvt_int4x8.
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
    h.x = pack_f16x2(bf16_lo(v.x), bf16_lo(v.z));
    h.y = pack_f16x2(bf16_hi(v.x), bf16_hi(v.z));
    h.z = pack_f16x2(bf16_lo(v.y), bf16_lo(v.w));
    h.w = pack_f16x2(bf16_hi(v.y), bf16_hi(v.w));
    xs[(blk * 8 + tok) * 4 + ttig] = h;
  }
  __syncwarp();
}

template <int WK, int TOK, bool WIDE>
__global__ void __launch_bounds__(WK * 32, 512 / (WK * 32)) gemv_int4_small_kernel(const uint32_t* __restrict__ packed, const __half* __restrict__ scales,
                                                                                   int gsh, const __nv_bfloat16* __restrict__ x, int tokens, int64_t N,
                                                                                   int64_t K, void* out, int out_type) {
  extern __shared__ __align__(16) uint8_t smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, tig = lane & 3;
  uint4* xs = reinterpret_cast<uint4*>(smem) + warp * 512;        // [16 blocks][8 tokens][4] x 16 bytes = 8 KiB per warp
  float* red = reinterpret_cast<float*>(smem);                    // [WK][16 rows][8 tokens], reused after the main loop
  const int64_t n0 = (int64_t)blockIdx.x * 16;
  const int64_t r0 = min(n0 + g, N - 1), r1 = min(n0 + g + 8, N - 1);
  const int chunks_total = (int)((K + KC - 1) / KC), cpw = (chunks_total + WK - 1) / WK;
  int c = warp * cpw;
  const int c_end = min(c + cpw, chunks_total);
  const int total_steps = (int)(K >> 7);
  const uint8_t* w0 = reinterpret_cast<const uint8_t*>(packed) + r0 * (K >> 1) + tig * 4 + (int64_t)c * (KC / 2);
  const uint8_t* w1 = reinterpret_cast<const uint8_t*>(packed) + r1 * (K >> 1) + tig * 4 + (int64_t)c * (KC / 2);
  const __half* s0 = scales + r0 * (K >> gsh);
  const __half* s1 = scales + r1 * (K >> gsh);
  const __nv_bfloat16* xk = x + (int64_t)c * KC;
  int64_t k = (int64_t)c * KC;

  ChunkRegs<WIDE> A, B;
  if (c < c_end) load_chunk(A, w0, w1, s0, s1, k, gsh, min(4, total_steps - c * 4));
#pragma unroll
  for (int i = 0; i < 16; ++i) xs[lane + 32 * i] = make_uint4(0, 0, 0, 0);   // rows of no token stay zero
  const uint4* xs_lane = xs + g * 4 + tig;
  float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
  while (c < c_end) {
    if (c + 1 < c_end) load_chunk(B, w0 + KC / 2, w1 + KC / 2, s0, s1, k + KC, gsh, min(4, total_steps - (c + 1) * 4));
    stage_x_warp<TOK>(xs, xk, tokens, K, (int)min((int64_t)KC, K - k), lane);
    mul_chunk(A, xs_lane, gsh, acc);
    ++c; w0 += KC / 2; w1 += KC / 2; xk += KC; k += KC;
    if (c >= c_end) break;
    if (c + 1 < c_end) load_chunk(A, w0 + KC / 2, w1 + KC / 2, s0, s1, k + KC, gsh, min(4, total_steps - (c + 1) * 4));
    stage_x_warp<TOK>(xs, xk, tokens, K, (int)min((int64_t)KC, K - k), lane);
    mul_chunk(B, xs_lane, gsh, acc);
    ++c; w0 += KC / 2; w1 += KC / 2; xk += KC; k += KC;
  }
  __syncthreads();                                       // every warp is done with its activation buffer
  red[(warp * 16 + g) * 8 + tig * 2 + 0] = acc[0];
  red[(warp * 16 + g) * 8 + tig * 2 + 1] = acc[1];
  red[(warp * 16 + g + 8) * 8 + tig * 2 + 0] = acc[2];
  red[(warp * 16 + g + 8) * 8 + tig * 2 + 1] = acc[3];
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

template <int WK, int TOK, bool WIDE>
int32_t launch_small_t(b2q_handle h, const uint32_t* packed, const __half* scales, int gsh, const void* x, int tokens, int64_t N, int64_t K,
                       void* out, int out_type) {
  const size_t smem = (size_t)WK * 8192;
  if (smem > 48 * 1024) {
    B2Q_SMEM_ATTR(h, (gemv_int4_small_kernel<WK, TOK, WIDE>), (int)smem);
  }
  gemv_int4_small_kernel<WK, TOK, WIDE><<<(unsigned)ceil_div64(N, 16), WK * 32, smem, h->stream>>>(packed, scales, gsh, (const __nv_bfloat16*)x, tokens,
                                                                                             N, K, out, out_type);
  B2Q_LAUNCH_CHECK(h, "gemv_int4_small_kernel");
  return B2Q_OK;
}
template <int WK>
int32_t launch_small(b2q_handle h, const uint32_t* packed, const __half* scales, int gsh, const void* x, int tokens, int64_t N, int64_t K,
                     void* out, int out_type) {
#define I4_SMALL(TOK)                                                                                              \
  return gsh == 5 ? launch_small_t<WK, TOK, true>(h, packed, scales, gsh, x, tokens, N, K, out, out_type)          \
                  : launch_small_t<WK, TOK, false>(h, packed, scales, gsh, x, tokens, N, K, out, out_type)
  if (tokens <= 1) { I4_SMALL(1); }
  if (tokens <= 2) { I4_SMALL(2); }
  if (tokens <= 4) { I4_SMALL(4); }
  I4_SMALL(8);
#undef I4_SMALL
}

template <int MT, int WARPS>
int32_t launch(b2q_handle h, const uint32_t* packed, const __half* scales, int gsh, const void* x, int tokens, int64_t N, int64_t K,
               void* out, int out_type) {
  constexpr int R = 16 * WARPS;
  const int64_t row_tiles = ceil_div64(N, R);
  const int chunks = (int)ceil_div64(K, KC);
  int split = 1;   // cluster size: a divisor of the chunk count, the smallest that gives about 1.5 CTAs per SM
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
  if (gsh == 5) B2Q_CUDA(h, cudaLaunchKernelEx(&cfg, gemv_int4_kernel<MT, WARPS, true>, packed, scales, gsh, (const __nv_bfloat16*)x, tokens, N, K, out, out_type, split));
  else B2Q_CUDA(h, cudaLaunchKernelEx(&cfg, gemv_int4_kernel<MT, WARPS, false>, packed, scales, gsh, (const __nv_bfloat16*)x, tokens, N, K, out, out_type, split));
  return B2Q_OK;
}

// Int4GemmConfig::validate (int_ops.rs:250-283)
int32_t validate(b2q_handle h, int64_t m, int64_t n, int64_t k, int64_t group) {
  if (m <= 0 || n <= 0 || k <= 0) B2Q_FAIL(h, B2Q_ERR_INVALID_DIMENSION, "INT4 GEMM dimensions must be non-zero: m=%lld, n=%lld, k=%lld", (long long)m, (long long)n, (long long)k);
  if (k % 8 != 0) B2Q_FAIL(h, B2Q_ERR_INVALID_DIMENSION, "INT4 GEMM K dimension must be a multiple of 8 for packing, got k=%lld", (long long)k);
  if (group <= 0 || (group & (group - 1)) != 0) B2Q_FAIL(h, B2Q_ERR_INVALID_ARGUMENT, "INT4 group_size must be a positive power of 2, got %lld", (long long)group);
  if (k % group != 0) B2Q_FAIL(h, B2Q_ERR_INVALID_ARGUMENT, "INT4 group_size (%lld) must divide K (%lld) evenly", (long long)group, (long long)k);
  return B2Q_OK;
}

}  // namespace i4w

extern "C" {

int32_t b2q_pack_int4(b2q_handle h, const int8_t* values, int64_t n, uint32_t* packed) {
  B2Q_REQUIRE_HANDLE(h);
  if (n % 8 != 0) B2Q_FAIL(h, B2Q_ERR_INVALID_ARGUMENT, "pack_int4 requires input length to be a multiple of 8, got %lld", (long long)n);
  if (n <= 0) return B2Q_OK;
  if (!values || !packed || (reinterpret_cast<uintptr_t>(values) & 7)) B2Q_FAIL(h, B2Q_ERR_INVALID_ARGUMENT, "pack_int4: bad pointer");
  const int64_t words = n / 8;
  int64_t grid = ceil_div64(words, 256);
  if (grid > (int64_t)h->sm_count * 16) grid = (int64_t)h->sm_count * 16;
  i4w::pack_int4_kernel<<<(unsigned)grid, 256, 0, h->stream>>>(values, words, packed, h->d_status);
  B2Q_LAUNCH_CHECK(h, "pack_int4_kernel");
  return B2Q_OK;
}

int32_t b2q_unpack_int4(b2q_handle h, const uint32_t* packed, int64_t words, int8_t* out) {
  B2Q_REQUIRE_HANDLE(h);
  if (words <= 0) return B2Q_OK;
  if (!packed || !out || (reinterpret_cast<uintptr_t>(out) & 7)) B2Q_FAIL(h, B2Q_ERR_INVALID_ARGUMENT, "unpack_int4: bad pointer");
  int64_t grid = ceil_div64(words, 256);
  if (grid > (int64_t)h->sm_count * 16) grid = (int64_t)h->sm_count * 16;
  i4w::unpack_int4_kernel<<<(unsigned)grid, 256, 0, h->stream>>>(packed, words, out);
  B2Q_LAUNCH_CHECK(h, "unpack_int4_kernel");
  return B2Q_OK;
}

int32_t b2q_gemm_int4_f32(b2q_handle h, const uint32_t* a_packed, const void* scales_f16, const float* b, float* c, int64_t m, int64_t n,
                          int64_t k, int64_t group_size) {
  B2Q_REQUIRE_HANDLE(h);
  const int32_t st = i4w::validate(h, m, n, k, group_size);
  if (st != B2Q_OK) return st;
  if (!a_packed || !scales_f16 || !b || !c) B2Q_FAIL(h, B2Q_ERR_INVALID_ARGUMENT, "gemm_int4: null pointer");
  if (ceil_div64(m, 8) > 65535) B2Q_FAIL(h, B2Q_ERR_INVALID_DIMENSION, "gemm_int4: m %lld above the reference-order kernel's grid", (long long)m);
  const dim3 block(32, 8), grid((unsigned)ceil_div64(n, 32), (unsigned)ceil_div64(m, 8));
  i4w::gemm_int4_ref_order_kernel<<<grid, block, 0, h->stream>>>(a_packed, static_cast<const __half*>(scales_f16), b, c, m, n, k, group_size);
  B2Q_LAUNCH_CHECK(h, "gemm_int4_ref_order_kernel");
  return B2Q_OK;
}

int32_t b2q_gemv_int4_wo(b2q_handle h, const uint32_t* packed, const void* scales_f16, int64_t group_size, const void* x_bf16, int64_t tokens,
                         int64_t n, int64_t k, void* out, int out_type) {
  B2Q_REQUIRE_HANDLE(h);
  const int32_t st = i4w::validate(h, n, tokens, k, group_size);
  if (st != B2Q_OK) return st;
  if (!packed || !scales_f16 || !x_bf16 || !out) B2Q_FAIL(h, B2Q_ERR_INVALID_ARGUMENT, "gemv_int4: null pointer");
  if (out_type != B2Q_OUT_BF16 && out_type != B2Q_OUT_F32) B2Q_FAIL(h, B2Q_ERR_INVALID_ARGUMENT, "gemv_int4: out_type %d", out_type);
  if (tokens > 32) B2Q_FAIL(h, B2Q_ERR_UNSUPPORTED, "gemv_int4: %lld tokens (the decode kernel takes up to 32)", (long long)tokens);
  if (k % 128 != 0 || group_size < 32) B2Q_FAIL(h, B2Q_ERR_UNSUPPORTED, "gemv_int4: needs K %% 128 == 0 and group_size >= 32 (K=%lld, group=%lld); b2q_gemm_int4_f32 takes every valid shape", (long long)k, (long long)group_size);
  int gsh = 0;
  while (((int64_t)1 << gsh) < group_size) ++gsh;
  const uintptr_t salign = gsh == 5 ? 7 : (gsh == 6 ? 3 : 1);
  if ((reinterpret_cast<uintptr_t>(packed) & 3) || (reinterpret_cast<uintptr_t>(x_bf16) & 15) || (reinterpret_cast<uintptr_t>(scales_f16) & salign))
    B2Q_FAIL(h, B2Q_ERR_INVALID_ARGUMENT, "gemv_int4: operands must be aligned (activations 16 bytes, scales %d bytes)", (int)salign + 1);
  const __half* sc = static_cast<const __half*>(scales_f16);
  const int t = (int)tokens;
  const bool small_n = n <= 8192;   // few row tiles: 4 warps (64 rows) per CTA give more CTAs
  // One or two tokens with groups of 64 and up: the prefetching kernel (measured 65.5 against 71.6 us on 8192 x 28672);
  // with more tokens or groups of 32 its registers spill and the cluster kernel is faster (73.7 against 102 us at 4 tokens).
  // B2Q_INT4_SMALL=1 / 0 forces the choice.
  if (h->sw.int4_small >= 0 ? (h->sw.int4_small == 1 && t <= 8) : (t <= 2 && gsh >= 6)) {
    return k >= 8192 ? i4w::launch_small<8>(h, packed, sc, gsh, x_bf16, t, n, k, out, out_type)
                     : i4w::launch_small<4>(h, packed, sc, gsh, x_bf16, t, n, k, out, out_type);
  }
  if (t <= 8) return small_n ? i4w::launch<1, 4>(h, packed, sc, gsh, x_bf16, t, n, k, out, out_type) : i4w::launch<1, 8>(h, packed, sc, gsh, x_bf16, t, n, k, out, out_type);
  if (t <= 16) return small_n ? i4w::launch<2, 4>(h, packed, sc, gsh, x_bf16, t, n, k, out, out_type) : i4w::launch<2, 8>(h, packed, sc, gsh, x_bf16, t, n, k, out, out_type);
  return small_n ? i4w::launch<4, 4>(h, packed, sc, gsh, x_bf16, t, n, k, out, out_type) : i4w::launch<4, 8>(h, packed, sc, gsh, x_bf16, t, n, k, out, out_type);
}

}  // extern "C"
