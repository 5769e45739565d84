// Block-scaled FP4 (E2M1 codes, E8M0 scale per 32) weight-only decode GEMV on tcgen05.mma kind::mxf4: the DENSE 4-bit
// operand format.     out[t, n] = sum_k x[t, k] * decode(codes[n, k]) * 2^(scale[n, k / 32] - 127)        tokens <= 16
// (Fp4GemmConfig / MicroScalingQuantizer semantics, crates/oxicuda-blas/src/precision/fp4_fp6_ops.rs:337-395, :879-897.)
//
// Why the dense format.  kind::mxf8f6f4 reads 4-bit codes from a padded layout (8 data + 8 pad bytes per 16 codes): a
// stage of 16 KiB from HBM takes 32 KiB of shared memory, so at most 64 KiB of HBM bytes are in flight per SM, and at a
// 1.2-1.5 us round trip that caps an SM at 36-40 GB/s (measured).  kind::mxf4 reads the codes as they are stored: a 32 KiB
// stage IS 32 KiB of HBM bytes, four stages keep 128 KiB in flight, and an MMA covers K = 64 instead of 32 (half the
// instructions per byte).  The price: both operands are 4-bit.  Every bf16 activation therefore enters as the sum of
// SEVEN E2M1 terms under power-of-two scales,  x = sum_i 2^(e - s_i) c_i,  s = {0, 2, 5, 8, 11, 14, 17},  e per (token,
// 32-block) the smallest exponent with max / 2^e <= 6,  c_i = rn_e2m1(residual_i / 2^(e - s_i)).  The residual after the
// first term is at most 2^e, after the second 2^(e-3), then it shrinks by 8 per term: after seven terms it is below
// 2^(e-18), i.e. under 2^-19 of the block maximum, and zero for every value of at least 2^-11 of the block maximum (a
// bf16 value has eight significant bits) -- the accuracy of the two-E4M3-term split of the other tensor-core kernel.
// The seven terms are seven rows of the M = 128 operand with their own scale bytes; the epilogue adds the seven
// accumulator rows of a token.  Row of token t, term i: (t / 4) * 32 + i * 4 + t % 4 (a TMEM lane quarter holds four tokens).
//
// Structure: one persistent CTA per SM, 4 stages of 256 weight rows x 256 K (32 KiB).  Warp 0 issues the weight copies,
// warps 6..9 own one ring slot each (weight scale atoms; for up to 4 tokens also the activation terms of the stage, so
// no pre-pass), warp 10 copies pre-quantized activations (5 to 16 tokens), warp 11 moves the scale atoms into TMEM one
// stage ahead of warp 1's MMAs, warps 2..5 are the epilogue.  (256-row tile, K stage) units are split evenly over the
// SMs; partial sums meet in a workspace, the last CTA to arrive at a tile adds them in CTA order.  Programmatic
// dependent launch; every mbarrier wait is bounded.
#include "tc_common.cuh"
#include <stdlib.h>

namespace mxf4 {

using namespace tcx;

constexpr int TILE_N = 256, BK = 256, kStages = 4, kTerms = 7, kTokPerQuarter = 4, kMaxTokens = 16;
constexpr int kBytesW = TILE_N * 128;            // 256 rows x 256 codes, dense: 32 KiB of HBM bytes
constexpr int kBytesA = 128 * 128;               // activation operand: 128 rows x 256 codes
constexpr int kBytesSf = 3072;                   // weight scale atoms (cell 0/1 x rows 0..127/128..255), activation scale atoms (cell 0/1)
constexpr int kStageBytes = kBytesW + kBytesA + kBytesSf;
constexpr int kBarOff = kStages * kStageBytes;
constexpr int kSmem = kBarOff + 256 + 1024;
constexpr int kTmemCols = 512, kSfCol = 256, kSfCols = 24;   // per stage: 16 columns of weight scales, 8 of activation scales
constexpr int kThreads = 32 * 12;
constexpr uint64_t kWaitLimitNs = 500000000ull;

__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int where) {
  return mbar_wait_bounded(bar, parity, abort_flag, kWaitLimitNs, where);
}
__device__ __forceinline__ void umma_mxf4(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t tsfa, uint32_t tsfb,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::mxf4.block_scale.scale_vec::2X [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(tsfa), "r"(tsfb) : "memory");
}
// two floats -> one byte of two E2M1 codes (lo in bits 0..3), and back
__device__ __forceinline__ uint32_t e2m1x2_encode(float lo, float hi) {
  uint32_t r;
  asm("{\n\t.reg .b8 t;\n\tcvt.rn.satfinite.e2m1x2.f32 t, %1, %2;\n\tcvt.u32.u8 %0, t;\n\t}" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}
__device__ __forceinline__ float2 e2m1x2_decode(uint32_t byte) {
  uint32_t h;
  asm("{\n\t.reg .b8 t;\n\tcvt.u8.u32 t, %1;\n\tcvt.rn.f16x2.e2m1x2 %0, t;\n\t}" : "=r"(h) : "r"(byte));
  return __half22float2(*reinterpret_cast<const __half2*>(&h));
}
__device__ __forceinline__ int term_row(int t, int term) { return (t / kTokPerQuarter) * 32 + term * kTokPerQuarter + t % kTokPerQuarter; }
__device__ __forceinline__ int term_shift(int i) { return i == 0 ? 0 : 3 * i - 1; }   // 0, 2, 5, 8, 11, 14, 17

// Block exponent: the smallest e with amax / 2^e <= 6 (= 1.5 * 2^2); 0 for an empty or non-finite block.
__device__ __forceinline__ int block_exponent(float amax) {
  const uint32_t ab = __float_as_uint(amax);
  int e = (int)((ab >> 23) & 0xFF) - 127 - 2 + ((ab & 0x007FFFFFu) > 0x00400000u ? 1 : 0);
  if (amax == 0.0f || !(amax <= 3.0e38f)) e = 0;
  return max(e, -104);                                           // keeps every term's exponent e - 17 inside E8M0
}
// Eight consecutive activations (f[0..7], block exponent e) -> the eight codes of term `i` as one 32-bit word
// (element j in nibble j), residuals updated in place.
__device__ __forceinline__ uint32_t term_codes(float (&f)[8], int e, int i) {
  const int ei = e - term_shift(i);
  const float inv = __uint_as_float((uint32_t)(127 - ei) << 23), s = __uint_as_float((uint32_t)(127 + ei) << 23);
  uint32_t w = 0;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const uint32_t b = e2m1x2_encode(f[2 * j] * inv, f[2 * j + 1] * inv);
    const float2 d = e2m1x2_decode(b);
    f[2 * j] -= d.x * s;                                         // exact: a bf16 value minus multiples of 2^(ei - 1)
    f[2 * j + 1] -= d.y * s;
    w |= b << (8 * j);
  }
  return w;
}

struct Params {
  const uint8_t* scales;      // [N][K/32] E8M0
  const __nv_bfloat16* x;     // [tokens][K] (inline mode)
  const uint8_t* xq;          // pre-pass output: per K stage `rows` x 128 code bytes (swizzled), then two 512-byte scale atoms
  float* partials;            // [tile][slot][kMaxTokens][256]
  int32_t* counters;
  void* out;
  int out_type;
  int tokens;
  int rows;                   // operand rows that hold token terms: 32 per four tokens
  int64_t N, K;
  int stages_per_tile, units, per, max_slots;
  uint32_t idesc;
  int wait_first, debug;
  int32_t* status;
};

// ---------------------------------------------------------------------------
// Activation pre-pass (5 to 16 tokens): one CTA per K stage; thread (token, 32-block) quantizes 32 values into the five
// term rows of the stage block (16-byte units XOR-swizzled by row & 7) and writes the block's scale byte of each term row
// into the stage's two scale atoms (row r, block b: atom b / 4, byte (r % 32) * 16 + (r / 32) * 4 + b % 4).
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256) x_quant_e2m1_kernel(const __nv_bfloat16* __restrict__ x, int tokens, int64_t K, int rows,
                                                          uint8_t* __restrict__ xq) {
  const int j = blockIdx.x;
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  uint8_t* blk = xq + (size_t)j * ((size_t)rows * 128 + 1024);
  uint8_t* atoms = blk + (size_t)rows * 128;
  for (int it = threadIdx.x; it < tokens * 8; it += 256) {
    const int t = it >> 3, b = it & 7;
    const uint4* src = reinterpret_cast<const uint4*>(x + (int64_t)t * K + (int64_t)j * BK + b * 32);
    uint4 v[4];
#pragma unroll
    for (int c = 0; c < 4; ++c) v[c] = __ldg(src + c);
    float f[4][8];
    float amax = 0.0f;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const uint32_t w[4] = {v[c].x, v[c].y, v[c].z, v[c].w};
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        f[c][2 * k] = __uint_as_float(w[k] << 16);
        f[c][2 * k + 1] = __uint_as_float(w[k] & 0xFFFF0000u);
        amax = fmaxf(amax, fmaxf(fabsf(f[c][2 * k]), fabsf(f[c][2 * k + 1])));
      }
    }
    const int e = block_exponent(amax);
#pragma unroll
    for (int i = 0; i < kTerms; ++i) {
      const int r = term_row(t, i);
      uint4 codes;
      codes.x = term_codes(f[0], e, i); codes.y = term_codes(f[1], e, i); codes.z = term_codes(f[2], e, i); codes.w = term_codes(f[3], e, i);
      *reinterpret_cast<uint4*>(blk + r * 128 + ((b ^ (r & 7)) << 4)) = codes;     // 32 codes = one 16-byte unit
      atoms[(b >> 2) * 512 + (r & 31) * 16 + (r >> 5) * 4 + (b & 3)] = (uint8_t)(e - term_shift(i) + 127);
    }
  }
}

template <bool INL>
__global__ void __launch_bounds__(kThreads, 1) gemv_fp4_mxf4_kernel(const __grid_constant__ CUtensorMap map_w, const Params p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t bar_base = base + kBarOff;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (kStages + s); };
  auto sf_bar = [&](int s) { return bar_base + 8u * (2 * kStages + s); };
  const uint32_t tfull_bar = bar_base + 8u * (3 * kStages), tempty_bar = tfull_bar + 8, drain_bar = tfull_bar + 16;
  __shared__ uint32_t s_tmem_base;
  __shared__ int s_abort;
  __shared__ int s_last;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int S = p.stages_per_tile;
  const int u0 = blockIdx.x * p.per, u1 = min(u0 + p.per, p.units);
  const int total = u1 - u0;
  const uint32_t bytes_a = (uint32_t)p.rows * 128u;

  if (p.wait_first) asm volatile("griddepcontrol.wait;" ::: "memory");
  if (threadIdx.x == 0) {
    s_abort = 0;
    for (int s = 0; s < kStages; ++s) { mbar_init(full_bar(s), INL ? 2 : 3); mbar_init(empty_bar(s), 1); mbar_init(sf_bar(s), 1); }
    mbar_init(tfull_bar, 1); mbar_init(tempty_bar, 4); mbar_init(drain_bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_w)) : "memory");
    for (int it = 0; it < kStages && it < total; ++it) {      // the first round of weight copies: start the HBM stream now
      const int u = u0 + it, tile = u / S, j = u - tile * S;
      mbar_expect_tx(full_bar(it), kBytesW);
      tma_load_2d(base + it * kStageBytes, &map_w, full_bar(it), j * BK, tile * TILE_N);
    }
  }
  // operand rows that hold no token term: zero codes and a scale of one, once (their accumulator rows are never read)
  for (int s = 0; s < kStages; ++s) {
    uint4* az = reinterpret_cast<uint4*>(base_ptr + s * kStageBytes + kBytesW);
    for (int k = threadIdx.x; k < kBytesA / 16; k += kThreads) az[k] = make_uint4(0, 0, 0, 0);
    uint32_t* sz = reinterpret_cast<uint32_t*>(base_ptr + s * kStageBytes + kBytesW + kBytesA + 2048);
    for (int k = threadIdx.x; k < 256; k += kThreads) sz[k] = 0x7F7F7F7Fu;
  }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  if (warp == 1) tmem_alloc(smem_u32(&s_tmem_base), kTmemCols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = s_tmem_base;
  volatile int* abort_flag = &s_abort;
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  if (warp == 0) {
    // ---------------- weight producer: one TMA copy (32 KiB) per stage ----------------
    if (lane == 0) {
      bool ok = true;
      for (int it = kStages; it < total; ++it) {
        const int u = u0 + it, tile = u / S, j = u - tile * S;
        const int s = it % kStages;
        const uint32_t ph = (uint32_t)(it / kStages) & 1;
        if (!mbar_wait(empty_bar(s), ph ^ 1, abort_flag, 1)) { ok = false; break; }
        if (p.debug == 6) { mbar_arrive(full_bar(s)); continue; }   // timing experiment: no weight copies
        mbar_expect_tx(full_bar(s), kBytesW);
        tma_load_2d(base + s * kStageBytes, &map_w, full_bar(s), j * BK, tile * TILE_N);
      }
      if (!ok || *abort_flag) {
        const uint64_t t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 2000000ull) {}
      }
    }
  } else if (warp == 10) {
    // ---------------- activation producer (pre-pass mode): the term rows and their two scale atoms per stage ----------------
    if (lane == 0 && !INL) {
      asm volatile("griddepcontrol.wait;" ::: "memory");
      const size_t stride = (size_t)bytes_a + 1024;
      for (int it = 0; it < total; ++it) {
        const int j = (u0 + it) % S;
        const int s = it % kStages;
        const uint32_t ph = (uint32_t)(it / kStages) & 1;
        if (!mbar_wait(empty_bar(s), ph ^ 1, abort_flag, 5)) break;
        const uint32_t sa = base + s * kStageBytes + kBytesW;
        mbar_expect_tx(full_bar(s), bytes_a + 1024);
        bulk_load(sa, p.xq + (size_t)j * stride, bytes_a, full_bar(s));
        bulk_load(sa + kBytesA + 2048, p.xq + (size_t)j * stride + bytes_a, 1024, full_bar(s));
      }
    }
  } else if (warp >= 6 && warp < 10) {
    // ---------------- weight scale atoms (and, inline mode, the activation terms): warp w owns ring slot w ----------------
    const int slot = warp - 6;
    const int64_t kblocks = p.K >> 5;
    constexpr int kRing = 2;
    uint2 q[kRing][8];                                           // the stage's eight scale bytes of rows lane + 32 i
    auto load_scales = [&](int u, uint2 (&dst)[8]) {
      const int tile = u / S, j = u - tile * S;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int64_t row = min((int64_t)tile * TILE_N + lane + 32 * i, p.N - 1);
        dst[i] = __ldg(reinterpret_cast<const uint2*>(p.scales + row * kblocks + j * 8));
      }
    };
    // inline activations: lane -> 32-block b = lane & 7 of the stage, token lane >> 3 (up to four tokens)
    const int xb = lane & 7, xt = lane >> 3;
    uint4 xr[kRing][4];
    auto load_x = [&](int u, uint4 (&dst)[4]) {
      const int j = u % S;
      const uint4* src = reinterpret_cast<const uint4*>(p.x + (int64_t)xt * p.K + (int64_t)j * BK + xb * 32);
#pragma unroll
      for (int c = 0; c < 4; ++c) dst[c] = xt < p.tokens ? __ldg(src + c) : make_uint4(0, 0, 0, 0);
    };
#pragma unroll
    for (int r = 0; r < kRing; ++r)
      if (slot + kStages * r < total) load_scales(u0 + slot + kStages * r, q[r]);
    if constexpr (INL) {
      asm volatile("griddepcontrol.wait;" ::: "memory");        // the activations may come from the previous kernel of the stream
#pragma unroll
      for (int r = 0; r < kRing; ++r)
        if (slot + kStages * r < total) load_x(u0 + slot + kStages * r, xr[r]);
    }
    bool ok = true;
    for (int it0 = slot; it0 < total && ok; it0 += kStages * kRing) {
#pragma unroll
      for (int r = 0; r < kRing; ++r) {
        const int it = it0 + kStages * r;
        if (it >= total) break;
        // quantize before waiting for the slot: the codes sit in registers when the slot frees
        uint4 codes[kTerms];
        int e = 0;
        if constexpr (INL) {
          float f[4][8];
          float amax = 0.0f;
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            const uint32_t w[4] = {xr[r][c].x, xr[r][c].y, xr[r][c].z, xr[r][c].w};
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              f[c][2 * k] = __uint_as_float(w[k] << 16);
              f[c][2 * k + 1] = __uint_as_float(w[k] & 0xFFFF0000u);
              amax = fmaxf(amax, fmaxf(fabsf(f[c][2 * k]), fabsf(f[c][2 * k + 1])));
            }
          }
          e = block_exponent(amax);
#pragma unroll
          for (int i = 0; i < kTerms; ++i) {
            codes[i].x = term_codes(f[0], e, i); codes[i].y = term_codes(f[1], e, i);
            codes[i].z = term_codes(f[2], e, i); codes[i].w = term_codes(f[3], e, i);
          }
        }
        const uint32_t ph = (uint32_t)(it / kStages) & 1;
        if (!mbar_wait(empty_bar(slot), ph ^ 1, abort_flag, 6)) { ok = false; break; }
        uint8_t* sa = base_ptr + slot * kStageBytes + kBytesW;
        uint8_t* sf = sa + kBytesA;
        // weight scale atoms: (cell 0 | 1) x (rows 0..127 | 128..255)
        *reinterpret_cast<uint4*>(sf + lane * 16) = make_uint4(q[r][0].x, q[r][1].x, q[r][2].x, q[r][3].x);
        *reinterpret_cast<uint4*>(sf + 512 + lane * 16) = make_uint4(q[r][4].x, q[r][5].x, q[r][6].x, q[r][7].x);
        *reinterpret_cast<uint4*>(sf + 1024 + lane * 16) = make_uint4(q[r][0].y, q[r][1].y, q[r][2].y, q[r][3].y);
        *reinterpret_cast<uint4*>(sf + 1536 + lane * 16) = make_uint4(q[r][4].y, q[r][5].y, q[r][6].y, q[r][7].y);
        if constexpr (INL) {
          if (xt < p.tokens) {
#pragma unroll
            for (int i = 0; i < kTerms; ++i) {
              const int row = term_row(xt, i);
              *reinterpret_cast<uint4*>(sa + row * 128 + ((xb ^ (row & 7)) << 4)) = codes[i];
              sf[2048 + (xb >> 2) * 512 + (row & 31) * 16 + (row >> 5) * 4 + (xb & 3)] = (uint8_t)(e - term_shift(i) + 127);
            }
          }
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0) mbar_arrive(full_bar(slot));
        if (it + kStages * kRing < total) {
          load_scales(u0 + it + kStages * kRing, q[r]);
          if constexpr (INL) load_x(u0 + it + kStages * kRing, xr[r]);
        }
      }
    }
  } else if (warp == 11) {
    // ---------------- scale atoms into TMEM, ahead of the MMAs ----------------
    if (lane == 0) {
      for (int it = 0; it < total; ++it) {
        const int s = it % kStages;
        const uint32_t ph = (uint32_t)(it / kStages) & 1;
        if (!mbar_wait(full_bar(s), ph, abort_flag, 8)) break;
        tc_fence_after();
        const uint32_t ssf = base + s * kStageBytes + kBytesW + kBytesA;
        const uint32_t tsf = tmem_base + kSfCol + s * kSfCols;
        // weights: cell c -> columns [8 c, 8 c + 8): rows 0..127 then rows 128..255; activations: cell c -> columns 16 + 4 c
        if (p.debug != 7) {                                      // 7: timing experiment without the scale copies
          tmem_cp_sf(tsf, make_desc_sf(ssf));
          tmem_cp_sf(tsf + 4, make_desc_sf(ssf + 512));
          tmem_cp_sf(tsf + 8, make_desc_sf(ssf + 1024));
          tmem_cp_sf(tsf + 12, make_desc_sf(ssf + 1536));
          tmem_cp_sf(tsf + 16, make_desc_sf(ssf + 2048));
          tmem_cp_sf(tsf + 20, make_desc_sf(ssf + 2560));
        }
        tc_commit(sf_bar(s));
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      bool ok = true;
      int it = 0;
      uint32_t seg_it = 0;
      for (int u = u0; u < u1 && ok; ++seg_it) {
        const int tile = u / S, j0 = u - tile * S;
        const int n = min(u1 - u, S - j0);
        if (!mbar_wait(tempty_bar, (seg_it & 1) ^ 1, abort_flag, 2)) { ok = false; break; }
        tc_fence_after();
        for (int i = 0; i < n; ++i, ++it) {
          const int s = it % kStages;
          const uint32_t ph = (uint32_t)(it / kStages) & 1;
          if (!mbar_wait(sf_bar(s), ph, abort_flag, 3)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sw = base + s * kStageBytes, sa = sw + kBytesW;
          const uint32_t tsf = tmem_base + kSfCol + s * kSfCols;
          const uint64_t adesc = make_desc_sw128(sa), bdesc = make_desc_sw128(sw);
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            if (p.debug == 5) break;                             // timing experiment: no MMAs
            // K = 64 per MMA: +32 bytes inside the swizzle atom; scale cell k / 2, bytes (k % 2) * 2 and + 1 of it
            const uint32_t sfid = (uint32_t)((k & 1) * 2);
            umma_mxf4(tmem_base, adesc + (uint64_t)(2 * k), bdesc + (uint64_t)(2 * k), p.idesc | (sfid << 29) | (sfid << 4),
                      tsf + 16 + (k >> 1) * 4, tsf + (k >> 1) * 8, (uint32_t)((i | k) != 0));
          }
          tc_commit(empty_bar(s));
        }
        if (ok) tc_commit(tfull_bar);
        u += n;
      }
      if (!ok) {
        tc_commit(drain_bar);
        const uint64_t t0 = globaltimer_ns();
        while (!mbar_try_wait(drain_bar, 0))
          if (globaltimer_ns() - t0 > 100000000ull) break;
      }
    }
  } else if (warp >= 2 && warp < 6) {
    // ---------------- epilogue: lane quarter q holds the terms of tokens 4 q .. 4 q + 3 ----------------
    const int q = warp & 3;
    const int t = q * kTokPerQuarter + lane;                     // valid for lane < 4
    const bool has_rows = q * 32 < p.rows;
    uint32_t seg_it = 0;
    bool ok = true;
    for (int u = u0; u < u1 && ok; ++seg_it) {
      const int tile = u / S, j0 = u - tile * S;
      const int n = min(u1 - u, S - j0);
      u += n;
      if (!mbar_wait(tfull_bar, seg_it & 1, abort_flag, 4)) { ok = false; break; }
      tc_fence_after();
      const int64_t n0 = (int64_t)tile * TILE_N;
      const bool whole = n == S;
      const int first = (tile * S) / p.per, last = (tile * S + S - 1) / p.per;
      const int nc = last - first + 1, slot = (int)blockIdx.x - first;
      float* mine = p.partials + ((int64_t)tile * p.max_slots + slot) * (kMaxTokens * TILE_N);
      if (has_rows) {
#pragma unroll 1
        for (int c = 0; c < TILE_N; c += 32) {
          uint32_t r[32];
          __syncwarp();
          tmem_ld32(tmem_base + c + ((uint32_t)(q * 32) << 16), r);
          tmem_ld_wait();
          float v[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const float a = __uint_as_float(r[i]);
            float sum = a;
#pragma unroll
            for (int k = 1; k < kTerms; ++k) sum += __shfl_down_sync(0xFFFFFFFFu, a, k * kTokPerQuarter);   // the token's other term rows
            v[i] = sum;
          }
          if (lane < kTokPerQuarter && t < p.tokens) {
            if (whole) {
              if (p.out_type == B2Q_OUT_BF16) {
                __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(p.out) + (int64_t)t * p.N + n0 + c;
                if (n0 + c + 32 <= p.N && ((reinterpret_cast<uintptr_t>(o) & 15) == 0)) {
#pragma unroll
                  for (int i = 0; i < 32; i += 8) {
                    uint4 pk;
                    __nv_bfloat162 h0 = __floats2bfloat162_rn(v[i], v[i + 1]), h1 = __floats2bfloat162_rn(v[i + 2], v[i + 3]);
                    __nv_bfloat162 h2 = __floats2bfloat162_rn(v[i + 4], v[i + 5]), h3 = __floats2bfloat162_rn(v[i + 6], v[i + 7]);
                    pk.x = *reinterpret_cast<uint32_t*>(&h0); pk.y = *reinterpret_cast<uint32_t*>(&h1);
                    pk.z = *reinterpret_cast<uint32_t*>(&h2); pk.w = *reinterpret_cast<uint32_t*>(&h3);
                    *reinterpret_cast<uint4*>(o + i) = pk;
                  }
                } else {
#pragma unroll
                  for (int i = 0; i < 32; ++i) if (n0 + c + i < p.N) o[i] = __float2bfloat16_rn(v[i]);
                }
              } else {
                float* o = reinterpret_cast<float*>(p.out) + (int64_t)t * p.N + n0 + c;
#pragma unroll
                for (int i = 0; i < 32; ++i) if (n0 + c + i < p.N) o[i] = v[i];
              }
            } else {
              float4* o = reinterpret_cast<float4*>(mine + t * TILE_N + c);
#pragma unroll
              for (int i = 0; i < 32; i += 4) o[i >> 2] = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(tempty_bar);
      if (!whole) {
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (warp == 2 && lane == 0) {
          __threadfence();
          const int old = atomicAdd(p.counters + tile, 1);
          s_last = (old == nc - 1);
          if (old == nc - 1) p.counters[tile] = 0;
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (s_last) {
          __threadfence();
          const float* all = p.partials + (int64_t)tile * p.max_slots * (kMaxTokens * TILE_N);
          const int e = (warp - 2) * 32 + lane;                 // columns e and e + 128 of the tile
          for (int tk0 = 0; tk0 < p.tokens; tk0 += 8) {
            float s0[8], s1[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) { s0[i] = 0.0f; s1[i] = 0.0f; }
            for (int cc = 0; cc < nc; ++cc) {
              float a0[8], a1[8];
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                const bool in = tk0 + i < p.tokens;
                a0[i] = in ? __ldcg(all + (int64_t)cc * (kMaxTokens * TILE_N) + (tk0 + i) * TILE_N + e) : 0.0f;
                a1[i] = in ? __ldcg(all + (int64_t)cc * (kMaxTokens * TILE_N) + (tk0 + i) * TILE_N + e + 128) : 0.0f;
              }
#pragma unroll
              for (int i = 0; i < 8; ++i) { s0[i] += a0[i]; s1[i] += a1[i]; }
            }
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const int tk = tk0 + i;
              if (tk >= p.tokens) break;
              const int64_t c0 = n0 + e, c1 = n0 + e + 128;
              if (p.out_type == B2Q_OUT_BF16) {
                __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(p.out) + (int64_t)tk * p.N;
                if (c0 < p.N) o[c0] = __float2bfloat16_rn(s0[i]);
                if (c1 < p.N) o[c1] = __float2bfloat16_rn(s1[i]);
              } else {
                float* o = reinterpret_cast<float*>(p.out) + (int64_t)tk * p.N;
                if (c0 < p.N) o[c0] = s0[i];
                if (c1 < p.N) o[c1] = s1[i];
              }
            }
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
  if (threadIdx.x == 0 && s_abort) atomicCAS(p.status, 0, p.debug ? 400 + s_abort : (int)B2Q_ERR_TIMEOUT);
}

static inline size_t align256(size_t v) { return (v + 255) & ~(size_t)255; }

int32_t launch(b2q_handle h, const uint8_t* codes, const uint8_t* scales, const void* x, int tokens, int64_t N, int64_t K, void* out,
               int out_type) {
  EncodeTiledFn enc = get_encode_fn();
  if (!enc) B2Q_FAIL(h, B2Q_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  // weight codes as a [N][K] tensor of packed 4-bit elements; a box is 256 codes x 256 rows = 128-byte rows, 128-byte swizzle
  CUtensorMap map_w;
  cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)N};
  cuuint64_t strides[1] = {(cuuint64_t)(K / 2)};
  cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)TILE_N};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(&map_w, CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN8B, 2, const_cast<uint8_t*>(codes), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) B2Q_FAIL(h, B2Q_ERR_CUDA, "cuTensorMapEncodeTiled (packed 4-bit weights) failed with CUresult %d", (int)r);

  Params p = {};
  const int S = (int)(K / BK);
  const int64_t tiles = ceil_div64(N, TILE_N);
  const int64_t units = tiles * S;
  const int64_t slots = h->sm_count;
  int grid, per;
  if (tiles * 10 >= slots * 7) {                                // enough tiles to occupy most SMs: whole tiles, no partial sums
    per = S * (int)ceil_div64(tiles, slots);
    grid = (int)ceil_div64(units, per);
  } else {
    grid = (int)(units < slots ? units : slots);
    per = (int)ceil_div64(units, grid);
    grid = (int)ceil_div64(units, per);
  }
  p.max_slots = (S + per - 1) / per + 1;
  p.rows = 32 * ((tokens + kTokPerQuarter - 1) / kTokPerQuarter);
  const size_t xq_bytes = align256((size_t)S * ((size_t)p.rows * 128 + 1024));
  const size_t part_bytes = (size_t)tiles * p.max_slots * kMaxTokens * TILE_N * sizeof(float);
  void* ws = nullptr;
  int32_t st = b2q_workspace(h, xq_bytes + part_bytes, &ws);
  if (st != B2Q_OK) return st;
  p.scales = scales;
  p.x = reinterpret_cast<const __nv_bfloat16*>(x);
  p.xq = reinterpret_cast<const uint8_t*>(ws);
  p.partials = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(ws) + xq_bytes);
  p.counters = h->d_tile_counters;
  p.out = out; p.out_type = out_type; p.tokens = tokens; p.N = N; p.K = K;
  p.stages_per_tile = S; p.units = (int)units; p.per = per;
  // kind::mxf4 descriptor: A and B = E2M1 (format 1 of this kind), both K-major, N = 256, E8M0 scales, M = 128, K = 64
  p.idesc = (1u << 7) | (1u << 10) | ((uint32_t)(TILE_N >> 3) << 17) | (1u << 23) | ((uint32_t)(128 >> 4) << 24);
  p.wait_first = h->dynamic_weights;
  if (h->sw.mx_debug > 0) p.debug = h->sw.mx_debug;
  p.status = h->d_status;

  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  const int num_attrs = h->sw.mx_pdl == 0 ? 0 : 1;
  const bool inl = tokens <= 4 && h->sw.mx_inline != 0;
  if (!inl) {
    cudaLaunchConfig_t pre = {};
    pre.gridDim = dim3((unsigned)S);
    pre.blockDim = dim3(256);
    pre.stream = h->stream;
    pre.attrs = attr;
    pre.numAttrs = num_attrs;
    B2Q_CUDA(h, cudaLaunchKernelEx(&pre, x_quant_e2m1_kernel, (const __nv_bfloat16*)x, tokens, K, p.rows, reinterpret_cast<uint8_t*>(ws)));
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)grid);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = kSmem;
  cfg.stream = h->stream;
  cfg.attrs = attr;
  cfg.numAttrs = num_attrs;
  if (inl) {
    B2Q_SMEM_ATTR(h, gemv_fp4_mxf4_kernel<true>, kSmem);
    B2Q_CUDA(h, cudaLaunchKernelEx(&cfg, gemv_fp4_mxf4_kernel<true>, map_w, p));
  } else {
    B2Q_SMEM_ATTR(h, gemv_fp4_mxf4_kernel<false>, kSmem);
    B2Q_CUDA(h, cudaLaunchKernelEx(&cfg, gemv_fp4_mxf4_kernel<false>, map_w, p));
  }
  return B2Q_OK;
}

}  // namespace mxf4

// Dense-format (kind::mxf4) FP4 decode GEMV; B2Q_ERR_UNSUPPORTED (nothing launched) when the shape or the alignment does
// not fit: up to 16 tokens, K % 256 == 0, codes 32-byte aligned, scales 8-byte aligned, activations 16-byte aligned.
int32_t b2q_gemv_fp4_mxf4_dispatch(b2q_handle h, const uint8_t* codes, const void* scales, const void* x, int tokens, int64_t N, int64_t K,
                                   void* out, int out_type) {
  if (tokens < 1 || tokens > mxf4::kMaxTokens || K % 256 != 0 || N < 1) return B2Q_ERR_UNSUPPORTED;
  if ((reinterpret_cast<uintptr_t>(codes) & 31) != 0 || (reinterpret_cast<uintptr_t>(scales) & 7) != 0 ||
      (reinterpret_cast<uintptr_t>(x) & 15) != 0)
    return B2Q_ERR_UNSUPPORTED;
  const int64_t tiles = ceil_div64(N, mxf4::TILE_N);
  if (tiles > (int64_t)kTileCounters || tiles * (K / mxf4::BK) > 0x7FFFFFFF) return B2Q_ERR_UNSUPPORTED;
  return mxf4::launch(h, codes, (const uint8_t*)scales, x, tokens, N, K, out, out_type);
}
