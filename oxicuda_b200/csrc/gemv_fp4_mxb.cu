// Block-scaled FP4 (E2M1 codes, E8M0 scale per 32) weight-only decode GEMV on tcgen05 with the WEIGHTS as the N
// operand:   out[t, n] = sum_k x[t, k] * decode(codes[n, k]) * 2^(scale[n, k / 32] - 127)          tokens <= 32
// (Fp4GemmConfig / MicroScalingQuantizer semantics, crates/oxicuda-blas/src/precision/fp4_fp6_ops.rs:337-395,
//  :879-897, with the weight-only bf16-activation contract of the decode GEMV.)
//
// Why this shape.  A tcgen05.mma of K = 32 occupies the tensor pipe for about 123 clocks whatever M is and for any
// N up to 128, and for about 171 clocks at N = 256 (measured on B200).  With the weights as the M = 128 operand an
// instruction covers 128 rows x 32 codes = 2 KiB of packed weights: 16.8 bytes per clock and SM, 4.9 TB/s on 148 SMs,
// below the HBM rate.  With the weights as the N = 256 operand it covers 4 KiB in 171 clocks: 24 bytes per clock and
// SM (7.0 TB/s), so the kernel is bound by HBM, not by the instruction stream.  The activations are then the M operand
// (rows = token terms, M = 128 is the only block-scaled shape of one CTA; unused rows stay zero).
//
// Activations: the instruction takes 8-bit floats, so a pre-pass writes every bf16 activation as the sum of TWO E4M3
// codes under ONE power-of-two scale per token:  x = 2^e (c1 + c2),  c1 = rn(x / 2^e),  c2 = rn(x / 2^e - c1), with
// 2^e the smallest power of two that brings the token's largest magnitude under 448.  c1 + c2 is exact for
// |x| >= 2^-11 of the token's maximum, below that the absolute error is under 2^-18 of it.  A per-token scale means
// the activation scale atom is loaded into TMEM once per launch instead of once per stage.
// Row of token t, term i inside the 128-row operand: (t / 16) * 32 + i * 16 + t % 16, so both terms of a token sit in
// one warp's TMEM lane quarter and the epilogue adds them with one shuffle.
//
// One persistent CTA per SM, a ring of 4 stages (256 weight rows x 128 K: 16 KiB from HBM, expanded by the TMA unit
// to the 32 KiB padded layout the MMA reads).  Work units are (256-row tile, K stage) pairs split evenly over the SMs;
// a CTA that owns only part of a tile's K range writes its partial sums to a workspace and the last CTA to arrive at
// the tile (a counter per tile) adds them in CTA order and stores, so results do not depend on arrival order.
// Launches are chained by programmatic dependent launch; every mbarrier wait is bounded.
#include "tc_common.cuh"
#include <stdlib.h>

namespace mxb {

using namespace tcx;

constexpr int TILE_N = 256;      // weight rows per tile = accumulator columns
constexpr int BK = 128;          // K per stage
constexpr int kStages = 4;
constexpr int kBytesW = TILE_N * 128;            // in shared memory (half of it crosses HBM)
constexpr int kBytesA = 128 * 128;               // activation operand: 128 rows x 128 bytes, rows past the used ones stay zero
constexpr int kBytesSfb = 2048;                  // scale atoms: weight rows 0..127, 128..255, and (inline mode) the stage's activation atom
constexpr int kStageBytes = kBytesW + kBytesA + kBytesSfb;
constexpr int kSfaOff = kStages * kStageBytes;   // activation scale atom (512 bytes), loaded once
constexpr int kBarOff = kSfaOff + 512;
constexpr int kSmem = kBarOff + 256 + 1024;
constexpr int kTmemCols = 512;
constexpr int kSfaCol = 256, kSfbCol = 264;      // TMEM: accumulator in columns 0..255, then the scale slots (12 columns per stage)
constexpr int kSfCols = 12;                      // per stage: 8 columns of weight scales, 4 of activation scales (inline mode)
constexpr int kThreads = 32 * 12;                // warp 0 weight copies, 1 MMA, 2..5 epilogue, 6..9 scales (+ inline activations), 10 activation copies, 11 scale-atom copies into TMEM
constexpr uint64_t kWaitLimitNs = 500000000ull;

__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int where) {
  return mbar_wait_bounded(bar, parity, abort_flag, kWaitLimitNs, where);
}
__device__ __forceinline__ void umma_mx(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t tsfa, uint32_t tsfb,
                                        uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(tsfa), "r"(tsfb) : "memory");
}

struct Params {
  const uint8_t* scales;      // [N][K/32] E8M0
  const __nv_bfloat16* x;     // [tokens][K] activations (read by the kernel itself in inline mode)
  const uint8_t* xq;          // pre-pass output: per K stage `rows` x 128 swizzled code bytes, then the 512-byte activation scale atom
  float* partials;            // [tile][slot][32 tokens][256]
  int32_t* counters;          // [tile], zero on entry and on exit
  void* out;
  int out_type;
  int tokens;
  int rows;                   // rows of the activation operand that hold token terms: 32 (<= 16 tokens) or 64
  int64_t N, K;
  int stages_per_tile;        // K / 128
  int units, per;             // work units in total and per CTA
  int max_slots;
  uint32_t idesc;
  int wait_first;             // 1: read nothing before the previous kernel of the stream has completed
  int debug;
  int32_t* status;
};

__device__ __forceinline__ int term_row(int t, int term) { return (t >> 4) * 32 + term * 16 + (t & 15); }

// ---------------------------------------------------------------------------
// Activation pre-pass: one CTA per token.  Pass 1 finds the token's largest magnitude (the row stays in registers),
// pass 2 writes both E4M3 terms of every value into the per-stage blocks (16-byte units XOR-swizzled by row & 7: the
// layout tcgen05.mma reads with the 128-byte swizzle) and the token's two entries of the scale atom
// (scale of row r: bytes (r % 32) * 16 + (r / 32) * 4 + 0..3, the same for the four K blocks of a stage).
// ---------------------------------------------------------------------------
constexpr int kPreThreads = 256;
constexpr int kPrePieces = 16;                     // 16-byte pieces a thread can hold: K <= 256 * 16 * 8 = 32768
__global__ void __launch_bounds__(kPreThreads) x_quant_token_kernel(const __nv_bfloat16* __restrict__ x, int tokens, int64_t K, int rows,
                                                                   uint8_t* __restrict__ xq) {
  __shared__ float s_max[kPreThreads / 32];
  const int t = blockIdx.x, tid = threadIdx.x;
  const int S = (int)(K / BK);
  // programmatic dependent launch on both sides (see the main kernel): the previous main grid may still be reading xq
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const int pieces = (int)(K / 8);
  uint4 v[kPrePieces];
  float amax = 0.0f;
#pragma unroll
  for (int i = 0; i < kPrePieces; ++i) {
    const int p = tid + i * kPreThreads;
    v[i] = make_uint4(0, 0, 0, 0);
    if (p < pieces) {
      v[i] = __ldg(reinterpret_cast<const uint4*>(x + (int64_t)t * K) + p);
      const uint32_t w[4] = {v[i].x, v[i].y, v[i].z, v[i].w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        amax = fmaxf(amax, fabsf(__uint_as_float(w[j] << 16)));
        amax = fmaxf(amax, fabsf(__uint_as_float(w[j] & 0xFFFF0000u)));
      }
    }
  }
  amax = warp_max(amax);
  if ((tid & 31) == 0) s_max[tid >> 5] = amax;
  __syncthreads();
  amax = s_max[0];
#pragma unroll
  for (int i = 1; i < kPreThreads / 32; ++i) amax = fmaxf(amax, s_max[i]);
  // exponent e: the smallest one with amax / 2^e <= 448 (= 1.75 * 2^8)
  const uint32_t ab = __float_as_uint(amax);
  int e = (int)((ab >> 23) & 0xFF) - 127 - 8 + ((ab & 0x007FFFFFu) > 0x00600000u ? 1 : 0);
  if (amax == 0.0f || !(amax <= 3.0e38f)) e = 0;               // empty row; inf/nan rows keep scale 1
  e = max(e, -127);
  const float inv = __uint_as_float((uint32_t)(127 - e) << 23);  // 2^-e
  const int r1 = term_row(t, 0), r2 = term_row(t, 1);
#pragma unroll
  for (int i = 0; i < kPrePieces; ++i) {
    const int p = tid + i * kPreThreads;
    if (p >= pieces) break;
    const uint32_t w[4] = {v[i].x, v[i].y, v[i].z, v[i].w};
    uint32_t c1[2], c2[2];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float q0 = __uint_as_float(w[j] << 16) * inv, q1 = __uint_as_float(w[j] & 0xFFFF0000u) * inv;   // exact (power-of-two scaling)
      const __nv_fp8x2_storage_t a = __nv_cvt_float2_to_fp8x2(make_float2(q0, q1), __NV_SATFINITE, __NV_E4M3);
      const __half2_raw hr = __nv_cvt_fp8x2_to_halfraw2(a, __NV_E4M3);
      const float2 back = __half22float2(*reinterpret_cast<const __half2*>(&hr));
      const __nv_fp8x2_storage_t b = __nv_cvt_float2_to_fp8x2(make_float2(q0 - back.x, q1 - back.y), __NV_SATFINITE, __NV_E4M3);
      if (j & 1) { c1[j >> 1] |= (uint32_t)a << 16; c2[j >> 1] |= (uint32_t)b << 16; }
      else       { c1[j >> 1] = (uint32_t)a;        c2[j >> 1] = (uint32_t)b; }
    }
    const int stage = p >> 4, piece = p & 15;
    uint8_t* blk = xq + (size_t)stage * rows * 128;
    *reinterpret_cast<uint2*>(blk + r1 * 128 + (((piece >> 1) ^ (r1 & 7)) << 4) + (piece & 1) * 8) = make_uint2(c1[0], c1[1]);
    *reinterpret_cast<uint2*>(blk + r2 * 128 + (((piece >> 1) ^ (r2 & 7)) << 4) + (piece & 1) * 8) = make_uint2(c2[0], c2[1]);
  }
  uint8_t* atom = xq + (size_t)S * rows * 128;
  if (tid == 0) {
    const uint32_t sb = (uint32_t)(e + 127) * 0x01010101u;
    *reinterpret_cast<uint32_t*>(atom + (r1 & 31) * 16 + (r1 >> 5) * 4) = sb;
    *reinterpret_cast<uint32_t*>(atom + (r2 & 31) * 16 + (r2 >> 5) * 4) = sb;
  }
  // Rows of the operand that belong to no token keep whatever the buffer held: an accumulator row depends on its own
  // operand row only, and the epilogue never reads the rows of tokens that do not exist.
}

// ---------------------------------------------------------------------------
// Main kernel
// ---------------------------------------------------------------------------
// INL (up to 4 tokens): no pre-pass.  The scale warps quantize the activations of their stage themselves, under one
// power-of-two scale per (token, stage), so the activation scale atom is per stage too.
template <bool INL>
__global__ void __launch_bounds__(kThreads, 1) gemv_fp4_mxb_kernel(const __grid_constant__ CUtensorMap map_w, const Params p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t bar_base = base + kBarOff;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (kStages + s); };
  auto sf_bar = [&](int s) { return bar_base + 8u * (2 * kStages + s); };     // scale atoms of the stage are in TMEM
  const uint32_t tfull_bar = bar_base + 8u * (3 * kStages), tempty_bar = tfull_bar + 8, sfa_bar = tfull_bar + 16, drain_bar = tfull_bar + 24;
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
    // a stage is full after: weight copy landed, activation copy landed, weight scale atoms written
    for (int s = 0; s < kStages; ++s) { mbar_init(full_bar(s), INL ? 2 : 3); mbar_init(empty_bar(s), 1); mbar_init(sf_bar(s), 1); }
    mbar_init(tfull_bar, 1); mbar_init(tempty_bar, 4); mbar_init(sfa_bar, 1); mbar_init(drain_bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_w)) : "memory");
    // the first round of weight copies needs nothing but the barriers: start the HBM stream before the rest of the prologue
    for (int it = 0; it < kStages && it < total; ++it) {
      const int u = u0 + it, tile = u / S, j = u - tile * S;
      mbar_expect_tx(full_bar(it), kBytesW / 2);             // the transaction count of a 4-bit box is the packed byte count
      tma_load_2d(base + it * kStageBytes, &map_w, full_bar(it), j * BK, tile * TILE_N);
    }
  }
  // rows of the activation operand past the token terms stay zero for the whole kernel
  for (int s = 0; s < kStages; ++s) {
    uint4* az = reinterpret_cast<uint4*>(base_ptr + s * kStageBytes + kBytesW + bytes_a);
    for (int k = threadIdx.x; k < (kBytesA - (int)bytes_a) / 16; k += kThreads) az[k] = make_uint4(0, 0, 0, 0);
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
    // ---------------- weight producer: one TMA copy (16 KiB from HBM) per stage ----------------
    if (lane == 0) {
      bool ok = true;
      for (int it = kStages; it < total; ++it) {                // the first round was issued in the prologue
        const int u = u0 + it, tile = u / S, j = u - tile * S;
        const int s = it % kStages;
        const uint32_t ph = (uint32_t)(it / kStages) & 1;
        if (!mbar_wait(empty_bar(s), ph ^ 1, abort_flag, 1)) { ok = false; break; }
        if (p.debug == 6) { mbar_arrive(full_bar(s)); continue; }   // timing experiment: no weight copies
        mbar_expect_tx(full_bar(s), kBytesW / 2);
        tma_load_2d(base + s * kStageBytes, &map_w, full_bar(s), j * BK, tile * TILE_N);
      }
      if (!ok || *abort_flag) {                                 // give the copies in flight time to land before shared memory is released
        const uint64_t t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 2000000ull) {}
      }
    }
  } else if (warp == 10) {
    // ---------------- activation producer (pre-pass mode): the scale atom once, then one bulk copy of the token rows per stage ----------------
    if (lane == 0 && !INL) {
      asm volatile("griddepcontrol.wait;" ::: "memory");        // the activations come from the pre-pass
      mbar_expect_tx(sfa_bar, 512);
      bulk_load(base + kSfaOff, p.xq + (size_t)S * bytes_a, 512, sfa_bar);
      for (int it = 0; it < total; ++it) {
        const int j = (u0 + it) % S;
        const int s = it % kStages;
        const uint32_t ph = (uint32_t)(it / kStages) & 1;
        if (!mbar_wait(empty_bar(s), ph ^ 1, abort_flag, 5)) break;
        mbar_expect_tx(full_bar(s), bytes_a);
        bulk_load(base + s * kStageBytes + kBytesW, p.xq + (size_t)j * bytes_a, bytes_a, full_bar(s));
      }
    }
  } else if (warp >= 6 && warp < 10) {
    // ---------------- weight scale atoms: warp w owns ring slot w; lane l holds the scale word (4 blocks) of rows l + 32 i ----------------
    const int slot = warp - 6;
    const int64_t kblocks = p.K >> 5;
    constexpr int kRing = 3;                                     // stages of this warp loaded ahead into registers
    uint32_t q[kRing][8];
    auto load_scales = [&](int u, uint32_t (&dst)[8]) {
      const int tile = u / S, j = u - tile * S;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int64_t row = min((int64_t)tile * TILE_N + lane + 32 * i, p.N - 1);
        dst[i] = __ldg(reinterpret_cast<const uint32_t*>(p.scales + row * kblocks + j * 4));
      }
    };
    // inline activations: lane -> 16-byte piece pi of the stage (8 values) of token tb (and tb + 2)
    const int pi = lane & 15, tb = lane >> 4;
    uint4 xr[kRing][2];
    auto load_x = [&](int u, uint4 (&dst)[2]) {
      const int j = u % S;
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        const int t = tb + 2 * r;
        dst[r] = t < p.tokens ? __ldg(reinterpret_cast<const uint4*>(p.x + (int64_t)t * p.K + (int64_t)j * BK + pi * 8)) : make_uint4(0, 0, 0, 0);
      }
    };
#pragma unroll
    for (int r = 0; r < kRing; ++r)
      if (slot + kStages * r < total) load_scales(u0 + slot + kStages * r, q[r]);
    if constexpr (INL) {
      // the activations may come from the previous kernel of the stream (programmatic dependent launch): nothing of them
      // is read before it has completed; the weight scales above are static and were fetched early
      asm volatile("griddepcontrol.wait;" ::: "memory");
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
        const uint32_t ph = (uint32_t)(it / kStages) & 1;
        if (!mbar_wait(empty_bar(slot), ph ^ 1, abort_flag, 6)) { ok = false; break; }
        uint8_t* sa = base_ptr + slot * kStageBytes + kBytesW;
        uint8_t* sf = sa + kBytesA;
        *reinterpret_cast<uint4*>(sf + lane * 16) = make_uint4(q[r][0], q[r][1], q[r][2], q[r][3]);
        *reinterpret_cast<uint4*>(sf + 512 + lane * 16) = make_uint4(q[r][4], q[r][5], q[r][6], q[r][7]);
        if constexpr (INL) {
#pragma unroll
          for (int k = 0; k < 2; ++k) {
            const int t = tb + 2 * k;
            const uint32_t w[4] = {xr[r][k].x, xr[r][k].y, xr[r][k].z, xr[r][k].w};
            float f[8];
            float amax = 0.0f;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              f[2 * j] = __uint_as_float(w[j] << 16);
              f[2 * j + 1] = __uint_as_float(w[j] & 0xFFFF0000u);
              amax = fmaxf(amax, fmaxf(fabsf(f[2 * j]), fabsf(f[2 * j + 1])));
            }
#pragma unroll
            for (int o = 1; o < 16; o <<= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, o));   // the 16 lanes of one token
            const uint32_t ab = __float_as_uint(amax);
            int e = (int)((ab >> 23) & 0xFF) - 127 - 8 + ((ab & 0x007FFFFFu) > 0x00600000u ? 1 : 0);   // smallest e with amax / 2^e <= 448
            if (amax == 0.0f || !(amax <= 3.0e38f)) e = 0;
            e = max(e, -127);
            const float inv = __uint_as_float((uint32_t)(127 - e) << 23);
            uint32_t c1[2], c2[2];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const float q0 = f[2 * j] * inv, q1 = f[2 * j + 1] * inv;
              const __nv_fp8x2_storage_t a = __nv_cvt_float2_to_fp8x2(make_float2(q0, q1), __NV_SATFINITE, __NV_E4M3);
              const __half2_raw hr = __nv_cvt_fp8x2_to_halfraw2(a, __NV_E4M3);
              const float2 back = __half22float2(*reinterpret_cast<const __half2*>(&hr));
              const __nv_fp8x2_storage_t b = __nv_cvt_float2_to_fp8x2(make_float2(q0 - back.x, q1 - back.y), __NV_SATFINITE, __NV_E4M3);
              if (j & 1) { c1[j >> 1] |= (uint32_t)a << 16; c2[j >> 1] |= (uint32_t)b << 16; }
              else       { c1[j >> 1] = (uint32_t)a;        c2[j >> 1] = (uint32_t)b; }
            }
            if (t < p.tokens) {
              const int r1 = term_row(t, 0), r2 = term_row(t, 1);
              *reinterpret_cast<uint2*>(sa + r1 * 128 + (((pi >> 1) ^ (r1 & 7)) << 4) + (pi & 1) * 8) = make_uint2(c1[0], c1[1]);
              *reinterpret_cast<uint2*>(sa + r2 * 128 + (((pi >> 1) ^ (r2 & 7)) << 4) + (pi & 1) * 8) = make_uint2(c2[0], c2[1]);
              if (pi == 0) {
                const uint32_t sb = (uint32_t)(e + 127) * 0x01010101u;   // the same scale for the four K blocks of the stage
                *reinterpret_cast<uint32_t*>(sf + 1024 + (r1 & 31) * 16 + (r1 >> 5) * 4) = sb;
                *reinterpret_cast<uint32_t*>(sf + 1024 + (r2 & 31) * 16 + (r2 >> 5) * 4) = sb;
              }
            }
          }
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // read by tcgen05.cp / tcgen05.mma
        __syncwarp();
        if (lane == 0) mbar_arrive(full_bar(slot));
        if (it + kStages * kRing < total) {
          load_scales(u0 + it + kStages * kRing, q[r]);
          if constexpr (INL) load_x(u0 + it + kStages * kRing, xr[r]);
        }
      }
    }
  } else if (warp == 11) {
    // ---------------- scale atoms into TMEM, one stage ahead of the MMAs (a thread of its own: tcgen05.cp issued between
    // the MMAs of one thread would sit in their dependency chain) ----------------
    if (lane == 0) {
      bool ok = true;
      if constexpr (!INL) {
        ok = mbar_wait(sfa_bar, 0, abort_flag, 7);
        if (ok) {
          tc_fence_after();
          tmem_cp_sf(tmem_base + kSfaCol, make_desc_sf(base + kSfaOff));
        }
      }
      for (int it = 0; it < total && ok; ++it) {
        const int s = it % kStages;
        const uint32_t ph = (uint32_t)(it / kStages) & 1;
        if (!mbar_wait(full_bar(s), ph, abort_flag, 8)) break;
        tc_fence_after();
        const uint32_t ssf = base + s * kStageBytes + kBytesW + kBytesA;
        const uint32_t tsfb = tmem_base + kSfbCol + s * kSfCols;
        tmem_cp_sf(tsfb, make_desc_sf(ssf));
        tmem_cp_sf(tsfb + 4, make_desc_sf(ssf + 512));
        if constexpr (INL) tmem_cp_sf(tsfb + 8, make_desc_sf(ssf + 1024));
        tc_commit(sf_bar(s));                                    // arrives when the copies above (and the earlier ones) are done
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
          if (!mbar_wait(sf_bar(s), ph, abort_flag, 3)) { ok = false; break; }   // operands in shared memory, scales in TMEM
          tc_fence_after();
          const uint32_t sw = base + s * kStageBytes, sa = sw + kBytesW;
          const uint32_t tsfb = tmem_base + kSfbCol + s * kSfCols;
          const uint32_t tsfa = INL ? tsfb + 8 : tmem_base + kSfaCol;
          const uint64_t adesc = make_desc_sw128(sa), bdesc = make_desc_sw128(sw);
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            if (p.debug == 5) break;                             // timing experiment: no MMAs
            // K advance inside the swizzle atom: +32 bytes; weight scale byte k of the slot's columns
            umma_mx(tmem_base, adesc + (uint64_t)(2 * k), bdesc + (uint64_t)(2 * k), p.idesc | ((uint32_t)k << 4), tsfa, tsfb,
                    (uint32_t)((i | k) != 0));
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
    // ---------------- epilogue: lane quarter q holds the terms of tokens 16 q .. 16 q + 15 ----------------
    const int q = warp & 3;
    const int t = q * 16 + (lane & 15);                          // this lane's token (lanes 16..31 hold the second term)
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
      float* mine = p.partials + ((int64_t)tile * p.max_slots + slot) * (32 * TILE_N);
      if (has_rows) {
#pragma unroll 1
        for (int c = 0; c < TILE_N; c += 32) {
          uint32_t r[32];
          tmem_ld32(tmem_base + c + ((uint32_t)(q * 32) << 16), r);
          tmem_ld_wait();
          float v[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const float a = __uint_as_float(r[i]);
            v[i] = a + __shfl_xor_sync(0xFFFFFFFFu, a, 16);      // first term + residual term
          }
          if (lane < 16 && t < p.tokens) {
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
          __syncwarp();
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(tempty_bar);                   // the accumulator may be overwritten
      if (!whole && p.debug < 3) {                              // B2Q_MX_DEBUG=3/4: timing experiment without the partial-sum exchange
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (warp == 2 && lane == 0) {
          __threadfence();                                      // cumulative: the partial sums of all 128 threads (ordered by the barrier) before the arrival
          const int old = atomicAdd(p.counters + tile, 1);
          s_last = (old == nc - 1);
          if (old == nc - 1) p.counters[tile] = 0;              // every contributor has arrived: leave the counter zero
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (s_last) {
          __threadfence();
          // 128 threads: thread e covers columns e and e + 128 of the tile for every token, contributors in CTA order
          const float* all = p.partials + (int64_t)tile * p.max_slots * (32 * TILE_N);
          const int e = (warp - 2) * 32 + lane;
          for (int tk0 = 0; tk0 < p.tokens; tk0 += 8) {            // eight tokens at a time: their loads are independent
            float s0[8], s1[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) { s0[i] = 0.0f; s1[i] = 0.0f; }
            for (int cc = 0; cc < nc; ++cc) {
              float a0[8], a1[8];
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                const bool in = tk0 + i < p.tokens;
                a0[i] = in ? __ldcg(all + (int64_t)cc * (32 * TILE_N) + (tk0 + i) * TILE_N + e) : 0.0f;
                a1[i] = in ? __ldcg(all + (int64_t)cc * (32 * TILE_N) + (tk0 + i) * TILE_N + e + 128) : 0.0f;
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

  // ---------------- teardown ----------------
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
  // weight codes as a [N][K] tensor of 4-bit elements; a box is 128 codes x 256 rows and lands in shared memory
  // as 128-byte rows (8 data bytes + 8 pad bytes per 16 codes), 128-byte swizzle, zero fill past row N
  CUtensorMap map_w;
  cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)N};
  cuuint64_t strides[1] = {(cuuint64_t)(K / 2)};
  cuuint32_t box[2] = {128, (cuuint32_t)TILE_N};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(&map_w, CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN16B, 2, const_cast<uint8_t*>(codes), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) B2Q_FAIL(h, B2Q_ERR_CUDA, "cuTensorMapEncodeTiled (4-bit weights) failed with CUresult %d", (int)r);

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
  p.rows = tokens <= 16 ? 32 : 64;
  const size_t xq_bytes = align256((size_t)S * p.rows * 128 + 512);
  const size_t part_bytes = (size_t)tiles * p.max_slots * 32 * TILE_N * sizeof(float);
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
  // block-scaled instruction descriptor: A = E4M3 (0) activations, B = E2M1 (5) weights, both K-major, N = 256, E8M0 scales, M = 128
  p.idesc = (0u << 7) | (5u << 10) | ((uint32_t)(TILE_N >> 3) << 17) | (1u << 23) | ((uint32_t)(128 >> 4) << 24);
  p.wait_first = h->dynamic_weights;
  if (h->sw.mx_debug > 0) p.debug = h->sw.mx_debug;
  p.status = h->d_status;

  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  const int num_attrs = h->sw.mx_pdl == 0 ? 0 : 1;
  cudaLaunchConfig_t pre = {};
  pre.gridDim = dim3((unsigned)tokens);
  pre.blockDim = dim3(kPreThreads);
  pre.stream = h->stream;
  pre.attrs = attr;
  pre.numAttrs = num_attrs;
  const bool inl = tokens <= 4 && h->sw.mx_inline != 0;         // B2Q_MX_INLINE=0 keeps the pre-pass for every token count
  if (!inl && p.debug != 2 && p.debug != 4)   // B2Q_MX_DEBUG=2/4: timing experiment without the pre-pass (results are then stale)
    B2Q_CUDA(h, cudaLaunchKernelEx(&pre, x_quant_token_kernel, (const __nv_bfloat16*)x, tokens, K, p.rows, reinterpret_cast<uint8_t*>(ws)));
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)grid);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = kSmem;
  cfg.stream = h->stream;
  cfg.attrs = attr;
  cfg.numAttrs = num_attrs;
  if (inl) {
    B2Q_SMEM_ATTR(h, gemv_fp4_mxb_kernel<true>, kSmem);
    B2Q_CUDA(h, cudaLaunchKernelEx(&cfg, gemv_fp4_mxb_kernel<true>, map_w, p));
  } else {
    B2Q_SMEM_ATTR(h, gemv_fp4_mxb_kernel<false>, kSmem);
    B2Q_CUDA(h, cudaLaunchKernelEx(&cfg, gemv_fp4_mxb_kernel<false>, map_w, p));
  }
  return B2Q_OK;
}

}  // namespace mxb

// Tensor-core FP4 decode GEMV with the weights as the N = 256 operand; B2Q_ERR_UNSUPPORTED (nothing launched) when the
// shape or the alignment does not fit: K % 128, K <= 32768, codes 32-byte aligned, scales 4-byte aligned, tokens <= 32.
int32_t b2q_gemv_fp4_mxb_dispatch(b2q_handle h, const uint8_t* codes, const void* scales, const void* x, int tokens, int64_t N, int64_t K,
                                  void* out, int out_type) {
  if (tokens < 1 || tokens > 32 || K % 128 != 0 || K > 32768 || N < 1) return B2Q_ERR_UNSUPPORTED;
  if ((reinterpret_cast<uintptr_t>(codes) & 31) != 0 || (reinterpret_cast<uintptr_t>(scales) & 3) != 0 ||
      (reinterpret_cast<uintptr_t>(x) & 15) != 0 || (K / 2) % 16 != 0)
    return B2Q_ERR_UNSUPPORTED;
  const int64_t tiles = ceil_div64(N, mxb::TILE_N);
  if (tiles > (int64_t)kTileCounters || tiles * (K / mxb::BK) > 0x7FFFFFFF) return B2Q_ERR_UNSUPPORTED;
  return mxb::launch(h, codes, (const uint8_t*)scales, x, tokens, N, K, out, out_type);
}
