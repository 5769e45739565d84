// Block-scaled FP4 (E2M1 codes, E8M0 scale per 32) weight-only decode GEMV on the 5th-generation tensor
// cores: tcgen05.mma kind::mxf8f6f4.block_scale consumes the 4-bit codes and their block scales directly,
// so no CUDA core touches a weight.
//   out[t, n] = sum_k x[t, k] * decode(codes[n, k]) * 2^(scale[n, k / 32] - 127)          tokens <= 32
// (Fp4GemmConfig / MicroScalingQuantizer semantics, crates/oxicuda-blas/src/precision/fp4_fp6_ops.rs:337-395,
//  :879-897, with the weight-only bf16-activation contract of the decode GEMV.)
//
// Activations: the instruction takes 8-bit floats, so a small pre-pass writes every bf16 activation as the
// sum of TWO E4M3 codes under an E8M0 scale per (token, 32-block):  x = 2^e * (c1 + c2),  c1 = rn(x / 2^e),
// c2 = rn(x / 2^e - c1).  c2 is exact whenever |x| >= 2^-11 of its block's maximum (bf16 has 8 significant
// bits, c1 keeps 4 and the remainder fits in 4), below that the absolute error is < 2^-18 of the block maximum.
// The two codes are two accumulator columns of the same MMA (N = 2 * padded tokens) added in the epilogue.
//
// Main kernel: one persistent CTA per SM, a ring of 8 stages (128 weight rows x 128 K each).  A single thread can
// issue only one asynchronous copy per ~250 ns and one stage of tcgen05 work per ~270 ns (measured), far below an
// SM's share of the HBM stream, so every role is spread over several warps, and stage s always belongs to warp
// s % 4 of each role (fixed owners keep the parity waits on the stage barriers one phase apart at most):
//   weight warps (4)             per stage one TMA copy of 128 weight rows (4-bit data expanded by the TMA unit to the
//                                16-byte-aligned layout the MMA reads, 128-byte swizzle);
//   scale/activation warps (4)   the weight scales of the stage (16-byte loads, a register ring four stages ahead,
//                                written in the 32 x 16-byte scale-factor atom layout) and one bulk copy of the
//                                activation codes + their scale atom;
//   MMA threads (4; 2 above 16 tokens)  tcgen05.cp of both scale atoms into TMEM, four tcgen05.mma (K = 32 = one
//                                scale block each) into the thread's own accumulator, tcgen05.commit to release the stage;
//   epilogue warps (4)           tcgen05.ld of the accumulators, add them and the two activation terms, store.
// Pre-pass and main grid are chained by programmatic dependent launch: a grid's prologue, weight copies and scale
// loads overlap the previous grid's tail, only the activation copies wait for the pre-pass (griddepcontrol.wait),
// and the pre-pass waits for the previous main grid before it touches the shared code buffer.
// Work units are (128-row tile, K stage) pairs.  With at least 0.7 tiles per SM every CTA owns whole tiles; otherwise
// the units are split evenly over the SMs (stream-K): a CTA that owns only part of a tile's K range writes its partial
// sums to a workspace and the last CTA to arrive at the tile (a counter per tile) adds the partials in CTA order and
// stores, so results do not depend on arrival order.  Every mbarrier wait is bounded.
#include "tc_common.cuh"
#include <stdlib.h>

namespace mx {

constexpr int TILE_ROWS = 128;   // weight rows per tile = TMEM lanes
constexpr int BK = 128;          // K per stage
constexpr uint64_t kWaitLimitNs = 500000000ull;

template <int MT> struct Cfg {
  static constexpr int MPAD = 8 * MT;
  static constexpr int NB = 2 * MPAD;                          // accumulator columns
  static constexpr int kBytesW = TILE_ROWS * 128;              // in shared memory (half of it crosses HBM)
  static constexpr int kBytesX = NB * 128 + 512;               // activation codes + activation scale atom
  static constexpr int kStageBytes = kBytesW + kBytesX + 512;  // + weight scale atom
  // One thread sustains about one asynchronous copy per 250 ns (measured: wait on the stage, expect_tx, issue), far
  // less than one SM's share of the HBM stream, so the copies of consecutive stages are issued by kWWarps weight
  // warps and kXWarps scale/activation warps in turn; with that one CTA per SM keeps the memory pipe full.
  // The stage count is a multiple of every role's warp count, so a stage is always filled and consumed by the same
  // warps: the parity waits on its barriers then never see a party more than one phase away (with a round-robin
  // that walks the ring, a warp running ahead of its siblings could mistake phase r-2 for phase r).
  static constexpr int kWWarps = 4;
  static constexpr int kXWarps = 4;
  static constexpr int kStages = 8;
  // Likewise one thread needs about 270 ns to issue the two tcgen05.cp, four tcgen05.mma and the commit of a stage, so
  // kMmaWarps threads issue the stages in turn, each into an accumulator of its own (added in the epilogue).
  static constexpr int kMmaWarps = MT == 4 ? 2 : 4;
  static constexpr int kSfCol = 2 * kMmaWarps * NB;             // TMEM: two buffers x kMmaWarps accumulators of NB columns, then an 8-column scale slot per stage
  static constexpr int kTmemCols = MT == 1 ? 256 : 512;
  // warp 0 (weights) + warp 1 (MMA) + 4 epilogue + scale/activation warps + extra weight warps + extra MMA warps
  static constexpr int kThreads = 32 * (6 + kXWarps + (kWWarps - 1) + (kMmaWarps - 1));
  static_assert(kStages % kWWarps == 0 && kStages % kXWarps == 0 && kStages % kMmaWarps == 0, "a stage must belong to one warp of each role");
  static constexpr int kSmem = kStages * kStageBytes + 1024 + 256;
};

struct Params {
  const uint8_t* scales;      // [N][K/32] E8M0
  const uint8_t* xq;          // per K stage: NB x 128 swizzled code bytes, then the 512-byte scale atom (pre-pass output)
  const __nv_bfloat16* x;     // [tokens][K] activations (read by the main kernel when it quantizes them itself)
  float* partials;            // [tile][slot][MPAD][128]
  int32_t* counters;          // [tile], zero on entry and on exit
  void* out;
  int out_type;
  int tokens;
  int64_t N, K;
  int stages_per_tile;        // K / 128
  int units, per;             // work units in total and per CTA
  int max_slots;
  uint32_t idesc;
  int wait_first;             // 1: read nothing before the previous kernel of the stream has completed
  int debug;                  // report which wait expired (status 400 + role) instead of B2Q_ERR_TIMEOUT
  int32_t* status;
};

using namespace tcx;
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int where = 1) {
  return mbar_wait_bounded(bar, parity, abort_flag, kWaitLimitNs, where);
}
__device__ __forceinline__ void umma_mx(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t tsfa, uint32_t tsfb,
                                        uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(tsfa), "r"(tsfb) : "memory");
}
// ---------------------------------------------------------------------------
// Activation pre-pass: bf16 [tokens x K] -> per K stage of 128 a block of NB rows x 128 bytes of E4M3 codes
// (rows 0..MPAD-1 first term, rows MPAD..2*MPAD-1 residual term; 16-byte units XOR-swizzled by row & 7, the
// layout tcgen05.mma reads with the 128-byte swizzle) followed by the 512-byte E8M0 scale atom
// (scale of row n, block j at byte (n % 32) * 16 + (n / 32) * 4 + j).  One CTA per stage, 16 threads per
// token row, 8 values per thread.
// ---------------------------------------------------------------------------
// Eight bf16 activations (one quarter of a 32-block; the four lanes of a block are consecutive) -> eight
// first-term and eight residual E4M3 codes; returns the block exponent e (scale byte e + 127).
// Warp-collective (two shuffles).
__device__ __forceinline__ int quant_piece(const uint4& v, uint32_t (&c1)[2], uint32_t (&c2)[2]) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
  float f[8];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    f[2 * j] = __uint_as_float(w[j] << 16);
    f[2 * j + 1] = __uint_as_float(w[j] & 0xFFFF0000u);
  }
  float amax = 0.0f;
#pragma unroll
  for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(f[j]));
  amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 1));
  amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 2));   // the four threads of one 32-block
  // block exponent e: the smallest one with amax / 2^e <= 448 (= 1.75 * 2^8)
  const uint32_t ab = __float_as_uint(amax);
  int e = (int)((ab >> 23) & 0xFF) - 127 - 8 + ((ab & 0x007FFFFFu) > 0x00600000u ? 1 : 0);
  if (amax == 0.0f || !(amax <= 3.0e38f)) e = 0;               // empty block; inf/nan blocks keep scale 1
  e = max(e, -127);
  const float inv = __uint_as_float((uint32_t)(127 - e) << 23);  // 2^-e, exponent field in [7, 254]
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float q0 = f[2 * j] * inv, q1 = f[2 * j + 1] * inv;  // exact (power-of-two scaling)
    const __nv_fp8x2_storage_t a = __nv_cvt_float2_to_fp8x2(make_float2(q0, q1), __NV_SATFINITE, __NV_E4M3);
    const __half2_raw hr = __nv_cvt_fp8x2_to_halfraw2(a, __NV_E4M3);
    const float2 back = __half22float2(*reinterpret_cast<const __half2*>(&hr));
    const __nv_fp8x2_storage_t b = __nv_cvt_float2_to_fp8x2(make_float2(q0 - back.x, q1 - back.y), __NV_SATFINITE, __NV_E4M3);
    if (j & 1) { c1[j >> 1] |= (uint32_t)a << 16; c2[j >> 1] |= (uint32_t)b << 16; }
    else       { c1[j >> 1] = (uint32_t)a;        c2[j >> 1] = (uint32_t)b; }
  }
  return e;
}

template <int MT>
__global__ void __launch_bounds__(128 * MT) x_quant_mx_kernel(const __nv_bfloat16* __restrict__ x, int tokens, int64_t K, uint8_t* __restrict__ xq) {
  using C = Cfg<MT>;
  __shared__ uint32_t sf[128];
  const int tid = threadIdx.x;
  const int i = tid & 15, t = tid >> 4;                        // 16-byte piece of the stage, token row
  const int64_t kb = blockIdx.x;
  // Programmatic dependent launch on both sides: the main kernel may start now (it waits for this grid only
  // where it reads the codes written here), and this grid may itself have started before the previous kernel
  // of the stream finished, so it waits for that kernel before it reads the activations or overwrites the
  // code buffer the previous GEMV may still be reading.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  if (tid < 128) sf[tid] = 0;
  __syncthreads();

  uint4 v = make_uint4(0, 0, 0, 0);
  if (t < tokens) v = __ldg(reinterpret_cast<const uint4*>(x + (int64_t)t * K + kb * BK + i * 8));
  uint32_t c1[2], c2[2];
  const int e = quant_piece(v, c1, c2);
  uint8_t* blk = xq + kb * C::kBytesX;
  const int n1 = t, n2 = C::MPAD + t;
  *reinterpret_cast<uint2*>(blk + n1 * 128 + (((i >> 1) ^ (n1 & 7)) << 4) + (i & 1) * 8) = make_uint2(c1[0], c1[1]);
  *reinterpret_cast<uint2*>(blk + n2 * 128 + (((i >> 1) ^ (n2 & 7)) << 4) + (i & 1) * 8) = make_uint2(c2[0], c2[1]);
  if ((i & 3) == 0) {
    uint8_t* sfb = reinterpret_cast<uint8_t*>(sf);
    const uint8_t sb = (uint8_t)(e + 127);
    sfb[(n1 & 31) * 16 + (n1 >> 5) * 4 + (i >> 2)] = sb;
    sfb[(n2 & 31) * 16 + (n2 >> 5) * 4 + (i >> 2)] = sb;
  }
  __syncthreads();
  if (tid < 128) reinterpret_cast<uint32_t*>(blk + C::NB * 128)[tid] = sf[tid];
}

// ---------------------------------------------------------------------------
// Main kernel
// ---------------------------------------------------------------------------

// INL (up to 4 tokens): the scale/activation warps quantize the activations of each stage themselves, no pre-pass.
template <int MT, bool INL>
__global__ void __launch_bounds__(Cfg<MT>::kThreads, 1) gemv_fp4_mx_kernel(const __grid_constant__ CUtensorMap map_w, const Params p) {
  using C = Cfg<MT>;
  constexpr int kStages = C::kStages;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t bar_base = base + kStages * C::kStageBytes;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (kStages + s); };
  auto tfull_bar = [&](int b) { return bar_base + 8u * (2 * kStages + b); };
  auto tempty_bar = [&](int b) { return bar_base + 8u * (2 * kStages + 2 + b); };
  const uint32_t drain_bar = bar_base + 8u * (2 * kStages + 4);
  __shared__ uint32_t s_tmem_base;
  __shared__ int s_abort;
  __shared__ int s_last;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int S = p.stages_per_tile;
  const int u0 = blockIdx.x * p.per, u1 = min(u0 + p.per, p.units);

  if (p.wait_first) asm volatile("griddepcontrol.wait;" ::: "memory");
  if (threadIdx.x == 0) {
    s_abort = 0;
    // a stage is full after: weight copy issued, (activation copy issued,) weight scale atom (and activation codes) written
    for (int s = 0; s < kStages; ++s) { mbar_init(full_bar(s), INL ? 2 : 3); mbar_init(empty_bar(s), 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(tfull_bar(b), C::kMmaWarps); mbar_init(tempty_bar(b), 4); }
    mbar_init(drain_bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_w)) : "memory");
    // the first round of weight copies needs nothing but the barriers: start the HBM stream before the rest of the prologue
    for (int it = 0; it < kStages && u0 + it < u1; ++it) {
      const int u = u0 + it, tile = u / S, j = u - tile * S;
      mbar_expect_tx(full_bar(it), C::kBytesW / 2);
      tma_load_2d(base + it * C::kStageBytes, &map_w, full_bar(it), j * BK, tile * TILE_ROWS);
    }
  }
  if (warp == 1) tmem_alloc(smem_u32(&s_tmem_base), C::kTmemCols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = s_tmem_base;
  volatile int* abort_flag = &s_abort;
  // the next kernel of the stream may be scheduled as SMs free up; whatever it reads of this grid's output it reads
  // after its own griddepcontrol.wait, i.e. after this grid has completed
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  const int w_idx = warp == 0 ? 0 : warp - (6 + C::kXWarps) + 1;   // weight warps: warp 0 and the warps after the scale/activation warps
  const int m_idx = warp == 1 ? 0 : warp - (6 + C::kXWarps + C::kWWarps - 1) + 1;   // MMA warps: warp 1 and the last warps
  if (warp == 0 || (warp >= 6 + C::kXWarps && warp < 6 + C::kXWarps + C::kWWarps - 1)) {
    // ---------------- weight producers: one TMA copy per stage, stages dealt round-robin to the weight warps ----------------
    if (lane == 0) {
      bool ok = true;
      const int total = u1 - u0;
      // the first round (kStages copies) was issued in the prologue by thread 0
      for (int it = kStages + ((w_idx - kStages % C::kWWarps + C::kWWarps) % C::kWWarps); it < total; it += C::kWWarps) {
        const int u = u0 + it, tile = u / S, j = u - tile * S;
        const int s = it % kStages;
        const uint32_t ph = (uint32_t)(it / kStages) & 1;
        if (!mbar_wait(empty_bar(s), ph ^ 1, abort_flag, 1)) { ok = false; break; }
        // the mbarrier counts the packed bytes read from global memory (64 per row), not the padded bytes written
        mbar_expect_tx(full_bar(s), C::kBytesW / 2);
        tma_load_2d(base + s * C::kStageBytes, &map_w, full_bar(s), j * BK, tile * TILE_ROWS);
      }
      if (!ok || *abort_flag) {
        // a wait expired somewhere: give the copies in flight time to land before shared memory is released
        const uint64_t t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 2000000ull) {}
      }
    }
  } else if (warp >= 6 && warp < 6 + C::kXWarps) {
    // ---------------- scale + activation producers (whole warps: every lane owns one 16-byte line of the weight scale atom),
    // stages dealt round-robin to the kXWarps warps ----------------
    const int x_idx = warp - 6;
    const int64_t kblocks = p.K >> 5;
    // A warp takes every fourth stage, so every stage it takes lies in a new 512-wide chunk of scale bytes.  The
    // chunks are read kRing stages of this warp ahead into a register ring with compile-time slot indices (a ring
    // that shifts its registers would wait for the newest load at every shift).
    static_assert(C::kXWarps == 4, "one chunk of scale bytes per stage of a warp");
    constexpr int kRing = 4;
    uint32_t q[kRing][4];                                      // the stage's scale word (4 blocks) of rows lane, lane+32, lane+64, lane+96
    const int total = u1 - u0;
    auto load_scales = [&](int u, uint32_t (&dst)[4]) {
      const int tile = u / S, j = u - tile * S;
#pragma unroll
      for (int r1 = 0; r1 < 4; ++r1) {
        const int64_t row = min((int64_t)tile * TILE_ROWS + lane + 32 * r1, p.N - 1);
        dst[r1] = __ldg(reinterpret_cast<const uint32_t*>(p.scales + row * kblocks + j * 4));
      }
    };
#pragma unroll
    for (int r = 0; r < kRing; ++r)
      if (x_idx + 4 * r < total) load_scales(u0 + x_idx + 4 * r, q[r]);
    // inline quantization: lane -> 16-byte piece i of the stage and token tb (+2 for the second piece)
    constexpr int kPieces = 2;                                 // tokens <= 4
    const int pi = lane & 15, tb = lane >> 4;
    uint4 xr[kRing][kPieces];
    auto load_x = [&](int u, uint4 (&dst)[kPieces]) {
      const int j = u % S;
#pragma unroll
      for (int r = 0; r < kPieces; ++r) {
        const int t = tb + 2 * r;
        dst[r] = t < p.tokens ? __ldg(reinterpret_cast<const uint4*>(p.x + (int64_t)t * p.K + (int64_t)j * BK + pi * 8)) : make_uint4(0, 0, 0, 0);
      }
    };
    if constexpr (INL) {
      // rows of the activation tile that belong to no token, and the unused part of its scale atom, stay zero: clear
      // this warp's stages once (a stage keeps its owner)
      for (int s = x_idx; s < kStages; s += C::kXWarps) {
        uint4* xz = reinterpret_cast<uint4*>(base_ptr + s * C::kStageBytes + C::kBytesW);
        for (int k = lane; k < C::kBytesX / 16; k += 32) xz[k] = make_uint4(0, 0, 0, 0);
      }
    }
    // the activations come from the previous kernel of the stream (the pre-pass, or whatever produced x), which this
    // grid may overlap (programmatic dependent launch): nothing of them is read before this point
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if constexpr (INL) {
#pragma unroll
      for (int r = 0; r < kRing; ++r)
        if (x_idx + 4 * r < total) load_x(u0 + x_idx + 4 * r, xr[r]);
    }
    bool ok = true;
    for (int it0 = x_idx; it0 < total && ok; it0 += 4 * kRing) {
#pragma unroll
      for (int r = 0; r < kRing; ++r) {
        const int it = it0 + 4 * r;
        if (it >= total) break;
        const int u = u0 + it;
        const int j = u % S;
        const int s = it % kStages;
        const uint32_t ph = (uint32_t)(it / kStages) & 1;
        if (!mbar_wait(empty_bar(s), ph ^ 1, abort_flag, 5)) { ok = false; break; }
        uint8_t* xs = base_ptr + s * C::kStageBytes + C::kBytesW;
        if constexpr (INL) {
#pragma unroll
          for (int k = 0; k < kPieces; ++k) {
            uint32_t c1[2], c2[2];
            const int e = quant_piece(xr[r][k], c1, c2);
            const int n1 = tb + 2 * k, n2 = C::MPAD + n1;
            if (n1 < p.tokens) {
              *reinterpret_cast<uint2*>(xs + n1 * 128 + (((pi >> 1) ^ (n1 & 7)) << 4) + (pi & 1) * 8) = make_uint2(c1[0], c1[1]);
              *reinterpret_cast<uint2*>(xs + n2 * 128 + (((pi >> 1) ^ (n2 & 7)) << 4) + (pi & 1) * 8) = make_uint2(c2[0], c2[1]);
              if ((pi & 3) == 0) {
                xs[C::NB * 128 + n1 * 16 + (pi >> 2)] = (uint8_t)(e + 127);
                xs[C::NB * 128 + n2 * 16 + (pi >> 2)] = (uint8_t)(e + 127);
              }
            }
          }
        } else if (lane == 0) {                                // the copy is in flight while the warp writes the scale atom
          mbar_expect_tx(full_bar(s), C::kBytesX);
          bulk_load(base + s * C::kStageBytes + C::kBytesW, p.xq + (int64_t)j * C::kBytesX, C::kBytesX, full_bar(s));
        }
        *reinterpret_cast<uint4*>(xs + C::kBytesX + lane * 16) = make_uint4(q[r][0], q[r][1], q[r][2], q[r][3]);
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // read by tcgen05.cp / tcgen05.mma
        __syncwarp();
        if (lane == 0) mbar_arrive(full_bar(s));
        if (it + 4 * kRing < total) {                          // this slot's next use
          load_scales(u + 4 * kRing, q[r]);
          if constexpr (INL) load_x(u + 4 * kRing, xr[r]);
        }
      }
    }
    // on a failed wait the weight warps hold the CTA until the copies in flight have landed
  } else if (warp == 1 || warp >= 6 + C::kXWarps + C::kWWarps - 1) {
    // ---------------- MMA issuers: thread m_idx takes the stages with ring position % kMmaWarps == m_idx ----------------
    if (lane == 0) {
      int it0 = 0;                                             // ring position of the segment's first stage
      uint32_t seg_it = 0;
      bool ok = true;
      for (int u = u0; u < u1 && ok; ++seg_it) {
        const int tile = u / S, j0 = u - tile * S;
        const int n = min(u1 - u, S - j0);
        const uint32_t buf = seg_it & 1, aph = (seg_it >> 1) & 1;
        if (!mbar_wait(tempty_bar(buf), aph ^ 1, abort_flag, 2)) { ok = false; break; }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + (buf * C::kMmaWarps + m_idx) * C::NB;
        bool first = true;
        for (int it = it0 + ((m_idx - it0 % C::kMmaWarps + C::kMmaWarps) % C::kMmaWarps); it < it0 + n; it += C::kMmaWarps) {
          const int s = it % kStages;
          const uint32_t ph = (uint32_t)(it / kStages) & 1;
          if (!mbar_wait(full_bar(s), ph, abort_flag, 3)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sw = base + s * C::kStageBytes, sx = sw + C::kBytesW;
          const uint32_t tsfa = tmem_base + C::kSfCol + s * 8, tsfb = tsfa + 4;
          tmem_cp_sf(tsfa, make_desc_sf(sx + C::kBytesX));
          tmem_cp_sf(tsfb, make_desc_sf(sx + C::NB * 128));
          const uint64_t adesc = make_desc_sw128(sw), bdesc = make_desc_sw128(sx);
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            // K advance inside the swizzle atom: +32 bytes; scale byte k of the atom's columns
            umma_mx(tmem_d, adesc + (uint64_t)(2 * k), bdesc + (uint64_t)(2 * k), p.idesc | ((uint32_t)k << 29) | ((uint32_t)k << 4),
                    tsfa, tsfb, (uint32_t)(!first || k != 0));
          }
          first = false;
          tc_commit(empty_bar(s));
        }
        if (ok) tc_commit(tfull_bar(buf));                     // arrives once this thread's MMAs of the segment are complete (at once if it had none)
        u += n;
        it0 += n;
      }
      if (!ok && m_idx == 0) {
        tc_commit(drain_bar);
        const uint64_t t0 = globaltimer_ns();
        while (!mbar_try_wait(drain_bar, 0))
          if (globaltimer_ns() - t0 > 100000000ull) break;
      }
    }
  } else {
    // ---------------- epilogue (warps 2..5) ----------------
    const int q = warp & 3;                                   // TMEM lane quarter this warp may access
    const int row_local = q * 32 + lane;
    int it0 = 0;
    uint32_t seg_it = 0;
    bool ok = true;
    for (int u = u0; u < u1 && ok; ++seg_it) {
      const int tile = u / S, j0 = u - tile * S;
      const int n = min(u1 - u, S - j0);
      u += n;
      const uint32_t buf = seg_it & 1, aph = (seg_it >> 1) & 1;
      if (!mbar_wait(tfull_bar(buf), aph, abort_flag, 4)) { ok = false; break; }
      tc_fence_after();
      float v[C::MPAD];
#pragma unroll
      for (int t = 0; t < C::MPAD; ++t) v[t] = 0.0f;
#pragma unroll
      for (int g = 0; g < C::kMmaWarps; ++g) {
        // accumulator g holds something only if MMA thread g had a stage in this segment
        const bool used = n >= C::kMmaWarps || ((g - it0 % C::kMmaWarps + C::kMmaWarps) % C::kMmaWarps) < n;
        if (used) {                                           // uniform over the warp
#pragma unroll
          for (int c = 0; c < C::NB; c += 16) {
            uint32_t r[16];
            tmem_ld16(tmem_base + (buf * C::kMmaWarps + g) * C::NB + c + ((uint32_t)(q * 32) << 16), r);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 16; ++i) v[(c + i) % C::MPAD] += __uint_as_float(r[i]);   // first term and residual term of a token
          }
        }
      }
      it0 += n;
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(tempty_bar(buf));            // accumulators are in registers now
      const int64_t row = (int64_t)tile * TILE_ROWS + row_local;
      auto store_out = [&](int t, float val) {
        if (row < p.N) {
          if (p.out_type == B2Q_OUT_BF16) reinterpret_cast<__nv_bfloat16*>(p.out)[(int64_t)t * p.N + row] = __float2bfloat16_rn(val);
          else reinterpret_cast<float*>(p.out)[(int64_t)t * p.N + row] = val;
        }
      };
      if (n == S) {                                           // this CTA owns the tile's whole K range
#pragma unroll
        for (int t = 0; t < C::MPAD; ++t) if (t < p.tokens) store_out(t, v[t]);
      } else {
        const int first = (tile * S) / p.per, last = (tile * S + S - 1) / p.per;
        const int nc = last - first + 1, slot = (int)blockIdx.x - first;
        float* mine = p.partials + ((int64_t)tile * p.max_slots + slot) * (C::MPAD * TILE_ROWS);
#pragma unroll
        for (int t = 0; t < C::MPAD; ++t) if (t < p.tokens) mine[t * TILE_ROWS + row_local] = v[t];
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (warp == 2 && lane == 0) {
          __threadfence();                                    // cumulative: the partial sums of all 128 threads (ordered by the barrier) before the arrival
          const int old = atomicAdd(p.counters + tile, 1);
          s_last = (old == nc - 1);
          if (old == nc - 1) p.counters[tile] = 0;            // every contributor has arrived: leave the counter zero
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (s_last) {
          __threadfence();
          const float* all = p.partials + (int64_t)tile * p.max_slots * (C::MPAD * TILE_ROWS);
          float sum[C::MPAD];
#pragma unroll
          for (int t = 0; t < C::MPAD; ++t) sum[t] = 0.0f;
          for (int c = 0; c < nc; ++c) {                      // contributors in CTA order; the loads of one contributor are independent
            float part[C::MPAD];
#pragma unroll
            for (int t = 0; t < C::MPAD; ++t)
              part[t] = t < p.tokens ? __ldcg(all + (int64_t)c * (C::MPAD * TILE_ROWS) + t * TILE_ROWS + row_local) : 0.0f;
#pragma unroll
            for (int t = 0; t < C::MPAD; ++t) sum[t] += part[t];
          }
#pragma unroll
          for (int t = 0; t < C::MPAD; ++t) if (t < p.tokens) store_out(t, sum[t]);
        }
      }
    }
  }

  // ---------------- teardown ----------------
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, C::kTmemCols);
  }
  if (threadIdx.x == 0 && s_abort) atomicCAS(p.status, 0, p.debug ? 400 + s_abort : (int)B2Q_ERR_TIMEOUT);
}

// ---- host side --------------------------------------------------------------
static inline size_t align256(size_t v) { return (v + 255) & ~(size_t)255; }

template <int MT, bool INL>
int32_t launch(b2q_handle h, const uint8_t* codes, const uint8_t* scales, const void* x, int tokens, int64_t N, int64_t K, void* out,
               int out_type) {
  using C = Cfg<MT>;
  EncodeTiledFn enc = get_encode_fn();
  if (!enc) B2Q_FAIL(h, B2Q_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  // weight codes as a [N][K] tensor of 4-bit elements; a box is 128 codes x 128 rows and lands in shared memory
  // as 128-byte rows (8 data bytes + 8 pad bytes per 16 codes), 128-byte swizzle, zero fill past row N
  CUtensorMap map_w;
  cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)N};
  cuuint64_t strides[1] = {(cuuint64_t)(K / 2)};
  cuuint32_t box[2] = {128, (cuuint32_t)TILE_ROWS};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(&map_w, CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN16B, 2, const_cast<uint8_t*>(codes), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) B2Q_FAIL(h, B2Q_ERR_CUDA, "cuTensorMapEncodeTiled (4-bit weights) failed with CUresult %d", (int)r);

  Params p = {};
  const int S = (int)(K / BK);
  const int64_t tiles = ceil_div64(N, TILE_ROWS);
  const int64_t units = tiles * S;
  const int64_t slots = h->sm_count;                            // one CTA per SM
  int grid, per;
  if (tiles * 10 >= slots * 7) {
    // enough tiles to occupy most SMs: every CTA owns whole tiles, no partial sums to exchange
    per = S * (int)ceil_div64(tiles, slots);
    grid = (int)ceil_div64(units, per);
  } else {
    grid = (int)(units < slots ? units : slots);
    per = (int)ceil_div64(units, grid);
    grid = (int)ceil_div64(units, per);
  }
  if (h->sw.mx_streamk == 1) {                                  // experiment switch: 1 forces the even split over all SMs
    { grid = (int)(units < slots ? units : slots); per = (int)ceil_div64(units, grid); grid = (int)ceil_div64(units, per); }
  }
  p.max_slots = (S + per - 1) / per + 1;
  const size_t xq_bytes = align256((size_t)S * C::kBytesX);
  const size_t part_bytes = (size_t)tiles * p.max_slots * C::MPAD * TILE_ROWS * sizeof(float);
  void* ws = nullptr;
  int32_t st = b2q_workspace(h, xq_bytes + part_bytes, &ws);
  if (st != B2Q_OK) return st;
  p.scales = scales;
  p.xq = reinterpret_cast<const uint8_t*>(ws);
  p.x = reinterpret_cast<const __nv_bfloat16*>(x);
  p.partials = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(ws) + xq_bytes);
  p.counters = h->d_tile_counters;
  p.out = out;
  p.out_type = out_type;
  p.tokens = tokens;
  p.N = N;
  p.K = K;
  p.stages_per_tile = S;
  p.units = (int)units;
  p.per = per;
  // block-scaled instruction descriptor: A = E2M1 (5), B = E4M3 (0), both K-major, N = NB, E8M0 scales, M = 128
  p.idesc = (5u << 7) | (0u << 10) | ((uint32_t)(C::NB >> 3) << 17) | (1u << 23) | ((uint32_t)(TILE_ROWS >> 4) << 24);
  p.wait_first = h->dynamic_weights;
  if (h->sw.mx_debug > 0) p.debug = h->sw.mx_debug;            // 1: report which wait expired as status 400 + role
  p.status = h->d_status;

  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  const int num_attrs = h->sw.mx_pdl == 0 ? 0 : 1;             // B2Q_MX_PDL=0: plain stream-ordered launches
  if (!INL) {
    cudaLaunchConfig_t pre = {};
    pre.gridDim = dim3((unsigned)S);
    pre.blockDim = dim3(128 * MT);
    pre.stream = h->stream;
    pre.attrs = attr;
    pre.numAttrs = num_attrs;
    B2Q_CUDA(h, cudaLaunchKernelEx(&pre, x_quant_mx_kernel<MT>, (const __nv_bfloat16*)x, tokens, K, reinterpret_cast<uint8_t*>(ws)));
  }
  B2Q_SMEM_ATTR(h, (gemv_fp4_mx_kernel<MT, INL>), C::kSmem);
  // programmatic dependent launch: this grid may start while the pre-pass runs; its activation loads wait for it
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)grid);
  cfg.blockDim = dim3(C::kThreads);
  cfg.dynamicSmemBytes = C::kSmem;
  cfg.stream = h->stream;
  cfg.attrs = attr;
  cfg.numAttrs = num_attrs;
  B2Q_CUDA(h, cudaLaunchKernelEx(&cfg, gemv_fp4_mx_kernel<MT, INL>, map_w, p));
  return B2Q_OK;
}

}  // namespace mx

// Tensor-core FP4 decode GEMV for E8M0 scales; B2Q_ERR_UNSUPPORTED (nothing launched) when the shape or the
// alignment does not fit: K % 512, codes 32-byte aligned, scales 16-byte aligned, tokens <= 32.
int32_t b2q_gemv_fp4_mx_dispatch(b2q_handle h, const uint8_t* codes, const void* scales, const void* x, int tokens, int64_t N, int64_t K,
                                 void* out, int out_type) {
  if (tokens < 1 || tokens > 32 || K % 512 != 0 || N < 1) return B2Q_ERR_UNSUPPORTED;
  if ((reinterpret_cast<uintptr_t>(codes) & 31) != 0 || (reinterpret_cast<uintptr_t>(scales) & 15) != 0 ||
      (reinterpret_cast<uintptr_t>(x) & 15) != 0)
    return B2Q_ERR_UNSUPPORTED;
  if (ceil_div64(N, mx::TILE_ROWS) > (int64_t)kTileCounters || ceil_div64(N, mx::TILE_ROWS) * (K / mx::BK) > 0x7FFFFFFF)
    return B2Q_ERR_UNSUPPORTED;
  if (tokens <= 4 && h->sw.mx_inline != 0)                     // B2Q_MX_INLINE=0 keeps the pre-pass for every token count
    return mx::launch<1, true>(h, codes, (const uint8_t*)scales, x, tokens, N, K, out, out_type);
  if (tokens <= 8) return mx::launch<1, false>(h, codes, (const uint8_t*)scales, x, tokens, N, K, out, out_type);
  if (tokens <= 16) return mx::launch<2, false>(h, codes, (const uint8_t*)scales, x, tokens, N, K, out, out_type);
  return mx::launch<4, false>(h, codes, (const uint8_t*)scales, x, tokens, N, K, out, out_type);
}
