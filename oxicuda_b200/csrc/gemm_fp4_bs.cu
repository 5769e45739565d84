// Block-scaled FP4 prefill GEMM on tcgen05.mma kind::mxf8f6f4.block_scale:
//   out[t, n] = sum_k x[t, k] * decode(codes[n, k]) * 2^(scale[n, k / 32] - 127)
// Fp4GemmConfig / generate_fp4_gemm_ptx (crates/oxicuda-blas/src/precision/fp4_fp6_ops.rs:337-395, :1237-1362) with the
// defined semantics dequantize_fp4 (:879-897) followed by a matmul.  The E2M1 weight codes and their E8M0 block scales
// feed the tensor core as stored: TMA expands the packed nibbles into the padded layout the instruction reads, the
// scales travel shared memory -> TMEM with tcgen05.cp, and no weight is ever expanded in HBM.
//
// Operands of one MMA: A = 128 activation rows x 32 K of E4M3 codes with one E8M0 scale per (row, 32-block),
// B = 256 weight rows x 32 K of E2M1 codes (N = 256: the instruction occupies the tensor pipe for ~171 clocks at N = 256
// against ~123 at N <= 128, so wide N is what the pipe rewards), D = [128 x 256] fp32 in TMEM.
// Activation modes (the pre-pass writes the codes and the scale atoms):
//   B2Q_FP4_ACT_SPLIT  every bf16 activation is the sum of TWO E4M3 codes under its block's power-of-two scale
//                      (exact to 2^-18 of the block maximum): weight-only semantics; a 128-row tile holds 64 tokens,
//                      row (t / 16) * 32 + term * 16 + t % 16, and the epilogue adds the two rows with one shuffle;
//   B2Q_FP4_ACT_MXFP8  one E4M3 code per activation (the MX W4A8 recipe): a tile holds 128 tokens, twice the rate;
//                      the result is that of the quantized activations (its oracle quantizes them the same way).
// One persistent CTA per SM over (128-row, 256-column) output tiles, whole K per tile, 4 stages of 128 K.
#include "tc_common.cuh"
#include <stdlib.h>

namespace f4bs {

using namespace tcx;

constexpr int TILE_M = 128, TILE_N = 256, BK = 128, kStages = 4;
constexpr int kBytesW = TILE_N * 128, kBytesA = TILE_M * 128, kBytesSf = 2048;   // scale atoms: weights 0..127, 128..255, activations
constexpr int kStageBytes = kBytesW + kBytesA + kBytesSf;
constexpr int kBarOff = kStages * kStageBytes;
constexpr int kSmem = kBarOff + 256 + 1024;
constexpr int kTmemCols = 512, kSfCol = 256, kSfCols = 12;
constexpr int kThreads = 32 * 11;   // warp 0 TMA (weights + activations), 1 MMA, 2..5 epilogue, 6..9 weight scales, 10 scale-atom copies into TMEM
constexpr uint64_t kWaitLimitNs = 2000000000ull;

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
  const uint8_t* scales;      // weights: [N][K/32] E8M0
  const uint8_t* xsf;         // activations: per (row tile, K stage) one 512-byte scale atom
  void* out;
  int out_type;
  int split;                  // 1: two-term rows (64 tokens per tile), 0: one row per token
  int64_t tokens, N, K;
  int tiles_m, tiles_n, stages_per_tile;
  uint32_t idesc;
  int32_t* status;
  // grouped mode (tile_group != null): row tile mt multiplies with the weights of problem tile_group[mt], rows
  // [g * N, (g + 1) * N) of the stacked codes and scales; the output stays [rows x N]
  const int32_t* tile_group;
};

// Activation pre-pass.  One CTA per (row tile, K stage): 128 K values of up to 128 / 64 tokens -> E4M3 codes in the
// activation matrix xq [tiles_m * 128][K] (plain row-major: the TMA load swizzles) and the stage's scale atom
// (scale of row r, block j at byte (r % 32) * 16 + (r / 32) * 4 + j).  Four lanes share a 32-block.
template <bool SPLIT>
__global__ void __launch_bounds__(512) x_quant_tile_kernel(const __nv_bfloat16* __restrict__ x, int64_t tokens, int64_t K, uint8_t* __restrict__ xq,
                                                           uint8_t* __restrict__ xsf) {
  __shared__ uint32_t sf[128];
  const int64_t mt = blockIdx.y, kb = blockIdx.x;
  const int S = gridDim.x;
  constexpr int TOK = SPLIT ? 64 : 128;                        // tokens per tile
  if (threadIdx.x < 128) sf[threadIdx.x] = 0x7F7F7F7Fu;
  __syncthreads();
  for (int it = threadIdx.x; it < TOK * 16; it += 512) {       // (token, 16-byte piece): the four lanes of a block are adjacent
    const int tl = it >> 4, i = it & 15;
    const int64_t t = mt * TOK + tl;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (t < tokens) v = __ldg(reinterpret_cast<const uint4*>(x + t * K + kb * BK + i * 8));
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
    float f[8];
    float amax = 0.0f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      f[2 * j] = __uint_as_float(w[j] << 16);
      f[2 * j + 1] = __uint_as_float(w[j] & 0xFFFF0000u);
      amax = fmaxf(amax, fmaxf(fabsf(f[2 * j]), fabsf(f[2 * j + 1])));
    }
    amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 2));
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
    const int r1 = SPLIT ? (tl >> 4) * 32 + (tl & 15) : tl, r2 = r1 + 16;
    uint8_t* row1 = xq + (mt * TILE_M + r1) * K + kb * BK + i * 8;
    *reinterpret_cast<uint2*>(row1) = make_uint2(c1[0], c1[1]);
    if (SPLIT) *reinterpret_cast<uint2*>(row1 + 16 * K) = make_uint2(c2[0], c2[1]);
    if ((i & 3) == 0) {
      uint8_t* sfb = reinterpret_cast<uint8_t*>(sf);
      sfb[(r1 & 31) * 16 + (r1 >> 5) * 4 + (i >> 2)] = (uint8_t)(e + 127);
      if (SPLIT) sfb[(r2 & 31) * 16 + (r2 >> 5) * 4 + (i >> 2)] = (uint8_t)(e + 127);
    }
  }
  __syncthreads();
  if (threadIdx.x < 128) reinterpret_cast<uint32_t*>(xsf + (mt * S + kb) * 512)[threadIdx.x] = sf[threadIdx.x];
}

__global__ void __launch_bounds__(kThreads, 1) gemm_fp4_bs_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_a,
                                                                  const Params p) {
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

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int S = p.stages_per_tile;
  const int total_tiles = p.tiles_m * p.tiles_n;
  // tiles in column-major order of the tile grid: consecutive CTAs share a weight panel (L2) and differ in the row tile
  auto tile_mn = [&](int tile, int& mt, int& nt) { nt = tile / p.tiles_m; mt = tile - nt * p.tiles_m; };

  if (threadIdx.x == 0) {
    s_abort = 0;
    // a stage is full after: the TMA bytes (weights, activations, activation scale atom) landed and the weight scale atoms are written
    for (int s = 0; s < kStages; ++s) { mbar_init(full_bar(s), 2); mbar_init(empty_bar(s), 1); mbar_init(sf_bar(s), 1); }
    mbar_init(tfull_bar, 1); mbar_init(tempty_bar, 4); mbar_init(drain_bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_w)) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_a)) : "memory");
  }
  if (warp == 1) tmem_alloc(smem_u32(&s_tmem_base), kTmemCols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = s_tmem_base;
  volatile int* abort_flag = &s_abort;

  if (warp == 0) {
    // ---------------- TMA producer: weights (16 KiB from HBM), activation codes (16 KiB) and their scale atom per stage ----------------
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
        int mt, nt;
        tile_mn(tile, mt, nt);
        for (int j = 0; j < S; ++j, ++it) {
          const int s = it % kStages;
          const uint32_t ph = (it / kStages) & 1;
          if (!mbar_wait(empty_bar(s), ph ^ 1, abort_flag, 1)) { ok = false; break; }
          const uint32_t sw = base + s * kStageBytes;
          mbar_expect_tx(full_bar(s), kBytesW / 2 + kBytesA + 512);   // the transaction count of a 4-bit box is the packed byte count
          tma_load_2d(sw, &map_w, full_bar(s), j * BK, nt * TILE_N + (p.tile_group ? __ldg(p.tile_group + mt) * (int)p.N : 0));
          tma_load_2d(sw + kBytesW, &map_a, full_bar(s), j * BK, mt * TILE_M);
          bulk_load(sw + kBytesW + kBytesA + 1024, p.xsf + ((size_t)mt * S + j) * 512, 512, full_bar(s));
        }
      }
      if (!ok || *abort_flag) {
        const uint64_t t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 2000000ull) {}
      }
    }
  } else if (warp >= 6 && warp < 10) {
    // ---------------- weight scale atoms: warp w owns ring slot w; lane l holds the scale word (4 blocks) of rows l + 32 i ----------------
    const int slot = warp - 6;
    const int64_t kblocks = p.K >> 5;
    uint32_t it = slot;
    bool ok = true;
    const int my_tiles = blockIdx.x < total_tiles ? (total_tiles - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;
    const uint32_t total = (uint32_t)my_tiles * S;
    uint32_t q[8], qn[8];
    auto load_scales = [&](uint32_t itx, uint32_t (&dst)[8]) {
      const int tile = blockIdx.x + (int)(itx / S) * gridDim.x, j = (int)(itx % S);
      int mt, nt;
      tile_mn(tile, mt, nt);
      const int64_t grow = p.tile_group ? (int64_t)__ldg(p.tile_group + mt) * p.N : 0;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int64_t row = grow + min((int64_t)nt * TILE_N + lane + 32 * i, p.N - 1);
        dst[i] = __ldg(reinterpret_cast<const uint32_t*>(p.scales + row * kblocks + j * 4));
      }
    };
    if (it < total) load_scales(it, q);
    for (; it < total && ok; it += kStages) {
      if (it + kStages < total) load_scales(it + kStages, qn);
      const uint32_t ph = (it / kStages) & 1;
      if (!mbar_wait(empty_bar(slot), ph ^ 1, abort_flag, 6)) { ok = false; break; }
      uint8_t* sf = base_ptr + slot * kStageBytes + kBytesW + kBytesA;
      *reinterpret_cast<uint4*>(sf + lane * 16) = make_uint4(q[0], q[1], q[2], q[3]);
      *reinterpret_cast<uint4*>(sf + 512 + lane * 16) = make_uint4(q[4], q[5], q[6], q[7]);
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(full_bar(slot));
#pragma unroll
      for (int i = 0; i < 8; ++i) q[i] = qn[i];
    }
  } else if (warp == 10) {
    // ---------------- scale atoms into TMEM, ahead of the MMAs ----------------
    if (lane == 0) {
      const int my_tiles = blockIdx.x < total_tiles ? (total_tiles - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;
      const uint32_t total = (uint32_t)my_tiles * S;
      for (uint32_t it = 0; it < total; ++it) {
        const int s = it % kStages;
        const uint32_t ph = (it / kStages) & 1;
        if (!mbar_wait(full_bar(s), ph, abort_flag, 8)) break;
        tc_fence_after();
        const uint32_t ssf = base + s * kStageBytes + kBytesW + kBytesA;
        const uint32_t tsf = tmem_base + kSfCol + s * kSfCols;
        tmem_cp_sf(tsf, make_desc_sf(ssf));
        tmem_cp_sf(tsf + 4, make_desc_sf(ssf + 512));
        tmem_cp_sf(tsf + 8, make_desc_sf(ssf + 1024));
        tc_commit(sf_bar(s));
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      uint32_t it = 0, tile_it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++tile_it) {
        if (!mbar_wait(tempty_bar, (tile_it & 1) ^ 1, abort_flag, 2)) { ok = false; break; }
        tc_fence_after();
        for (int j = 0; j < S; ++j, ++it) {
          const int s = it % kStages;
          const uint32_t ph = (it / kStages) & 1;
          if (!mbar_wait(sf_bar(s), ph, abort_flag, 3)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sw = base + s * kStageBytes, sa = sw + kBytesW;
          const uint32_t tsfb = tmem_base + kSfCol + s * kSfCols, tsfa = tsfb + 8;
          const uint64_t adesc = make_desc_sw128(sa), bdesc = make_desc_sw128(sw);
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma_mx(tmem_base, adesc + (uint64_t)(2 * k), bdesc + (uint64_t)(2 * k), p.idesc | ((uint32_t)k << 29) | ((uint32_t)k << 4), tsfa, tsfb,
                    (uint32_t)((j | k) != 0));
          tc_commit(empty_bar(s));
        }
        if (ok) tc_commit(tfull_bar);
      }
      if (!ok) {
        tc_commit(drain_bar);
        const uint64_t t0 = globaltimer_ns();
        while (!mbar_try_wait(drain_bar, 0))
          if (globaltimer_ns() - t0 > 100000000ull) break;
      }
    }
  } else if (warp >= 2 && warp < 6) {
    // ---------------- epilogue ----------------
    const int q = warp & 3;
    uint32_t tile_it = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++tile_it) {
      int mt, nt;
      tile_mn(tile, mt, nt);
      if (!mbar_wait(tfull_bar, tile_it & 1, abort_flag, 4)) { ok = false; break; }
      tc_fence_after();
      const int64_t n0 = (int64_t)nt * TILE_N;
      // two-term rows: lane l < 16 of quarter q holds token 64 mt + 16 q + l (the residual term sits 16 lanes up)
      const int64_t t = p.split ? (int64_t)mt * 64 + q * 16 + (lane & 15) : (int64_t)mt * TILE_M + q * 32 + lane;
      const bool writer = p.split ? lane < 16 : true;
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
          v[i] = p.split ? a + __shfl_xor_sync(0xFFFFFFFFu, a, 16) : a;
        }
        if (!writer || t >= p.tokens || n0 + c >= p.N) continue;
        if (p.out_type == B2Q_OUT_BF16) {
          __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(p.out) + t * p.N + n0 + c;
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
          float* o = reinterpret_cast<float*>(p.out) + t * p.N + n0 + c;
#pragma unroll
          for (int i = 0; i < 32; ++i) if (n0 + c + i < p.N) o[i] = v[i];
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(tempty_bar);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
  if (threadIdx.x == 0 && s_abort) atomicCAS(p.status, 0, (int)B2Q_ERR_TIMEOUT);
}

static inline size_t align256(size_t v) { return (v + 255) & ~(size_t)255; }

// group of every row tile: the problem whose padded row range holds the tile's first row (ranges start at multiples of
// 256 rows and are whole tiles); tiles behind the last range take the last problem (their rows are never read back)
__global__ void __launch_bounds__(256) tile_group_kernel(const int32_t* __restrict__ offsets, int groups, int tiles_m, int rows_per_tile,
                                                         int32_t* __restrict__ tile_group) {
  for (int mt = blockIdx.x * blockDim.x + threadIdx.x; mt < tiles_m; mt += gridDim.x * blockDim.x) {
    const int row = mt * rows_per_tile;
    int g = 0;
    while (g + 1 < groups && row >= offsets[g + 1]) ++g;
    tile_group[mt] = g;
  }
}

}  // namespace f4bs

static int32_t gemm_fp4_bs_impl(b2q_handle h, const uint8_t* codes, const uint8_t* scales_e8m0, const void* x_bf16, int64_t tokens, int64_t N,
                                int64_t K, int act_mode, void* out, int out_type, const int32_t* row_offsets, int groups);

extern "C" int32_t b2q_gemm_fp4_blockscaled(b2q_handle h, const uint8_t* codes, const uint8_t* scales_e8m0, const void* x_bf16, int64_t tokens,
                                            int64_t N, int64_t K, int act_mode, void* out, int out_type) {
  B2Q_REQUIRE_HANDLE(h);
  return gemm_fp4_bs_impl(h, codes, scales_e8m0, x_bf16, tokens, N, K, act_mode, out, out_type, nullptr, 0);
}

// Grouped form (the expert GEMMs of a mixture-of-experts layer in ONE launch, table on the device): problem g multiplies
// rows [row_offsets[g], row_offsets[g + 1]) of x (offsets are multiples of 256; rows behind a problem's real count are
// padding and are computed like any other) with the weights [g * N, (g + 1) * N) of the stacked codes and scales.
extern "C" int32_t b2q_grouped_gemm_fp4_rows(b2q_handle h, const uint8_t* codes, const uint8_t* scales_e8m0, const void* x_bf16,
                                             const int32_t* row_offsets, int groups, int64_t capacity_rows, int64_t N, int64_t K, int act_mode,
                                             void* out, int out_type) {
  B2Q_REQUIRE_HANDLE(h);
  if (groups <= 0 || !row_offsets) B2Q_FAIL(h, B2Q_ERR_INVALID_ARGUMENT, "grouped_gemm_fp4_rows: bad problem table");
  if ((int64_t)groups * N > 0x7FFFFFFF) B2Q_FAIL(h, B2Q_ERR_UNSUPPORTED, "grouped_gemm_fp4_rows: too many weight rows");
  return gemm_fp4_bs_impl(h, codes, scales_e8m0, x_bf16, capacity_rows, N, K, act_mode, out, out_type, row_offsets, groups);
}

static int32_t gemm_fp4_bs_impl(b2q_handle h, const uint8_t* codes, const uint8_t* scales_e8m0, const void* x_bf16, int64_t tokens, int64_t N,
                                int64_t K, int act_mode, void* out, int out_type, const int32_t* row_offsets, int groups) {
  using namespace f4bs;
  if (tokens <= 0 || N <= 0 || K <= 0)
    B2Q_FAIL(h, B2Q_ERR_INVALID_DIMENSION, "FP4 GEMM dimensions must be non-zero: m=%lld, n=%lld, k=%lld", (long long)N, (long long)tokens, (long long)K);
  if (K % 2 != 0) B2Q_FAIL(h, B2Q_ERR_INVALID_DIMENSION, "FP4 GEMM K dimension must be even for packing, got k=%lld", (long long)K);
  if (!codes || !scales_e8m0 || !x_bf16 || !out || act_mode < 0 || act_mode > 1 || out_type < 0 || out_type > 1)
    B2Q_FAIL(h, B2Q_ERR_INVALID_ARGUMENT, "gemm_fp4_blockscaled: bad argument");
  if (K % 128 != 0) B2Q_FAIL(h, B2Q_ERR_UNSUPPORTED, "gemm_fp4_blockscaled: K must be a multiple of 128, got %lld", (long long)K);
  if ((reinterpret_cast<uintptr_t>(codes) & 31) != 0 || (reinterpret_cast<uintptr_t>(scales_e8m0) & 3) != 0 ||
      (reinterpret_cast<uintptr_t>(x_bf16) & 15) != 0)
    B2Q_FAIL(h, B2Q_ERR_INVALID_ARGUMENT, "gemm_fp4_blockscaled: codes must be 32-byte, scales 4-byte and activations 16-byte aligned");
  const bool split = act_mode == B2Q_FP4_ACT_SPLIT;
  const int tok_per_tile = split ? 64 : 128;
  const int64_t tiles_m = ceil_div64(tokens, tok_per_tile), tiles_n = ceil_div64(N, TILE_N);
  if (tiles_m * tiles_n > 0x7FFFFFFF) B2Q_FAIL(h, B2Q_ERR_UNSUPPORTED, "gemm_fp4_blockscaled: too many tiles");
  const int S = (int)(K / BK);
  // workspace: activation codes [tiles_m * 128][K] and the scale atoms [tiles_m][S][512]
  const size_t xq_bytes = align256((size_t)tiles_m * TILE_M * K), sf_bytes = align256((size_t)tiles_m * S * 512);
  void* ws = nullptr;
  int32_t st = b2q_workspace(h, xq_bytes + sf_bytes + (groups > 0 ? (size_t)tiles_m * 4 : 0), &ws);
  if (st != B2Q_OK) return st;
  uint8_t* xq = reinterpret_cast<uint8_t*>(ws);
  uint8_t* xsf = xq + xq_bytes;
  int32_t* tile_group = nullptr;
  if (groups > 0) {
    tile_group = reinterpret_cast<int32_t*>(xsf + sf_bytes);
    tile_group_kernel<<<(int)ceil_div64(tiles_m, 256), 256, 0, h->stream>>>(row_offsets, groups, (int)tiles_m, tok_per_tile, tile_group);
    B2Q_LAUNCH_CHECK(h, "tile_group_kernel");
  }
  dim3 pg((unsigned)S, (unsigned)tiles_m);
  if (split) x_quant_tile_kernel<true><<<pg, 512, 0, h->stream>>>((const __nv_bfloat16*)x_bf16, tokens, K, xq, xsf);
  else x_quant_tile_kernel<false><<<pg, 512, 0, h->stream>>>((const __nv_bfloat16*)x_bf16, tokens, K, xq, xsf);
  B2Q_LAUNCH_CHECK(h, "x_quant_tile_kernel");

  EncodeTiledFn enc = get_encode_fn();
  if (!enc) B2Q_FAIL(h, B2Q_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  CUtensorMap map_w, map_a;
  cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)(groups > 0 ? (int64_t)groups * N : N)};
  cuuint64_t strides[1] = {(cuuint64_t)(K / 2)};
  cuuint32_t box[2] = {128, (cuuint32_t)TILE_N};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(&map_w, CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN16B, 2, const_cast<uint8_t*>(codes), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) B2Q_FAIL(h, B2Q_ERR_CUDA, "cuTensorMapEncodeTiled (4-bit weights) failed with CUresult %d", (int)r);
  st = b2q_tensor_map_2d(h, &map_a, xq, 1, (uint64_t)K, (uint64_t)(tiles_m * TILE_M), 128u, (uint32_t)TILE_M);
  if (st != B2Q_OK) return st;

  Params p = {};
  p.scales = scales_e8m0; p.xsf = xsf; p.out = out; p.out_type = out_type; p.split = split ? 1 : 0;
  p.tokens = tokens; p.N = N; p.K = K;
  p.tiles_m = (int)tiles_m; p.tiles_n = (int)tiles_n; p.stages_per_tile = S;
  // A = E4M3 (0) activations, B = E2M1 (5) weights, both K-major, N = 256, E8M0 scales, M = 128
  p.idesc = (0u << 7) | (5u << 10) | ((uint32_t)(TILE_N >> 3) << 17) | (1u << 23) | ((uint32_t)(TILE_M >> 4) << 24);
  p.status = h->d_status;
  p.tile_group = tile_group;
  B2Q_SMEM_ATTR(h, gemm_fp4_bs_kernel, kSmem);
  const int64_t tiles = tiles_m * tiles_n;
  const int grid = (int)(tiles < h->sm_count ? tiles : h->sm_count);
  gemm_fp4_bs_kernel<<<grid, kThreads, kSmem, h->stream>>>(map_w, map_a, p);
  B2Q_LAUNCH_CHECK(h, "gemm_fp4_bs_kernel");
  return B2Q_OK;
}
