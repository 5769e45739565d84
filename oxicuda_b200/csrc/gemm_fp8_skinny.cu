// FP8 (W8A8) GEMM for few tokens (M <= 128) on tcgen05: out[m, n] = (sum_k a[m,k] * w[n,k]) * scale_a * scale_w.
// The decode / small-batch branch of gemm::<E4M3> (the reference's Skinny category,
// crates/oxicuda-blas/src/level3/gemm/dispatch.rs:493-534, and its level-2 gemv,
// crates/oxicuda-blas/src/level2/gemv.rs:63-143).  The work is reading W once, so the kernel is shaped like the FP4
// decode GEMV (gemv_fp4_mx.cu), not like the prefill GEMM:
//   * the WEIGHTS are the M = 128 operand of tcgen05.mma.kind::f8f6f4 (128 weight rows x 32 K per instruction), the
//     activations the N operand (tokens padded to 16, 32, 64 or 128 columns), the accumulator [128 rows x tokens] lives
//     in TMEM; one 128-byte K slab of 128 rows (16 KiB from HBM) costs five tcgen05 instructions, well inside an SM's
//     share of the HBM stream;
//   * one persistent CTA per SM, a ring of 128-byte-swizzled stages; two warps issue the weight TMA copies (a stage
//     always belongs to the same warp), one warp the activation copies, one thread the MMAs, four warps the epilogue;
//   * (128-row tile, K stage) work units: whole tiles per CTA when at least 0.7 tiles per SM exist, else an even split
//     with partial sums in a workspace and an ordered fix-up by the last CTA to arrive at a tile (deterministic);
//   * programmatic dependent launch: the prologue and the weight copies may overlap the previous kernel of the stream,
//     the activation copies wait for it.
// Every mbarrier wait is bounded; on expiry the kernel records B2Q_ERR_TIMEOUT and leaves.
#include "tc_common.cuh"
#include <stdlib.h>

namespace skinny {

constexpr int TILE_ROWS = 128;
constexpr int BK = 128;          // K bytes per stage: one swizzle atom
constexpr int kWWarps = 2;
constexpr int kThreads = 32 * (7 + kWWarps - 1);   // warp 0 weights, 1 MMA, 2..5 epilogue, 6 activations, 7.. more weight warps
constexpr uint64_t kWaitLimitNs = 500000000ull;

template <int NB> struct Cfg {                        // NB: accumulator columns = padded tokens
  static constexpr int kBytesW = TILE_ROWS * BK;      // 16 KiB
  static constexpr int kBytesX = NB * BK;
  static constexpr int kStageBytes = kBytesW + kBytesX;
  static constexpr int kStages = NB == 128 ? 6 : 8;   // even: a stage keeps its weight warp
  static constexpr int kSmem = kStages * kStageBytes + 1024 + 256;
  static constexpr int kTmemCols = NB <= 16 ? 32 : 2 * NB;   // two accumulators
  static_assert(kStages % kWWarps == 0, "a stage must belong to one weight warp");
};

struct Params {
  const float* scale_a; int scale_a_rows;
  const float* scale_w; int scale_w_rows;
  float* partials;            // [tile][slot][NB][128]
  int32_t* counters;          // [tile], zero on entry and on exit
  void* out; int out_type;
  int tokens;
  int64_t N, K;
  int stages_per_tile, units, per, max_slots;
  uint32_t idesc;
  int wait_first;             // 1: read nothing before the previous kernel of the stream has completed
  int32_t* status;
};

using namespace tcx;
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  return mbar_wait_bounded(bar, parity, abort_flag, kWaitLimitNs, 1);
}
__device__ __forceinline__ void umma_f8(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
template <int NB>
__global__ void __launch_bounds__(kThreads, 1)
gemm_fp8_skinny_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_a, const Params p) {
  using C = Cfg<NB>;
  constexpr int kStages = C::kStages;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
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
  const int total = u1 - u0;

  if (p.wait_first) asm volatile("griddepcontrol.wait;" ::: "memory");
  if (threadIdx.x == 0) {
    s_abort = 0;
    // a stage is full after two arrivals (weight copy issued, activation copy issued) and their bytes
    for (int s = 0; s < kStages; ++s) { mbar_init(full_bar(s), 2); mbar_init(empty_bar(s), 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(tfull_bar(b), 1); mbar_init(tempty_bar(b), 4); }
    mbar_init(drain_bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_w)) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_a)) : "memory");
    // the first round of weight copies needs nothing but the barriers: start the HBM stream before the rest of the prologue
    for (int it = 0; it < kStages && it < total; ++it) {
      const int u = u0 + it, tile = u / S, j = u - tile * S;
      mbar_expect_tx(full_bar(it), C::kBytesW);
      tma_load_2d(base + it * C::kStageBytes, &map_w, full_bar(it), j * BK, tile * TILE_ROWS);
    }
  }
  if (warp == 1) tmem_alloc(smem_u32(&s_tmem_base), C::kTmemCols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = s_tmem_base;
  volatile int* abort_flag = &s_abort;
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  if (warp == 0 || warp >= 7) {
    // ---------------- weight producers: stage s belongs to weight warp s % kWWarps ----------------
    const int w_idx = warp == 0 ? 0 : warp - 6;
    if (lane == 0) {
      bool ok = true;
      for (int it = kStages + w_idx; it < total; it += kWWarps) {      // kStages % kWWarps == 0
        const int u = u0 + it, tile = u / S, j = u - tile * S;
        const int s = it % kStages;
        const uint32_t ph = (uint32_t)(it / kStages) & 1;
        if (!mbar_wait(empty_bar(s), ph ^ 1, abort_flag)) { ok = false; break; }
        mbar_expect_tx(full_bar(s), C::kBytesW);
        tma_load_2d(base + s * C::kStageBytes, &map_w, full_bar(s), j * BK, tile * TILE_ROWS);
      }
      if (!ok || *abort_flag) {
        // a wait expired somewhere: give the copies in flight time to land before shared memory is released
        const uint64_t t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 2000000ull) {}
      }
    }
  } else if (warp == 6) {
    // ---------------- activation producer: rows past the last token are zero-filled by the TMA unit ----------------
    if (lane == 0) {
      // the activations come from the previous kernel of the stream, which this grid may overlap
      asm volatile("griddepcontrol.wait;" ::: "memory");
      for (int it = 0; it < total; ++it) {
        const int j = (u0 + it) % S;
        const int s = it % kStages;
        const uint32_t ph = (uint32_t)(it / kStages) & 1;
        if (!mbar_wait(empty_bar(s), ph ^ 1, abort_flag)) break;
        mbar_expect_tx(full_bar(s), C::kBytesX);
        tma_load_2d(base + s * C::kStageBytes + C::kBytesW, &map_a, full_bar(s), j * BK, 0);
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      int it = 0;
      uint32_t seg_it = 0;
      bool ok = true;
      for (int u = u0; u < u1 && ok; ++seg_it) {
        const int tile = u / S, j0 = u - tile * S;
        const int n = min(u1 - u, S - j0);
        const uint32_t buf = seg_it & 1, aph = (seg_it >> 1) & 1;
        if (!mbar_wait(tempty_bar(buf), aph ^ 1, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + buf * NB;
        for (int jj = 0; jj < n; ++jj, ++it) {
          const int s = it % kStages;
          const uint32_t ph = (uint32_t)(it / kStages) & 1;
          if (!mbar_wait(full_bar(s), ph, abort_flag)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sw = base + s * C::kStageBytes;
          const uint64_t adesc = make_desc_sw128(sw), bdesc = make_desc_sw128(sw + C::kBytesW);
#pragma unroll
          for (int k = 0; k < 4; ++k)                          // K advance inside the swizzle atom: +32 bytes
            umma_f8(tmem_d, adesc + (uint64_t)(2 * k), bdesc + (uint64_t)(2 * k), p.idesc, (uint32_t)((jj | k) != 0));
          tc_commit(empty_bar(s));
        }
        if (ok) tc_commit(tfull_bar(buf));
        u += n;
      }
      if (!ok) {
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
    uint32_t seg_it = 0;
    bool ok = true;
    for (int u = u0; u < u1 && ok; ++seg_it) {
      const int tile = u / S, j0 = u - tile * S;
      const int n = min(u1 - u, S - j0);
      u += n;
      const uint32_t buf = seg_it & 1, aph = (seg_it >> 1) & 1;
      if (!mbar_wait(tfull_bar(buf), aph, abort_flag)) { ok = false; break; }
      tc_fence_after();
      const int64_t row = (int64_t)tile * TILE_ROWS + row_local;
      const bool whole = n == S;
      const int first = (tile * S) / p.per, last = (tile * S + S - 1) / p.per;
      const int nc = last - first + 1, slot = (int)blockIdx.x - first;
      float* mine = p.partials + ((int64_t)tile * p.max_slots + slot) * (NB * TILE_ROWS);
      const float sw = p.scale_w_rows ? (row < p.N ? p.scale_w[row] : 0.0f) : p.scale_w[0];
      auto store_out = [&](int t, float acc) {
        if (row < p.N && t < p.tokens) {
          const float v = acc * ((p.scale_a_rows ? p.scale_a[t] : p.scale_a[0]) * sw);
          if (p.out_type == B2Q_OUT_BF16) reinterpret_cast<__nv_bfloat16*>(p.out)[(int64_t)t * p.N + row] = __float2bfloat16_rn(v);
          else reinterpret_cast<float*>(p.out)[(int64_t)t * p.N + row] = v;
        }
      };
#pragma unroll 1
      for (int c = 0; c < NB; c += 16) {                      // 16 tokens at a time
        if (c >= p.tokens) break;                             // uniform: no token in the remaining columns
        uint32_t r[16];
        tmem_ld16(tmem_base + buf * NB + c + ((uint32_t)(q * 32) << 16), r);
        tmem_ld_wait();
        if (whole) {
#pragma unroll
          for (int i = 0; i < 16; ++i) store_out(c + i, __uint_as_float(r[i]));
        } else {
#pragma unroll
          for (int i = 0; i < 16; ++i) if (c + i < p.tokens) mine[(c + i) * TILE_ROWS + row_local] = __uint_as_float(r[i]);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(tempty_bar(buf));            // the accumulator has been read
      if (!whole) {
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
          const float* all = p.partials + (int64_t)tile * p.max_slots * (NB * TILE_ROWS);
#pragma unroll 1
          for (int c = 0; c < p.tokens; c += 16) {
            float sum[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) sum[i] = 0.0f;
            for (int k = 0; k < nc; ++k) {                    // contributors in CTA order
              float part[16];
#pragma unroll
              for (int i = 0; i < 16; ++i)
                part[i] = c + i < p.tokens ? __ldcg(all + (int64_t)k * (NB * TILE_ROWS) + (c + i) * TILE_ROWS + row_local) : 0.0f;
#pragma unroll
              for (int i = 0; i < 16; ++i) sum[i] += part[i];
            }
#pragma unroll
            for (int i = 0; i < 16; ++i) store_out(c + i, sum[i]);
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
    tmem_dealloc(tmem_base, C::kTmemCols);
  }
  if (threadIdx.x == 0 && s_abort) atomicCAS(p.status, 0, (int)B2Q_ERR_TIMEOUT);
}

// ---- host side --------------------------------------------------------------
// rows x K bytes, K-major; box = 128 bytes x box_rows, 128-byte swizzle, zero fill out of bounds
static int32_t make_map(b2q_handle h, EncodeTiledFn enc, CUtensorMap* map, const void* ptr, int64_t rows, int64_t K, int box_rows) {
  cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)K};
  cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) B2Q_FAIL(h, B2Q_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
  return B2Q_OK;
}

template <int NB>
int32_t launch(b2q_handle h, const uint8_t* a, const uint8_t* w, int tokens, int64_t N, int64_t K, int fmt, const float* scale_a,
               int ka, const float* scale_w, int kw, void* out, int out_type) {
  using C = Cfg<NB>;
  EncodeTiledFn enc = get_encode_fn();
  if (!enc) B2Q_FAIL(h, B2Q_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  CUtensorMap map_w, map_a;
  int32_t st = make_map(h, enc, &map_w, w, N, K, TILE_ROWS);
  if (st != B2Q_OK) return st;
  st = make_map(h, enc, &map_a, a, tokens, K, NB);
  if (st != B2Q_OK) return st;

  Params p = {};
  const int S = (int)(K / BK);
  const int64_t tiles = ceil_div64(N, TILE_ROWS);
  const int64_t units = tiles * S;
  const int64_t slots = h->sm_count;
  const int64_t rounds = ceil_div64(tiles, slots);
  int grid, per;
  if (tiles * 10 >= rounds * slots * 7) {                      // whole tiles keep most SMs busy: no partial sums to exchange
    per = S * (int)rounds;
    grid = (int)ceil_div64(units, per);
  } else {
    grid = (int)(units < slots ? units : slots);
    per = (int)ceil_div64(units, grid);
    grid = (int)ceil_div64(units, per);
  }
  p.max_slots = (S + per - 1) / per + 1;
  const size_t part_bytes = (size_t)tiles * p.max_slots * NB * TILE_ROWS * sizeof(float);
  void* ws = nullptr;
  st = b2q_workspace(h, part_bytes, &ws);
  if (st != B2Q_OK) return st;
  p.scale_a = scale_a; p.scale_a_rows = ka;
  p.scale_w = scale_w; p.scale_w_rows = kw;
  p.partials = reinterpret_cast<float*>(ws);
  p.counters = h->d_tile_counters;
  p.out = out; p.out_type = out_type;
  p.tokens = tokens;
  p.N = N; p.K = K;
  p.stages_per_tile = S;
  p.units = (int)units;
  p.per = per;
  // instruction descriptor (kind::f8f6f4): fp32 accumulate, A = weights and B = activations in `fmt`, both K-major, N = NB, M = 128
  p.idesc = (1u << 4) | ((uint32_t)fmt << 7) | ((uint32_t)fmt << 10) | ((uint32_t)(NB >> 3) << 17) | ((uint32_t)(TILE_ROWS >> 4) << 24);
  p.wait_first = h->dynamic_weights;
  p.status = h->d_status;

  B2Q_SMEM_ATTR(h, (gemm_fp8_skinny_kernel<NB>), C::kSmem);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)grid);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = C::kSmem;
  cfg.stream = h->stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = h->sw.skinny_pdl == 0 ? 0 : 1;                // B2Q_SKINNY_PDL=0: plain stream-ordered launch
  B2Q_CUDA(h, cudaLaunchKernelEx(&cfg, gemm_fp8_skinny_kernel<NB>, map_w, map_a, p));
  return B2Q_OK;
}

}  // namespace skinny

// FP8 GEMM for M <= 128 tokens on the weight-stationary tcgen05 kernel; B2Q_ERR_UNSUPPORTED (nothing launched) when
// the shape does not fit: K % 128, 16-byte aligned operands.
int32_t b2q_gemm_fp8_skinny_dispatch(b2q_handle h, const uint8_t* a, const uint8_t* w, int64_t M, int64_t N, int64_t K, int fmt,
                                     const float* scale_a, int ka, const float* scale_w, int kw, void* out, int out_type) {
  if (M < 1 || M > 128 || K % 128 != 0 || N < 1) return B2Q_ERR_UNSUPPORTED;
  if (((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(w)) & 15) != 0) return B2Q_ERR_UNSUPPORTED;
  const int64_t tiles = ceil_div64(N, skinny::TILE_ROWS);
  if (tiles > (int64_t)kTileCounters || tiles * (K / skinny::BK) > 0x7FFFFFFF) return B2Q_ERR_UNSUPPORTED;
  const int t = (int)M;
  if (t <= 16) return skinny::launch<16>(h, a, w, t, N, K, fmt, scale_a, ka, scale_w, kw, out, out_type);
  if (t <= 32) return skinny::launch<32>(h, a, w, t, N, K, fmt, scale_a, ka, scale_w, kw, out, out_type);
  if (t <= 64) return skinny::launch<64>(h, a, w, t, N, K, fmt, scale_a, ka, scale_w, kw, out, out_type);
  return skinny::launch<128>(h, a, w, t, N, K, fmt, scale_a, ka, scale_w, kw, out, out_type);
}
