// Prefill-shaped quantized GEMM on the 5th-generation tensor cores (sm_100a):
//   out[m,n] = (sum_k A[m,k] * W[n,k]) * scale_a * scale_w
// A [M x K] and W [N x K] are 8-bit codes (E4M3/E5M2, or INT8), both K-major.
//
// One persistent CTA per SM, 6 warps:
//   warp 0      TMA producer: cp.async.bulk.tensor (each CTA issues its own copies) into a ring of
//               128-byte-swizzled shared-memory stages, completion on mbarriers;
//   warp 1      allocates TMEM and issues tcgen05.mma (one elected thread), the
//               accumulator (128 lanes x BN fp32/s32 columns) lives in TMEM and is
//               double-buffered so the epilogue of tile i overlaps the MMAs of i+1;
//   warps 2..5  epilogue: the tile's scales are fetched before the accumulator is waited for, then tcgen05.ld of
//               their 32-lane quarter, scale (alpha / beta / bias / activation, or SwiGLU over column pairs), convert
//               to bf16/f32 into a swizzled shared-memory buffer, one TMA store per buffer (raw s32 and odd pitches:
//               vectorised global stores).
// Every mbarrier wait is bounded (wall-clock limit); on expiry the kernel records
// B2Q_ERR_TIMEOUT in the status word, drains what it issued, frees TMEM and returns.
#include "tc_common.cuh"
#include <stdlib.h>

namespace tc {

constexpr int BM = 128;        // accumulator rows (= TMEM lanes)
constexpr int BK = 128;        // K bytes per stage: one 128-byte swizzle atom
constexpr int UMMA_K = 32;     // K per tcgen05.mma for 8-bit operands
constexpr int kThreads = 192;
constexpr int GROUP_M = 8;     // tile rasterisation: 8 row-blocks share each W panel in L2
constexpr uint64_t kWaitLimitNs = 2000000000ull;

enum Kind { kF8 = 0, kI8 = 1, kBF16 = 2 };   // kBF16: 16-bit operands, K counted in BYTES by the kernels (BK = 64 elements)

constexpr int kEpiBytes = 4 * 2 * 4096;   // epilogue staging: per warp two buffers of 32 rows x 128 bytes (TMA store sources)

template <int BN> struct Cfg {
  static constexpr int kStages = BN == 256 ? 4 : 6;
  static constexpr int kBytesA = BM * BK;
  static constexpr int kBytesB = BN * BK;
  static constexpr int kStageBytes = kBytesA + kBytesB;
  static constexpr int kTmemCols = 2 * BN;                       // two accumulators
  static constexpr int kSmem = kStages * kStageBytes + kEpiBytes + 1024 /*align*/ + 256 /*barriers*/;
};

struct Params {
  int64_t M, N, K;
  int tiles_m, tiles_n;
  uint32_t idesc;
  const float* scale_a; int scale_a_rows;
  const float* scale_w; int scale_w_rows;
  void* out; int out_type;          // kF8: bf16 / f32 scaled
  int32_t* c_s32; float* c_f32;     // kI8: raw accumulators and/or scaled f32
  int32_t* status;
  // pair kernel only: units [0, full_units) are whole 256x256 tiles, units beyond are 256x128 halves of the last tiles
  int full_units, total_units;
  uint32_t idesc_half;
  // epilogue (EpilogueOp of the reference): out = act(alpha * acc * sa * sw + beta * out_old + bias[n])
  int epi;                          // 0: plain scaled store; else the fields below apply
  float alpha, beta;
  const float* bias;                // [N] or null
  int act;                          // 0 none, 1 relu, 2 gelu as x * sigmoid(1.702 x); 3 SwiGLU over column pairs (pair kernel
                                    // only): columns [256 j, 256 j + 128) of the product are gate, the next 128 up, and
                                    // out [M x N / 2] gets silu(gate) * up at columns [128 j, 128 j + 128)
  int tma_store;                    // 1: bf16 / f32 rows leave through shared memory and TMA stores (16-byte aligned pitch)
  // grouped mode of the pair kernel (groups > 0, table on the device): problem g multiplies rows
  // [group_offsets[g], group_offsets[g] + group_counts[g]) of A (offsets are multiples of 256, so a tile never spans
  // two problems) with rows [g * N, (g + 1) * N) of W and scale_w, and stores into the same rows of out
  const int32_t* group_offsets; const int32_t* group_counts; int groups;
  // scatter mode of the pair kernel (rs_tp > 0, the row-parallel boundary of a tensor-parallel linear): the tile rows
  // [o * rs_rows, (o + 1) * rs_rows) belong to rank o; they are stored, as bf16, through that rank's tensor map (its
  // inbox in peer-mapped memory) at rows rs_rank * rs_rows + (row - o * rs_rows), i.e. into the slot of THIS rank
  int rs_tp, rs_rank, rs_rows;
  // tile rasterisation of the pair kernel: groups of group_m row tiles sweep the columns (0: GROUP_M); with group_rot the
  // groups are walked starting at group group_rot (scatter mode: every rank starts at another owner's rows, so no rank's
  // NVLink ingress is the target of all the others at once)
  int group_m, group_rot;
};
constexpr int kMaxGroups = 64;
constexpr int kMaxScatterRanks = 8;
struct ScatterMaps { CUtensorMap m[kMaxScatterRanks]; };

using namespace tcx;
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  return mbar_wait_bounded(bar, parity, abort_flag, kWaitLimitNs, 1);
}
template <int KIND>
__device__ __forceinline__ void umma(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  if constexpr (KIND == kF8) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
  } else if constexpr (KIND == kI8) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
  } else {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
  }
}
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t smem_addr) { return make_desc_sw128(smem_addr); }

__device__ __forceinline__ void tile_coords(int tile, int tiles_m, int tiles_n, int& mb, int& nb, int group_m = GROUP_M, int group_rot = 0) {
  const int group_size = group_m * tiles_n;
  int group = tile / group_size;
  const int in_tile = tile - group * group_size;
  if (group_rot) {                                     // only with tiles_m % group_m == 0: all groups are whole
    const int ngroups = tiles_m / group_m;
    group = (group + group_rot) % ngroups;
    tile = group * group_size + in_tile;
  }
  const int first_m = group * group_m;
  const int gm = min(tiles_m - first_m, group_m);
  const int in_group = tile - group * group_size;
  mb = first_m + in_group % gm;
  nb = in_group / gm;
}

// alpha / beta / bias / activation of the reference's EpilogueOp (crates/oxicuda-blas/src/level3/gemm/epilogue.rs:99-196):
// result = acc * alpha; result = fma(beta, c_old, result); + bias[col]; relu or gelu (x * sigmoid(1.702 x), :153-190).
__device__ __forceinline__ float epi_apply(const Params& p, float v, float c_old, int64_t col) {
  v *= p.alpha;
  if (p.beta != 0.0f) v = fmaf(p.beta, c_old, v);
  if (p.bias) v += __ldg(p.bias + col);
  if (p.act == 1) v = fmaxf(v, 0.0f);
  else if (p.act == 2) v = v * __frcp_rn(1.0f + exp2f(-1.702f * 1.4426950408889634f * v));
  return v;
}

// Eight consecutive per-column weight scales (every lane of the warp needs the same eight: one 16-byte load serves four).
__device__ __forceinline__ void load_sw8(const float* scale_w, int64_t n, int64_t N, bool vec, float (&sw)[8]) {
  if (vec) {
    const float4 a = __ldg(reinterpret_cast<const float4*>(scale_w + n)), b = __ldg(reinterpret_cast<const float4*>(scale_w + n + 4));
    sw[0] = a.x; sw[1] = a.y; sw[2] = a.z; sw[3] = a.w; sw[4] = b.x; sw[5] = b.y; sw[6] = b.z; sw[7] = b.w;
  } else {
#pragma unroll
    for (int i = 0; i < 8; ++i) sw[i] = n + i < N ? __ldg(scale_w + n + i) : 0.0f;
  }
}

// Scales, converts and stores 32 consecutive accumulator columns of one output row.
template <int KIND>
__device__ __forceinline__ void store_chunk(const Params& p, const uint32_t (&r)[32], int64_t m, int64_t n, float sa, float sw0) {
  const bool full = n + 32 <= p.N;
  if constexpr (KIND != kI8) {
    float v[32];
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      const float sw = p.scale_w_rows ? (n + j < p.N ? __ldg(p.scale_w + n + j) : 0.0f) : sw0;
      v[j] = __uint_as_float(r[j]) * (sa * sw);
      if (p.epi && n + j < p.N) {
        const float cold = p.beta == 0.0f ? 0.0f
                         : (p.out_type == B2Q_OUT_BF16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p.out)[m * p.N + n + j])
                                                       : reinterpret_cast<const float*>(p.out)[m * p.N + n + j]);
        v[j] = epi_apply(p, v[j], cold, n + j);
      }
    }
    if (p.out_type == B2Q_OUT_BF16) {
      __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(p.out) + m * p.N + n;
      if (full && ((reinterpret_cast<uintptr_t>(o) & 15) == 0)) {
#pragma unroll
        for (int j = 0; j < 32; j += 8) {
          uint4 pk;
          __nv_bfloat162 h0 = __floats2bfloat162_rn(v[j], v[j + 1]), h1 = __floats2bfloat162_rn(v[j + 2], v[j + 3]);
          __nv_bfloat162 h2 = __floats2bfloat162_rn(v[j + 4], v[j + 5]), h3 = __floats2bfloat162_rn(v[j + 6], v[j + 7]);
          pk.x = *reinterpret_cast<uint32_t*>(&h0); pk.y = *reinterpret_cast<uint32_t*>(&h1);
          pk.z = *reinterpret_cast<uint32_t*>(&h2); pk.w = *reinterpret_cast<uint32_t*>(&h3);
          *reinterpret_cast<uint4*>(o + j) = pk;
        }
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) if (n + j < p.N) o[j] = __float2bfloat16_rn(v[j]);
      }
    } else {
      float* o = reinterpret_cast<float*>(p.out) + m * p.N + n;
      if (full && ((reinterpret_cast<uintptr_t>(o) & 15) == 0)) {
#pragma unroll
        for (int j = 0; j < 32; j += 4) *reinterpret_cast<float4*>(o + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) if (n + j < p.N) o[j] = v[j];
      }
    }
  } else {
    if (p.c_s32) {
      int32_t* o = p.c_s32 + m * p.N + n;
      if (full && ((reinterpret_cast<uintptr_t>(o) & 15) == 0)) {
#pragma unroll
        for (int j = 0; j < 32; j += 4) *reinterpret_cast<uint4*>(o + j) = make_uint4(r[j], r[j + 1], r[j + 2], r[j + 3]);
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) if (n + j < p.N) o[j] = (int32_t)r[j];
      }
    }
    if (p.c_f32) {
      float* o = p.c_f32 + m * p.N + n;
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        if (n + j < p.N) {
          float f = __int2float_rn((int32_t)r[j]);
          if (p.scale_a) f = __fmul_rn(f, __fmul_rn(sa, p.scale_w[n + j]));
          o[j] = f;
        }
      }
    }
  }
}

// One warp's share of an output tile: its 32 accumulator rows (TMEM lane quarter) x `width` columns.
// Fast path (bf16 / f32 with a 16-byte aligned pitch): 64 (bf16) or 32 (f32) columns at a time go through a
// 128-byte-swizzled shared-memory buffer of 32 rows x 128 bytes and leave with one TMA store per buffer, i.e. as
// full 128-byte row segments; two buffers per warp, so a store is in flight while the next chunk is converted.
// TMA clips rows >= M and columns >= N.  Other outputs (INT8 accumulators, odd pitches) store from registers.
struct EpiWarp { uint32_t smem_u; uint8_t* smem_p; uint32_t it; };

// The scales one warp needs for one unit, fetched BEFORE the accumulator is waited for (so their latency hides behind the
// MMAs instead of sitting in every chunk of the epilogue): sa, the scale of this lane's row, and eight consecutive
// per-column weight scales per lane, handed round with shuffles.  Plain: lane l holds columns [8 l, 8 l + 8) of the
// unit.  SwiGLU pairs: lanes [0, width / 16) hold the gate columns, the next width / 16 lanes the matching up columns
// (128 rows of W further on).
struct TileScales { float sw[8]; float sa; };
__device__ __forceinline__ TileScales prefetch_scales(const Params& p, const float* scale_w, int64_t n0, int width, int64_t m, bool swiglu, int lane) {
  TileScales t;
  t.sa = (m < p.M && p.scale_a) ? (p.scale_a_rows ? __ldg(p.scale_a + m) : __ldg(p.scale_a)) : 1.0f;
#pragma unroll
  for (int i = 0; i < 8; ++i) t.sw[i] = 1.0f;
  if (scale_w && p.scale_w_rows) {
    const int half_l = width >> 4;
    const bool live = swiglu ? lane < 2 * half_l : 8 * lane < width;
    const int64_t idx = !swiglu ? n0 + 8 * lane : (lane < half_l ? n0 + 8 * lane : n0 + 128 + 8 * (lane - half_l));
    if (live) load_sw8(scale_w, idx, p.N, idx + 8 <= p.N && (reinterpret_cast<uintptr_t>(scale_w + idx) & 15) == 0, t.sw);
  }
  return t;
}

template <int KIND>
__device__ __forceinline__ void epilogue_rows(const Params& pp, const CUtensorMap* map_out, EpiWarp& ew, uint32_t tmem_acc, int width,
                                              int64_t m_warp0, int lane, int64_t n0, const float* scale_w, int64_t m_store, const TileScales& ts) {
  Params p = pp;
  p.scale_w = scale_w;                       // this tile's weight scales (grouped mode: the problem's slice)
  const int64_t m = m_warp0 + lane;
  const bool row_ok = m < p.M;
  const float sa = ts.sa;
  const float sw0 = p.scale_w && !p.scale_w_rows ? p.scale_w[0] : 1.0f;
  if constexpr (KIND != kI8) {
    if (p.tma_store) {
      const bool bf16 = p.out_type == B2Q_OUT_BF16;
      const int CH = bf16 ? 64 : 32;
#pragma unroll 1
      for (int c = 0; c < width; c += CH) {
        uint32_t r[64];
        __syncwarp();
        tmem_ld32(tmem_acc + c, *reinterpret_cast<uint32_t(*)[32]>(&r[0]));
        if (bf16) tmem_ld32(tmem_acc + c + 32, *reinterpret_cast<uint32_t(*)[32]>(&r[32]));
        tmem_ld_wait();
        const int64_t n = n0 + c;
        if (n >= p.N || m_warp0 >= p.M) continue;                // nothing of this chunk lies inside the output (warp-uniform)
        const uint32_t buf = (ew.it & 1u) * 4096u;
        if (lane == 0) tma_store_wait_read<1>();                 // the store that last read this buffer has read it
        __syncwarp();
        uint8_t* row = ew.smem_p + buf + lane * 128;
        if (bf16) {
#pragma unroll
          for (int j = 0; j < 64; j += 8) {
            float v[8], sw[8];
            if (p.scale_w_rows) {                                // columns c + j .. c + j + 7 of the unit: lane (c + j) / 8 holds them
#pragma unroll
              for (int i = 0; i < 8; ++i) sw[i] = __shfl_sync(0xffffffffu, ts.sw[i], (c + j) >> 3);
            }
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = __uint_as_float(r[j + i]) * (sa * (p.scale_w_rows ? sw[i] : sw0));
            if (p.epi) {
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                const bool in = row_ok && n + j + i < p.N;
                const float cold = (p.beta != 0.0f && in) ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p.out)[m * p.N + n + j + i]) : 0.0f;
                v[i] = in ? epi_apply(p, v[i], cold, n + j + i) : 0.0f;
              }
            }
            uint4 pk;
            __nv_bfloat162 h0 = __floats2bfloat162_rn(v[0], v[1]), h1 = __floats2bfloat162_rn(v[2], v[3]);
            __nv_bfloat162 h2 = __floats2bfloat162_rn(v[4], v[5]), h3 = __floats2bfloat162_rn(v[6], v[7]);
            pk.x = *reinterpret_cast<uint32_t*>(&h0); pk.y = *reinterpret_cast<uint32_t*>(&h1);
            pk.z = *reinterpret_cast<uint32_t*>(&h2); pk.w = *reinterpret_cast<uint32_t*>(&h3);
            *reinterpret_cast<uint4*>(row + ((((j >> 3)) ^ (lane & 7)) << 4)) = pk;     // 128-byte swizzle: 16-byte unit ^ (row & 7)
          }
        } else {
#pragma unroll
          for (int j = 0; j < 32; j += 4) {
            float v[4];
            float4 sw4 = make_float4(sw0, sw0, sw0, sw0);
            if (p.scale_w_rows) {
              const int src = (c + j) >> 3;
              sw4.x = __shfl_sync(0xffffffffu, ts.sw[(j & 4) + 0], src); sw4.y = __shfl_sync(0xffffffffu, ts.sw[(j & 4) + 1], src);
              sw4.z = __shfl_sync(0xffffffffu, ts.sw[(j & 4) + 2], src); sw4.w = __shfl_sync(0xffffffffu, ts.sw[(j & 4) + 3], src);
            }
            const float swa[4] = {sw4.x, sw4.y, sw4.z, sw4.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const float sw = swa[i];
              v[i] = __uint_as_float(r[j + i]) * (sa * sw);
              if (p.epi) {
                const bool in = row_ok && n + j + i < p.N;
                const float cold = (p.beta != 0.0f && in) ? reinterpret_cast<const float*>(p.out)[m * p.N + n + j + i] : 0.0f;
                v[i] = in ? epi_apply(p, v[i], cold, n + j + i) : 0.0f;
              }
            }
            *reinterpret_cast<float4*>(row + ((((j >> 2)) ^ (lane & 7)) << 4)) = make_float4(v[0], v[1], v[2], v[3]);
          }
        }
        fence_async_smem();                                      // the TMA unit reads what the warp just wrote
        __syncwarp();
        if (lane == 0) {
          tma_store_2d(map_out, ew.smem_u + buf, (int)n, (int)m_store);     // m_store = m_warp0 except in scatter mode
          tma_store_commit();
        }
        ++ew.it;
      }
      return;
    }
  }
#pragma unroll 1
  for (int c = 0; c < width; c += 32) {
    uint32_t r[32];
    __syncwarp();                           // tcgen05.ld is warp-collective: reconverge after the guarded stores
    tmem_ld32(tmem_acc + c, r);
    tmem_ld_wait();
    const int64_t n = n0 + c;
    if (!row_ok || n >= p.N) continue;
    store_chunk<KIND>(p, r, m, n, sa, sw0);
  }
}

// SwiGLU over column pairs (Params::act == 3): one warp's 32 rows of a 256-column accumulator tile whose columns
// [0, 128) are gate and [128, 256) up projections of the same 128 hidden units (the weight rows are interleaved per 128).
// h = silu(gate) * up with both factors scaled in fp32 (SwiGluExpert::forward, crates/oxicuda-moe/src/expert/ffn.rs:208-243;
// silu(x) = x / (1 + exp(-x)), crates/oxicuda-lm/src/layer/ffn.rs:25-27), stored as bf16 into out [M x N / 2] through the
// same staging buffers and TMA stores as the plain epilogue.  The GEMM result itself never reaches memory.
// `width` accumulator columns: gate in the first half, up in the second (256 for a whole tile, 128 for a half unit of
// the last wave: 64 gate and the matching 64 up columns); n0 = the gate column (row of W) of accumulator column 0.
__device__ __forceinline__ void epilogue_rows_swiglu(const Params& p, const CUtensorMap* map_out, EpiWarp& ew, uint32_t tmem_acc, int width,
                                                     int64_t m_warp0, int lane, int64_t n0, const float* scale_w, const TileScales& ts) {
  const float sa = ts.sa;
  const float sw0 = scale_w && !p.scale_w_rows ? scale_w[0] : 1.0f;
  const int half_w = width >> 1;
  const int64_t out0 = (n0 >> 8) * 128 + (n0 & 255);             // column of out [M x N / 2] that gate column n0 maps to
#pragma unroll 1
  for (int c = 0; c < half_w; c += 64) {
    const uint32_t buf = (ew.it & 1u) * 4096u;
    uint8_t* row = ew.smem_p + buf + lane * 128;
#pragma unroll 1
    for (int sub = 0; sub < 2; ++sub) {
      uint32_t g[32], u[32];
      __syncwarp();
      tmem_ld32(tmem_acc + c + 32 * sub, g);
      tmem_ld32(tmem_acc + half_w + c + 32 * sub, u);
      tmem_ld_wait();
      if (m_warp0 >= p.M) continue;                              // warp-uniform: nothing of these rows is inside the output
      if (sub == 0) {
        if (lane == 0) tma_store_wait_read<1>();                 // the store that last read this buffer has read it
        __syncwarp();
      }
      const int64_t ng = n0 + c + 32 * sub;                      // gate column of g[0]; its up column is ng + 128
#pragma unroll
      for (int j = 0; j < 32; j += 8) {
        float h[8], swgv[8], swuv[8];
        if (p.scale_w_rows) {                                    // gate column c + 32 sub + j of the unit and its up partner
          const int src = (c + 32 * sub + j) >> 3;
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            swgv[i] = __shfl_sync(0xffffffffu, ts.sw[i], src);
            swuv[i] = __shfl_sync(0xffffffffu, ts.sw[i], (width >> 4) + src);
          }
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float swg = p.scale_w_rows ? swgv[i] : sw0;
          const float swu = p.scale_w_rows ? swuv[i] : sw0;
          const float gg = __uint_as_float(g[j + i]) * (sa * swg), uu = __uint_as_float(u[j + i]) * (sa * swu);
          h[i] = gg * uu * __frcp_rn(1.0f + exp2f(-1.4426950408889634f * gg));
        }
        uint4 pk;
        __nv_bfloat162 h0 = __floats2bfloat162_rn(h[0], h[1]), h1 = __floats2bfloat162_rn(h[2], h[3]);
        __nv_bfloat162 h2 = __floats2bfloat162_rn(h[4], h[5]), h3 = __floats2bfloat162_rn(h[6], h[7]);
        pk.x = *reinterpret_cast<uint32_t*>(&h0); pk.y = *reinterpret_cast<uint32_t*>(&h1);
        pk.z = *reinterpret_cast<uint32_t*>(&h2); pk.w = *reinterpret_cast<uint32_t*>(&h3);
        *reinterpret_cast<uint4*>(row + (((sub * 4 + (j >> 3)) ^ (lane & 7)) << 4)) = pk;
      }
    }
    if (m_warp0 >= p.M) continue;
    fence_async_smem();
    __syncwarp();
    if (lane == 0) {
      tma_store_2d(map_out, ew.smem_u + buf, (int)(out0 + c), (int)m_warp0);
      tma_store_commit();
    }
    ++ew.it;
  }
}

template <int BN, int KIND>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
               const __grid_constant__ CUtensorMap map_out, const Params p) {
  using C = Cfg<BN>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t epi_base = base + C::kStages * C::kStageBytes;     // 1024-byte aligned: the stage size is a multiple of 1024
  const uint32_t bar_base = epi_base + kEpiBytes;
  // barrier layout (8 bytes each): full[stages], empty[stages], tmem_full[2], tmem_empty[2], drain
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (C::kStages + s); };
  auto tfull_bar = [&](int b) { return bar_base + 8u * (2 * C::kStages + b); };
  auto tempty_bar = [&](int b) { return bar_base + 8u * (2 * C::kStages + 2 + b); };
  const uint32_t drain_bar = bar_base + 8u * (2 * C::kStages + 4);
  __shared__ uint32_t s_tmem_base;
  __shared__ int s_abort;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int total_tiles = p.tiles_m * p.tiles_n;
  const int num_kb = (int)((p.K + BK - 1) / BK);

  if (threadIdx.x == 0) {
    s_abort = 0;
    for (int s = 0; s < C::kStages; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(tfull_bar(b), 1); mbar_init(tempty_bar(b), 4); }
    mbar_init(drain_bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_a)) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_w)) : "memory");
    if (p.tma_store) asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_out)) : "memory");
  }
  if (warp == 1) tmem_alloc(smem_u32(&s_tmem_base), C::kTmemCols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = s_tmem_base;
  volatile int* abort_flag = &s_abort;

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
        int mb, nb;
        tile_coords(tile, p.tiles_m, p.tiles_n, mb, nb);
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % C::kStages;
          const uint32_t ph = (it / C::kStages) & 1;
          if (!mbar_wait(empty_bar(s), ph ^ 1, abort_flag)) { ok = false; break; }
          const uint32_t sa = base + s * C::kStageBytes, sb = sa + C::kBytesA;
          mbar_expect_tx(full_bar(s), C::kStageBytes);
          tma_load_2d(sa, &map_a, full_bar(s), kb * BK, mb * BM);
          tma_load_2d(sb, &map_w, full_bar(s), kb * BK, nb * BN);
        }
      }
      if (!ok) {
        // give every copy already issued a bounded chance to land before shared memory is released
        const uint32_t issued = it < (uint32_t)C::kStages ? it : (uint32_t)C::kStages;
        for (uint32_t j = 0; j < issued; ++j) {
          const uint32_t q = it - 1 - j;
          const uint64_t t0 = globaltimer_ns();
          while (!mbar_try_wait(full_bar(q % C::kStages), (q / C::kStages) & 1))
            if (globaltimer_ns() - t0 > 100000000ull) break;
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      uint32_t it = 0, tile_it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++tile_it) {
        const uint32_t buf = tile_it & 1, aph = (tile_it >> 1) & 1;
        if (!mbar_wait(tempty_bar(buf), aph ^ 1, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + buf * BN;
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % C::kStages;
          const uint32_t ph = (it / C::kStages) & 1;
          if (!mbar_wait(full_bar(s), ph, abort_flag)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = base + s * C::kStageBytes, sb = sa + C::kBytesA;
          const uint64_t adesc = make_smem_desc(sa), bdesc = make_smem_desc(sb);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            // advancing K inside the swizzle atom: +32 bytes on the start address (16-byte units)
            umma<KIND>(tmem_d, adesc + (uint64_t)(k * (UMMA_K >> 4)), bdesc + (uint64_t)(k * (UMMA_K >> 4)), p.idesc,
                       (uint32_t)((kb | k) != 0));
          }
          tc_commit(empty_bar(s));          // stage reusable once these MMAs have read it
        }
        if (ok) tc_commit(tfull_bar(buf));  // accumulator complete
      }
      if (!ok) {                            // wait (bounded) for MMAs in flight before TMEM is freed
        tc_commit(drain_bar);
        const uint64_t t0 = globaltimer_ns();
        while (!mbar_try_wait(drain_bar, 0))
          if (globaltimer_ns() - t0 > 100000000ull) break;
      }
    }
  } else {
    // ---------------- epilogue (4 warps) ----------------
    const int q = warp & 3;                 // TMEM lane quarter this warp may access
    uint32_t tile_it = 0;
    bool ok = true;
    EpiWarp ew{epi_base + (uint32_t)q * 8192u, smem_raw + (epi_base - smem_u32(smem_raw)) + q * 8192, 0u};
    for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++tile_it) {
      int mb, nb;
      tile_coords(tile, p.tiles_m, p.tiles_n, mb, nb);
      const uint32_t buf = tile_it & 1, aph = (tile_it >> 1) & 1;
      const TileScales ts = prefetch_scales(p, p.scale_w, (int64_t)nb * BN, BN, (int64_t)mb * BM + q * 32 + lane, false, lane);
      if (!mbar_wait(tfull_bar(buf), aph, abort_flag)) { ok = false; break; }
      tc_fence_after();
      epilogue_rows<KIND>(p, &map_out, ew, tmem_base + buf * BN + ((uint32_t)(q * 32) << 16), BN, (int64_t)mb * BM + q * 32, lane,
                          (int64_t)nb * BN, p.scale_w, (int64_t)mb * BM + q * 32, ts);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(tempty_bar(buf));
    }
    if (lane == 0) tma_store_wait<0>();     // shared memory stays valid until the last store has read it
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


// =============================================================================
// Two-CTA variant (cta_group::2): a cluster of two CTAs on one TPC computes a
// 256 x 256 output tile.  Each CTA stages its own 128 rows of A and its own 128
// rows of W per K block (32 KiB per stage instead of 48 KiB), the leader CTA
// issues one tcgen05.mma.cta_group::2 per 32-wide K step that reads both CTAs'
// shared memory, and each CTA's TMEM receives its 128 accumulator rows.  Shared
// memory traffic per SM drops from 192 to 128 bytes per MMA-clock, which is what
// bounds the one-CTA kernel.  Every CTA issues its own TMA copies: it loads its own halves and
// signals the leader's "full" barrier; stage release and accumulator hand-off use
// tcgen05.commit with a two-CTA mask.
// =============================================================================
namespace two {

constexpr int BN2 = 256;                 // output columns of the pair tile
constexpr int kStages = 6;
constexpr int kBytesA = BM * BK;         // this CTA's 128 rows of A
constexpr int kBytesB = (BN2 / 2) * BK;  // this CTA's 128 rows of W
constexpr int kStageBytes = kBytesA + kBytesB;
constexpr int kTmemCols = 2 * BN2;
constexpr int kSmem = kStages * kStageBytes + kEpiBytes + 1024 + 256;

__device__ __forceinline__ uint32_t cluster_ctarank() { uint32_t r; asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r)); return r; }
__device__ __forceinline__ uint32_t mapa_u32(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// TMA load into THIS CTA's shared memory; the byte count is credited to `bar`, a shared::cluster address
// (the leader CTA's barrier)..
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void tmem_alloc2(uint32_t dst_smem, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(cols) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc2(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
// arrive on the barrier at this shared-memory offset in both CTAs of the pair once the MMAs issued so far are done
__device__ __forceinline__ void tc_commit_pair(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(bar), "h"((uint16_t)3) : "memory");
}
template <int KIND>
__device__ __forceinline__ void umma2(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  if constexpr (KIND == kF8) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
  } else if constexpr (KIND == kI8) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
  } else {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
  }
}

template <int KIND>
__device__ __forceinline__ void gemm_tc2_body(const CUtensorMap& map_a, const CUtensorMap& map_w, const CUtensorMap& map_w_half,
                                              const CUtensorMap& map_out, const CUtensorMap* scatter_maps, const Params& p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t epi_base = base + kStages * kStageBytes;
  const uint32_t bar_base = epi_base + kEpiBytes;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (kStages + s); };
  auto tfull_bar = [&](int b) { return bar_base + 8u * (2 * kStages + b); };
  auto tempty_bar = [&](int b) { return bar_base + 8u * (2 * kStages + 2 + b); };
  const uint32_t drain_bar = bar_base + 8u * (2 * kStages + 4);
  __shared__ uint32_t s_tmem_base;
  __shared__ int s_abort;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();          // 0 = leader (issues the MMAs), 1 = peer
  const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
  // Work units: whole 256 x 256 tiles first; when the last wave would leave more than half of the CTA pairs idle, its
  // tiles are cut into two 256 x 128 halves (MMA N = 128, 64 rows of W per CTA) so that the tail takes half a wave.
  // Grouped mode: the units are the 256 x 256 tiles of every problem in turn; the table is read once per CTA.
  // (16-bit entries: with its 225 KiB of stages this CTA leaves just over 1 KiB of the SM's shared memory, which is
  // what lets a small exchange kernel of another stream become resident beside it)
  __shared__ int s_gstart[kMaxGroups + 1];
  __shared__ uint16_t s_goff256[kMaxGroups], s_gtm[kMaxGroups];   // row offset / 256, row tiles
  struct Unit { int a_row, w_row, width, half; int64_t n0; int64_t sw_off; };
  auto unit_coords = [&](int u) {
    Unit c;
    if (p.groups > 0) {
      int g = 0;
      while (g + 1 < p.groups && u >= s_gstart[g + 1]) ++g;
      int mb, nb;
      tile_coords(u - s_gstart[g], s_gtm[g], p.tiles_n, mb, nb);
      c.a_row = (int)s_goff256[g] * 256 + mb * 256; c.w_row = g * (int)p.N + nb * BN2; c.width = BN2; c.half = 0;
      c.n0 = (int64_t)nb * BN2; c.sw_off = (int64_t)g * p.N;
      return c;
    }
    int tile, mb, nb;
    if (u < p.full_units) { tile = u; c.half = 0; c.width = BN2; }
    else { const int v = u - p.full_units; tile = p.full_units + (v >> 1); c.half = v & 1; c.width = BN2 / 2; }
    tile_coords(tile, p.tiles_m, p.tiles_n, mb, nb, p.group_m > 0 ? p.group_m : GROUP_M, p.group_rot);
    c.a_row = mb * 256; c.sw_off = 0;
    if (p.act == 3) {
      // SwiGLU pairs: a half unit takes 64 gate and the matching 64 up columns (CTA 0 loads the gate rows, CTA 1 the up rows);
      // n0 is the gate column of the unit's first accumulator column
      c.w_row = nb * BN2 + c.half * (BN2 / 4); c.n0 = (int64_t)nb * BN2 + c.half * (BN2 / 4);
    } else {
      c.w_row = nb * BN2 + c.half * (BN2 / 2); c.n0 = (int64_t)nb * BN2 + c.half * (BN2 / 2);
    }
    return c;
  };
  const int num_kb = (int)((p.K + BK - 1) / BK);

  if (threadIdx.x == 0) {
    s_abort = 0;
    for (int s = 0; s < kStages; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(tfull_bar(b), 1); mbar_init(tempty_bar(b), 8); }   // 4 epilogue warps x 2 CTAs
    mbar_init(drain_bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_a)) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_w)) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_w_half)) : "memory");
    if (p.tma_store) asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_out)) : "memory");
    s_gstart[0] = 0;
    for (int g = 0; g < p.groups; ++g) {
      const int cnt = p.group_counts[g];
      s_goff256[g] = (uint16_t)(p.group_offsets[g] >> 8);
      s_gtm[g] = (uint16_t)((cnt + 255) / 256);
      s_gstart[g + 1] = s_gstart[g] + s_gtm[g] * p.tiles_n;
    }
  }
  if (warp == 1) tmem_alloc2(smem_u32(&s_tmem_base), kTmemCols);
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();                               // both CTAs' barriers exist before anyone signals across
  tc_fence_after();
  const uint32_t tmem_base = s_tmem_base;
  volatile int* abort_flag = &s_abort;
  const int total_units = p.groups > 0 ? s_gstart[p.groups] : p.total_units;

  if (warp == 0) {
    // ---------------- TMA producer (both CTAs) ----------------
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int u = pair; u < total_units && ok; u += num_pairs) {
        const Unit c = unit_coords(u);
        const int width = c.width;
        const uint32_t bytes = 2u * (uint32_t)(kBytesA + (width / 2) * BK);  // both CTAs' bytes land on the leader's barrier
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % kStages;
          const uint32_t ph = (it / kStages) & 1;
          if (!mbar_wait(empty_bar(s), ph ^ 1, abort_flag)) { ok = false; break; }
          const uint32_t sa = base + s * kStageBytes, sb = sa + kBytesA;
          const uint32_t leader_full = mapa_u32(full_bar(s), 0);
          if (rank == 0) mbar_expect_tx(full_bar(s), bytes);
          tma_load_2d_pair(sa, &map_a, leader_full, kb * BK, c.a_row + (int)rank * BM);
          if (width == BN2) tma_load_2d_pair(sb, &map_w, leader_full, kb * BK, c.w_row + (int)rank * (BN2 / 2));
          else tma_load_2d_pair(sb, &map_w_half, leader_full, kb * BK, c.w_row + (int)rank * (p.act == 3 ? BN2 / 2 : BN2 / 4));
        }
      }
      if (!ok) {   // give copies already issued time to land before shared memory is released
        const uint64_t t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 1000000ull) {}
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer (leader CTA only) ----------------
    if (lane == 0 && rank == 0) {
      uint32_t it = 0, tile_it = 0;
      bool ok = true;
      for (int u = pair; u < total_units && ok; u += num_pairs, ++tile_it) {
        const uint32_t idesc = (p.groups > 0 || u < p.full_units) ? p.idesc : p.idesc_half;
        const uint32_t buf = tile_it & 1, aph = (tile_it >> 1) & 1;
        if (!mbar_wait(tempty_bar(buf), aph ^ 1, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + buf * BN2;
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % kStages;
          const uint32_t ph = (it / kStages) & 1;
          if (!mbar_wait(full_bar(s), ph, abort_flag)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = base + s * kStageBytes, sb = sa + kBytesA;
          const uint64_t adesc = make_smem_desc(sa), bdesc = make_smem_desc(sb);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k)
            umma2<KIND>(tmem_d, adesc + (uint64_t)(k * (UMMA_K >> 4)), bdesc + (uint64_t)(k * (UMMA_K >> 4)), idesc,
                        (uint32_t)((kb | k) != 0));
          tc_commit_pair(empty_bar(s));
        }
        if (ok) tc_commit_pair(tfull_bar(buf));
      }
      if (!ok) {
        tc_commit(drain_bar);
        const uint64_t t0 = globaltimer_ns();
        while (!mbar_try_wait(drain_bar, 0))
          if (globaltimer_ns() - t0 > 100000000ull) break;
      }
    }
  } else {
    // ---------------- epilogue (4 warps in each CTA) ----------------
    const int q = warp & 3;
    uint32_t tile_it = 0;
    bool ok = true;
    EpiWarp ew{epi_base + (uint32_t)q * 8192u, smem_raw + (epi_base - smem_u32(smem_raw)) + q * 8192, 0u};
    for (int u = pair; u < total_units && ok; u += num_pairs, ++tile_it) {
      const Unit c = unit_coords(u);
      const uint32_t buf = tile_it & 1, aph = (tile_it >> 1) & 1;
      const int64_t m_warp0 = (int64_t)c.a_row + rank * BM + q * 32;
      const bool swiglu = KIND == kF8 && p.act == 3;
      const TileScales ts = prefetch_scales(p, p.scale_w ? p.scale_w + c.sw_off : nullptr, c.n0, c.width, m_warp0 + lane, swiglu, lane);
      if (!mbar_wait(tfull_bar(buf), aph, abort_flag)) { ok = false; break; }
      tc_fence_after();
      const CUtensorMap* mo = &map_out;
      int64_t m_store = m_warp0;
      if (scatter_maps) {                               // this warp's 32 rows belong to one rank (rs_rows is a multiple of 32)
        const int owner = min((int)(m_warp0 / p.rs_rows), p.rs_tp - 1);
        mo = scatter_maps + owner;
        m_store = (int64_t)p.rs_rank * p.rs_rows + (m_warp0 - (int64_t)owner * p.rs_rows);
      }
      if (swiglu)
        epilogue_rows_swiglu(p, mo, ew, tmem_base + buf * BN2 + ((uint32_t)(q * 32) << 16), c.width, m_warp0, lane, c.n0,
                             p.scale_w ? p.scale_w + c.sw_off : nullptr, ts);
      else
        epilogue_rows<KIND>(p, mo, ew, tmem_base + buf * BN2 + ((uint32_t)(q * 32) << 16), c.width, m_warp0, lane, c.n0,
                            p.scale_w ? p.scale_w + c.sw_off : nullptr, m_store, ts);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(mapa_u32(tempty_bar(buf), 0));   // the leader's MMA thread waits for both CTAs
    }
    if (lane == 0) tma_store_wait<0>();
  }

  // ---------------- teardown ----------------
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();                               // the peer's TMEM and barriers stay valid until both CTAs are done
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc2(tmem_base, kTmemCols);
  }
  if (threadIdx.x == 0 && s_abort) atomicCAS(p.status, 0, (int)B2Q_ERR_TIMEOUT);
}

template <int KIND>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tc2_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                const __grid_constant__ CUtensorMap map_w_half, const __grid_constant__ CUtensorMap map_out, const Params p) {
  gemm_tc2_body<KIND>(map_a, map_w, map_w_half, map_out, nullptr, p);
}
// The same kernel with one output map per rank: each accumulator row block goes to the rank that owns it (its inbox in
// peer-mapped memory), so the partial sums of a row-parallel linear cross NVLink tile by tile while the MMAs run.
template <int KIND>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tc2_scatter_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                        const __grid_constant__ CUtensorMap map_w_half, const __grid_constant__ ScatterMaps maps, const Params p) {
  gemm_tc2_body<KIND>(map_a, map_w, map_w_half, maps.m[0], maps.m, p);
}

}  // namespace two

// ---- host side --------------------------------------------------------------
// rows x K bytes, K-major; box = 128 bytes x box_rows, 128-byte swizzle, zero fill out of bounds.  Encoded maps are
// kept in the handle (keyed by pointer, extents, box and element type), so a steady-state call encodes nothing.
int32_t make_map(b2q_handle h, CUtensorMap* map, const void* ptr, int64_t rows, int64_t K, int box_rows) {
  return b2q_tensor_map_2d(h, map, ptr, /*elem_bytes=*/1, (uint64_t)K, (uint64_t)rows, (uint32_t)BK, (uint32_t)box_rows);
}
// The output [M x N] as a TMA store target: boxes of 32 rows x 128 bytes (64 bf16 or 32 f32 columns), 128-byte swizzle.
// Leaves p.tma_store = 0 (register stores) when the pointer or the pitch is not 16-byte aligned.
int32_t make_out_map(b2q_handle h, CUtensorMap* map, Params& p) {
  memset(map, 0, sizeof(*map));
  p.tma_store = 0;
  if (!p.out || p.c_s32 || p.c_f32) return B2Q_OK;
  const int es = p.out_type == B2Q_OUT_BF16 ? 2 : 4;
  if ((reinterpret_cast<uintptr_t>(p.out) & 15) != 0 || (p.N * es) % 16 != 0) return B2Q_OK;
  const int64_t out_cols = p.act == 3 ? p.N / 2 : p.N;
  int32_t st = b2q_tensor_map_2d(h, map, p.out, es, (uint64_t)out_cols, (uint64_t)p.M, (uint32_t)(128 / es), 32u);
  if (st == B2Q_OK) p.tma_store = 1;
  return st;
}

template <int BN, int KIND>
int32_t launch(b2q_handle h, const void* a, const void* w, Params p) {
  using C = Cfg<BN>;
  CUtensorMap map_a, map_w, map_out;
  int32_t st = make_map(h, &map_a, a, p.M, p.K, BM);
  if (st != B2Q_OK) return st;
  st = make_map(h, &map_w, w, p.N, p.K, BN);
  if (st != B2Q_OK) return st;
  st = make_out_map(h, &map_out, p);
  if (st != B2Q_OK) return st;
  p.tiles_m = (int)ceil_div64(p.M, BM);
  p.tiles_n = (int)ceil_div64(p.N, BN);
  // instruction descriptor: dense, D format, A/B formats, both K-major, N>>3 at bit 17, M>>4 at bit 24
  const uint32_t shape = ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
  p.idesc = KIND == kF8 ? (p.idesc | (1u << 4) | shape)                                   // fp32 accumulate, E4M3/E5M2 per p.idesc
          : KIND == kI8 ? ((2u << 4) | (1u << 7) | (1u << 10) | shape)                    // s32 accumulate, signed 8-bit A and B
                        : ((1u << 4) | (1u << 7) | (1u << 10) | shape);                   // fp32 accumulate, bf16 A and B
  B2Q_SMEM_ATTR(h, (gemm_tc_kernel<BN, KIND>), C::kSmem);
  int64_t tiles = (int64_t)p.tiles_m * p.tiles_n;
  int grid = (int)(tiles < h->sm_count ? tiles : h->sm_count);
  gemm_tc_kernel<BN, KIND><<<grid, kThreads, C::kSmem, h->stream>>>(map_a, map_w, map_out, p);
  B2Q_LAUNCH_CHECK(h, "gemm_tc_kernel");
  return B2Q_OK;
}

// 256 x 256 pair tiles on clusters of two CTAs.
template <int KIND>
int32_t launch2(b2q_handle h, const void* a, const void* w, Params p, const ScatterMaps* scatter = nullptr) {
  CUtensorMap map_a, map_w;
  int32_t st = make_map(h, &map_a, a, p.M, p.K, BM);
  if (st != B2Q_OK) return st;
  st = make_map(h, &map_w, w, p.N, p.K, two::BN2 / 2);
  if (st != B2Q_OK) return st;
  CUtensorMap map_w_half, map_out;
  st = make_map(h, &map_w_half, w, p.N, p.K, two::BN2 / 4);
  if (st != B2Q_OK) return st;
  if (scatter) { memset(&map_out, 0, sizeof(map_out)); p.tma_store = 1; }
  else st = make_out_map(h, &map_out, p);
  if (st != B2Q_OK) return st;
  p.tiles_m = (int)ceil_div64(p.M, 256);
  p.tiles_n = (int)ceil_div64(p.N, two::BN2);
  if (p.group_m == 0 && !scatter) {
    // row tiles per raster group: as many as keep the group's A panel (group_m x 256 x K bytes) within about 48 MB of the
    // 126 MB L2 while the weight tiles stream past it once per group; at least GROUP_M, at most all of them
    const int64_t fit = (48ll << 20) / (256 * (p.K > 0 ? p.K : 1));
    int gm = (int)(fit < GROUP_M ? GROUP_M : (fit > 64 ? 64 : fit));
    if (h->sw.force_group_m > 0) gm = h->sw.force_group_m;
    p.group_m = gm < p.tiles_m ? gm : (p.tiles_m > 0 ? p.tiles_m : 1);
  }
  const uint32_t idesc_fmt = p.idesc;
  uint32_t shape = ((uint32_t)((two::BN2 / 2) >> 3) << 17) | ((uint32_t)(256 >> 4) << 24);
  p.idesc_half = KIND == kF8 ? (idesc_fmt | (1u << 4) | shape)
               : KIND == kI8 ? ((2u << 4) | (1u << 7) | (1u << 10) | shape)
                             : ((1u << 4) | (1u << 7) | (1u << 10) | shape);
  shape = ((uint32_t)(two::BN2 >> 3) << 17) | ((uint32_t)(256 >> 4) << 24);
  p.idesc = KIND == kF8 ? (p.idesc | (1u << 4) | shape)                                   // fp32 accumulate, E4M3/E5M2 per p.idesc
          : KIND == kI8 ? ((2u << 4) | (1u << 7) | (1u << 10) | shape)                    // s32 accumulate, signed 8-bit A and B
                        : ((1u << 4) | (1u << 7) | (1u << 10) | shape);                   // fp32 accumulate, bf16 A and B
  B2Q_SMEM_ATTR(h, (two::gemm_tc2_kernel<KIND>), two::kSmem);
  const int64_t tiles = (int64_t)p.tiles_m * p.tiles_n;
  const int max_pairs = h->sm_count / 2;
  // tail split: when the last wave fills at most half of the pairs, its tiles become two half-width units each
  const int rem = (int)(tiles % max_pairs);
  // (in SwiGLU-pair mode a half unit is 64 gate and the matching 64 up columns)
  const bool split = tiles > max_pairs && rem > 0 && 2 * rem <= max_pairs && h->sw.no_tail_split < 0;
  p.full_units = split ? (int)(tiles - rem) : (int)tiles;
  p.total_units = split ? (int)(tiles + rem) : (int)tiles;
  const int pairs = (int)(p.total_units < max_pairs ? p.total_units : max_pairs);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(2 * pairs));
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = two::kSmem;
  cfg.stream = h->stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (scatter) {
    if constexpr (KIND == kF8) {
      B2Q_SMEM_ATTR(h, (two::gemm_tc2_scatter_kernel<kF8>), two::kSmem);
      B2Q_CUDA(h, cudaLaunchKernelEx(&cfg, two::gemm_tc2_scatter_kernel<kF8>, map_a, map_w, map_w_half, *scatter, p));
      return B2Q_OK;
    }
    return B2Q_ERR_UNSUPPORTED;
  }
  B2Q_CUDA(h, cudaLaunchKernelEx(&cfg, two::gemm_tc2_kernel<KIND>, map_a, map_w, map_w_half, map_out, p));
  return B2Q_OK;
}

}  // namespace tc

int32_t b2q_validate_gemm_fp8(b2q_handle h, const uint8_t* a, const uint8_t* w, int64_t M, int64_t N, int64_t K, int fmt,
                              const float* scale_a, int ka, const float* scale_w, int kw, void* out, int out_type, int64_t out_cols);

int32_t b2q_gemm_fp8_skinny_dispatch(b2q_handle h, const uint8_t* a, const uint8_t* w, int64_t M, int64_t N, int64_t K, int fmt,
                                     const float* scale_a, int ka, const float* scale_w, int kw, void* out, int out_type);
int32_t b2q_gemv_fp8_dispatch(b2q_handle h, const uint8_t* a, const uint8_t* w, int64_t M, int64_t N, int64_t K, int fmt,
                              const float* scale_a, int ka, const float* scale_w, int kw, void* out, int out_type);

int32_t b2q_gemm_i8_tc(b2q_handle h, const int8_t* a, const int8_t* b, int64_t M, int64_t N, int64_t K, int32_t* c_s32,
                       float* c_f32, const float* sa, const float* sb) {
  if (K % 16 != 0 || ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b)) & 15) != 0 || N < 64)
    return B2Q_ERR_UNSUPPORTED;
  tc::Params p{};
  p.M = M; p.N = N; p.K = K;
  p.scale_a = sa; p.scale_a_rows = 1; p.scale_w = sb; p.scale_w_rows = 1;
  p.c_s32 = c_s32; p.c_f32 = c_f32; p.status = h->d_status;
  b2q_tile_config t; int kid = 0;
  b2q_select_tile(2, (uint32_t)M, (uint32_t)N, (uint32_t)K, &t, &kid);
  if (kid == 4) return tc::launch2<tc::kI8>(h, a, b, p);
  return kid == 1 ? tc::launch<256, tc::kI8>(h, a, b, p) : tc::launch<128, tc::kI8>(h, a, b, p);
}

// bf16 x bf16 -> bf16/f32 on the same pipeline (tcgen05 kind::f16); a [M x K], w [N x K], both K-major.
// Used by the weight-only FP4 prefill GEMM after the weights are expanded to bf16.
int32_t b2q_gemm_bf16_tc(b2q_handle h, const void* a, const void* w, int64_t M, int64_t N, int64_t K, void* out, int out_type) {
  if (K % 8 != 0 || ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(w)) & 15) != 0) return B2Q_ERR_UNSUPPORTED;
  tc::Params p{};
  p.M = M; p.N = N; p.K = 2 * K;                        // bytes
  p.out = out; p.out_type = out_type; p.status = h->d_status;
  if (M > 128 && N > 128) return tc::launch2<tc::kBF16>(h, a, w, p);
  return N >= 256 ? tc::launch<256, tc::kBF16>(h, a, w, p) : tc::launch<128, tc::kBF16>(h, a, w, p);
}

namespace tc {

struct EpiArgs { float alpha, beta; const float* bias; int act; };

// out = act(alpha * plain + beta * out + bias[col]) for the kernels that have no fused epilogue (few-token and SIMT paths):
// `plain` is their f32 result.
__global__ void __launch_bounds__(256) epilogue_post_kernel(const float* __restrict__ plain, void* out, int out_type, int64_t M, int64_t N,
                                                            float alpha, float beta, const float* __restrict__ bias, int act) {
  const int64_t total = M * N;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    float v = plain[i] * alpha;
    if (beta != 0.0f) {
      const float cold = out_type == B2Q_OUT_BF16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(out)[i]) : reinterpret_cast<const float*>(out)[i];
      v = fmaf(beta, cold, v);
    }
    if (bias) v += bias[i % N];
    if (act == 1) v = fmaxf(v, 0.0f);
    else if (act == 2) v = v * __frcp_rn(1.0f + exp2f(-1.702f * 1.4426950408889634f * v));
    if (out_type == B2Q_OUT_BF16) reinterpret_cast<__nv_bfloat16*>(out)[i] = __float2bfloat16_rn(v);
    else reinterpret_cast<float*>(out)[i] = v;
  }
}

// SwiGLU over column pairs for the kernels without that epilogue: plain [M x N] f32 with gate at columns
// [256 j, 256 j + 128) and up at the next 128 -> out [M x N / 2].
__global__ void __launch_bounds__(256) swiglu_pairs_post_kernel(const float* __restrict__ plain, void* out, int out_type, int64_t M, int64_t N) {
  const int64_t F = N / 2, total = M * F;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t m = i / F, f = i - m * F, col = ((f >> 7) << 8) + (f & 127);
    const float g = plain[m * N + col], u = plain[m * N + col + 128];
    const float v = g * u * __frcp_rn(1.0f + exp2f(-1.4426950408889634f * g));
    if (out_type == B2Q_OUT_BF16) reinterpret_cast<__nv_bfloat16*>(out)[i] = __float2bfloat16_rn(v);
    else reinterpret_cast<float*>(out)[i] = v;
  }
}

// [K x N] row-major codes -> [N x K] (the layout every kernel here reads): 32 x 32 byte tiles through shared memory.
__global__ void __launch_bounds__(256) transpose_u8_kernel(const uint8_t* __restrict__ in, uint8_t* __restrict__ out, int64_t K, int64_t N) {
  __shared__ uint8_t tile[32][33];
  const int64_t n0 = (int64_t)blockIdx.x * 32, k0 = (int64_t)blockIdx.y * 32;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  for (int r = ty; r < 32; r += 8)
    if (k0 + r < K && n0 + tx < N) tile[r][tx] = in[(k0 + r) * N + n0 + tx];
  __syncthreads();
  for (int r = ty; r < 32; r += 8)
    if (n0 + r < N && k0 + tx < K) out[(n0 + r) * K + k0 + tx] = tile[tx][r];
}

int32_t gemm_fp8_impl(b2q_handle h, const uint8_t* a, const uint8_t* w, int64_t M, int64_t N, int64_t K, int fmt, const float* scale_a,
                      int scale_a_kind, const float* scale_w, int scale_w_kind, void* out, int out_type, const EpiArgs* epi) {
  b2q_tile_config t; int kid = 0;
  b2q_select_tile(0, (uint32_t)M, (uint32_t)N, (uint32_t)K, &t, &kid);
  if (kid != 0) {   // experiment switch: B2Q_FORCE_TILE_N=128|256|p overrides the static table
    if (h->sw.force_tile == 128) kid = 2;
    if (h->sw.force_tile == 256) kid = 1;
    if (h->sw.force_tile == 9) kid = 4;        // "p(air)": the two-CTA kernel
  }
  const bool tma_ok = K % 16 == 0 && ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(w)) & 15) == 0;
  bool fused = (kid == 1 || kid == 2 || kid == 4) && tma_ok;            // the prefill kernels apply the epilogue themselves
  if (epi && epi->act == 3)                                             // SwiGLU pairs: the pair kernel with TMA stores of bf16 only
    fused = kid == 4 && tma_ok && N % 256 == 0 && out_type == B2Q_OUT_BF16 && (reinterpret_cast<uintptr_t>(out) & 15) == 0;
  if (epi && !fused) {
    // few-token / SIMT kernels: plain f32 result into the second workspace (the kernels use the first themselves),
    // then one elementwise pass
    void* ws = nullptr;
    int32_t st = b2q_workspace2(h, (size_t)M * N * sizeof(float), &ws);
    if (st != B2Q_OK) return st;
    st = gemm_fp8_impl(h, a, w, M, N, K, fmt, scale_a, scale_a_kind, scale_w, scale_w_kind, ws, B2Q_OUT_F32, nullptr);
    if (st != B2Q_OK) return st;
    const int64_t total = M * N;
    int grid = (int)((total + 255) / 256);
    if (grid > h->sm_count * 8) grid = h->sm_count * 8;
    if (epi->act == 3) swiglu_pairs_post_kernel<<<grid, 256, 0, h->stream>>>((const float*)ws, out, out_type, M, N);
    else epilogue_post_kernel<<<grid, 256, 0, h->stream>>>((const float*)ws, out, out_type, M, N, epi->alpha, epi->beta, epi->bias, epi->act);
    B2Q_LAUNCH_CHECK(h, "epilogue_post_kernel");
    return B2Q_OK;
  }
  {
    // few tokens against a large weight matrix (kernel 6 of the static table): the weight-stationary tcgen05 kernel
    // streams W at HBM rate (B2Q_FP8_SKINNY=0 / 1 forces it off / on)
    if (M <= 128 && !epi && (h->sw.fp8_skinny >= 0 ? h->sw.fp8_skinny == 1 : kid == 6)) {
      int32_t sst = b2q_gemm_fp8_skinny_dispatch(h, a, w, M, N, K, fmt, scale_a, scale_a_kind, scale_w, scale_w_kind, out, out_type);
      if (sst != B2Q_ERR_UNSUPPORTED) return sst;
    }
    if (kid == 6) b2q_select_tile_ex(0, (uint32_t)M, (uint32_t)N, (uint32_t)K, &t, &kid, 0);   // not taken (alignment, switch)
  }
  if (kid == 5) {   // decode-sized: tensor-core GEMV over the codes
    int32_t gst = b2q_gemv_fp8_dispatch(h, a, w, M, N, K, fmt, scale_a, scale_a_kind, scale_w, scale_w_kind, out, out_type);
    if (gst != B2Q_ERR_UNSUPPORTED) return gst;
    kid = 0;
  }
  if (kid == 0 || !tma_ok)
    return b2q_gemm_fp8_simt(h, a, w, M, N, K, fmt, /*IEEE decode, as the tensor core*/ 1, scale_a, scale_a_kind, scale_w,
                             scale_w_kind, out, out_type);
  Params p{};
  p.M = M; p.N = N; p.K = K;
  p.scale_a = scale_a; p.scale_a_rows = scale_a_kind; p.scale_w = scale_w; p.scale_w_rows = scale_w_kind;
  p.out = out; p.out_type = out_type; p.status = h->d_status;
  p.idesc = ((uint32_t)fmt << 7) | ((uint32_t)fmt << 10);   // A/B format: 0 = E4M3, 1 = E5M2
  p.alpha = 1.0f;
  if (epi) { p.epi = 1; p.alpha = epi->alpha; p.beta = epi->beta; p.bias = epi->bias; p.act = epi->act; }
  if (kid == 4) return launch2<kF8>(h, a, w, p);
  return kid == 1 ? launch<256, kF8>(h, a, w, p) : launch<128, kF8>(h, a, w, p);
}

// Row-parallel partial product with the reduce-scatter folded into the epilogue: rows [o * M / tp, (o + 1) * M / tp) of
// a * w^T (bf16) are stored into rank o's inbox (inbox[o], mapped into this process; rank `rank`'s own inbox is local
// memory) at slot `rank`; an inbox is [tp slots][M / tp rows][N] bf16.  `bias` ([N] or null) is added to this rank's
// partial.  The caller sums the slots once every rank's kernel has completed.  B2Q_ERR_UNSUPPORTED when the shape does not take the pair kernel.
int32_t gemm_fp8_scatter(b2q_handle h, const uint8_t* a, const uint8_t* w, int64_t M, int64_t N, int64_t K, int fmt, const float* scale_a,
                         const float* scale_w, const float* bias, void* const* inbox, int tp, int rank) {
  if (tp < 1 || tp > kMaxScatterRanks || M <= 128 || N <= 128 || M % (32 * tp) != 0 || N % 8 != 0 || K % 16 != 0 ||
      ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(w)) & 15) != 0 || M > 0x7FFFFFFF)
    return B2Q_ERR_UNSUPPORTED;
  ScatterMaps maps;
  memset(&maps, 0, sizeof(maps));
  for (int r = 0; r < tp; ++r) {
    if (!inbox[r] || (reinterpret_cast<uintptr_t>(inbox[r]) & 15) != 0) return B2Q_ERR_UNSUPPORTED;
    int32_t st = b2q_tensor_map_2d(h, &maps.m[r], inbox[r], 2, (uint64_t)N, (uint64_t)M, 64u, 32u);
    if (st != B2Q_OK) return st;
  }
  Params p{};
  p.M = M; p.N = N; p.K = K;
  p.scale_a = scale_a; p.scale_a_rows = 1; p.scale_w = scale_w; p.scale_w_rows = 1;
  p.out = inbox[rank]; p.out_type = B2Q_OUT_BF16; p.status = h->d_status;
  p.idesc = ((uint32_t)fmt << 7) | ((uint32_t)fmt << 10);
  p.alpha = 1.0f;
  if (bias) { p.epi = 1; p.bias = bias; }
  p.rs_tp = tp; p.rs_rank = rank; p.rs_rows = (int)(M / tp);
  // one raster group per owner (or several owners per group when an owner has less than a row tile), walked from the
  // next rank's rows on: at every moment the ranks store into different inboxes
  const int64_t tiles_m = ceil_div64(M, 256);
  const int gm = p.rs_rows >= 256 && p.rs_rows % 256 == 0 ? (p.rs_rows / 256 < GROUP_M ? p.rs_rows / 256 : GROUP_M) : 0;
  if (gm > 0 && tiles_m % gm == 0) {
    p.group_m = gm;
    const int ngroups = (int)(tiles_m / gm);
    // rs_rows / 256 row tiles per owner, gm per group: the group in which the next rank's rows start
    p.group_rot = (int)(((int64_t)((rank + 1) % tp) * (p.rs_rows / 256) / gm) % ngroups);
  }
  return launch2<kF8>(h, a, w, p, &maps);
}

// Grouped launch of the pair kernel: every CTA pair walks the tiles of all problems (table on the device).
int32_t launch2_grouped(b2q_handle h, const void* a, const void* w, Params p, int64_t capacity_rows) {
  CUtensorMap map_a, map_w, map_w_half, map_out;
  int32_t st = make_map(h, &map_a, a, capacity_rows, p.K, BM);
  if (st != B2Q_OK) return st;
  st = make_map(h, &map_w, w, (int64_t)p.groups * p.N, p.K, two::BN2 / 2);
  if (st != B2Q_OK) return st;
  map_w_half = map_w;                                             // no half-width tail units in grouped mode
  p.M = capacity_rows;
  st = make_out_map(h, &map_out, p);
  if (st != B2Q_OK) return st;
  p.tiles_m = 0;
  p.tiles_n = (int)ceil_div64(p.N, two::BN2);
  const uint32_t shape = ((uint32_t)(two::BN2 >> 3) << 17) | ((uint32_t)(256 >> 4) << 24);
  p.idesc = p.idesc | (1u << 4) | shape;                          // fp32 accumulate, E4M3 / E5M2 per p.idesc
  p.idesc_half = p.idesc;
  p.full_units = p.total_units = 0;
  B2Q_SMEM_ATTR(h, (two::gemm_tc2_kernel<kF8>), two::kSmem);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(2 * (h->sm_count / 2)));          // the unit count is known on the device only: one pair per two SMs
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = two::kSmem;
  cfg.stream = h->stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  B2Q_CUDA(h, cudaLaunchKernelEx(&cfg, two::gemm_tc2_kernel<kF8>, map_a, map_w, map_w_half, map_out, p));
  return B2Q_OK;
}

}  // namespace tc

int32_t b2q_grouped_gemm_fp8_rows_act(b2q_handle h, const uint8_t* a, const float* scale_a, const uint8_t* w, const float* scale_w,
                                      const int32_t* row_offsets, const int32_t* row_counts, int groups, int64_t capacity_rows, int64_t N, int64_t K,
                                      int fmt, void* out, int out_type, int act);
extern "C" int32_t b2q_grouped_gemm_fp8_rows(b2q_handle h, const uint8_t* a, const float* scale_a, const uint8_t* w, const float* scale_w,
                                             const int32_t* row_offsets, const int32_t* row_counts, int groups, int64_t capacity_rows,
                                             int64_t N, int64_t K, int fmt, void* out, int out_type) {
  return b2q_grouped_gemm_fp8_rows_act(h, a, scale_a, w, scale_w, row_offsets, row_counts, groups, capacity_rows, N, K, fmt, out, out_type, 0);
}
// act 3: every problem's weight rows are gate and up rows interleaved per 128 and out is [capacity_rows x N / 2] bf16 =
// silu(gate) * up (the SwiGLU epilogue of the pair kernel); act 0: the plain product.
int32_t b2q_grouped_gemm_fp8_rows_act(b2q_handle h, const uint8_t* a, const float* scale_a, const uint8_t* w, const float* scale_w,
                                      const int32_t* row_offsets, const int32_t* row_counts, int groups, int64_t capacity_rows, int64_t N, int64_t K,
                                      int fmt, void* out, int out_type, int act) {
  B2Q_REQUIRE_HANDLE(h);
  if (act == 3 && (N % 256 != 0 || out_type != B2Q_OUT_BF16 || (reinterpret_cast<uintptr_t>(out) & 15) != 0))
    B2Q_FAIL(h, B2Q_ERR_INVALID_ARGUMENT, "grouped_gemm_fp8_rows: the SwiGLU epilogue needs N %% 256 == 0 and a 16-byte aligned bf16 output");
  if (groups <= 0 || capacity_rows <= 0 || N <= 0 || K <= 0)
    B2Q_FAIL(h, B2Q_ERR_INVALID_DIMENSION, "grouped_gemm_fp8_rows: dimensions must be non-zero: groups=%d, rows=%lld, n=%lld, k=%lld", groups,
             (long long)capacity_rows, (long long)N, (long long)K);
  if (groups > tc::kMaxGroups) B2Q_FAIL(h, B2Q_ERR_UNSUPPORTED, "grouped_gemm_fp8_rows: at most %d problems per call, got %d", tc::kMaxGroups, groups);
  if (!a || !w || !scale_a || !scale_w || !row_offsets || !row_counts || !out || fmt < 0 || fmt > 1 || out_type < 0 || out_type > 1)
    B2Q_FAIL(h, B2Q_ERR_INVALID_ARGUMENT, "grouped_gemm_fp8_rows: bad argument");
  if (K % 16 != 0 || ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(w)) & 15) != 0)
    B2Q_FAIL(h, B2Q_ERR_INVALID_DIMENSION, "grouped_gemm_fp8_rows: K must be a multiple of 16 and the operands 16-byte aligned (TMA row pitch)");
  if ((int64_t)groups * N > 0x7FFFFFFF || capacity_rows > (65535ll << 8)) B2Q_FAIL(h, B2Q_ERR_UNSUPPORTED, "grouped_gemm_fp8_rows: too many rows");
  tc::Params p{};
  p.N = N; p.K = K;
  p.scale_a = scale_a; p.scale_a_rows = 1; p.scale_w = scale_w; p.scale_w_rows = 1;
  p.out = out; p.out_type = out_type; p.status = h->d_status;
  p.idesc = ((uint32_t)fmt << 7) | ((uint32_t)fmt << 10);
  p.alpha = 1.0f;
  p.group_offsets = row_offsets; p.group_counts = row_counts; p.groups = groups;
  if (act == 3) { p.epi = 1; p.act = 3; }
  return tc::launch2_grouped(h, a, w, p, capacity_rows);
}

extern "C" int32_t b2q_gemm_fp8_scatter(b2q_handle h, const uint8_t* a, const uint8_t* w, int64_t M, int64_t N, int64_t K, int fmt,
                                        const float* scale_a, const float* scale_w, const float* bias, void* const* inbox, int tp, int rank) {
  B2Q_REQUIRE_HANDLE(h);
  if (M <= 0 || N <= 0 || K <= 0)
    B2Q_FAIL(h, B2Q_ERR_INVALID_DIMENSION, "GEMM dimensions must be non-zero: m=%lld, n=%lld, k=%lld", (long long)M, (long long)N, (long long)K);
  if (!a || !w || !scale_a || !scale_w || !inbox || fmt < 0 || fmt > 1 || tp < 1 || tp > tc::kMaxScatterRanks || rank < 0 || rank >= tp)
    B2Q_FAIL(h, B2Q_ERR_INVALID_ARGUMENT, "gemm_fp8_scatter: bad argument");
  int32_t st = tc::gemm_fp8_scatter(h, a, w, M, N, K, fmt, scale_a, scale_w, bias, inbox, tp, rank);
  if (st == B2Q_ERR_UNSUPPORTED)
    B2Q_FAIL(h, B2Q_ERR_UNSUPPORTED, "gemm_fp8_scatter: needs M > 128, N > 128, M %% (32 * tp) == 0, N %% 8 == 0, K %% 16 == 0 and 16-byte aligned operands "
             "(m=%lld, n=%lld, k=%lld, tp=%d)", (long long)M, (long long)N, (long long)K, tp);
  return st;
}

extern "C" int32_t b2q_gemm_fp8(b2q_handle h, const uint8_t* a, const uint8_t* w, int64_t M, int64_t N, int64_t K, int fmt,
                                const float* scale_a, int scale_a_kind, const float* scale_w, int scale_w_kind, void* out,
                                int out_type) {
  B2Q_REQUIRE_HANDLE(h);
  int32_t st = b2q_validate_gemm_fp8(h, a, w, M, N, K, fmt, scale_a, scale_a_kind, scale_w, scale_w_kind, out, out_type, 0);
  if (st != B2Q_OK) return st;
  return tc::gemm_fp8_impl(h, a, w, M, N, K, fmt, scale_a, scale_a_kind, scale_w, scale_w_kind, out, out_type, nullptr);
}

extern "C" int32_t b2q_gemm_fp8_ex(b2q_handle h, const b2q_gemm_fp8_desc* d) {
  B2Q_REQUIRE_HANDLE(h);
  if (!d) B2Q_FAIL(h, B2Q_ERR_INVALID_ARGUMENT, "gemm_fp8_ex: null descriptor");
  if (d->epilogue < 0 || d->epilogue > 5) B2Q_FAIL(h, B2Q_ERR_INVALID_ARGUMENT, "gemm_fp8_ex: unknown epilogue %d", d->epilogue);
  if (d->epilogue == B2Q_EPI_SWIGLU && (d->n % 256 != 0 || d->alpha != 1.0f || d->beta != 0.0f))
    B2Q_FAIL(h, B2Q_ERR_INVALID_ARGUMENT, "gemm_fp8_ex: the SwiGLU epilogue needs n %% 256 == 0 (gate / up rows interleaved per 128), alpha 1, beta 0");
  if (d->w_layout < 0 || d->w_layout > 1) B2Q_FAIL(h, B2Q_ERR_INVALID_ARGUMENT, "gemm_fp8_ex: unknown weight layout %d", d->w_layout);
  const bool needs_bias = d->epilogue == B2Q_EPI_BIAS || d->epilogue == B2Q_EPI_BIAS_RELU;
  if (needs_bias && !d->bias) B2Q_FAIL(h, B2Q_ERR_INVALID_ARGUMENT, "gemm_fp8_ex: this epilogue needs a bias vector");
  int32_t st = b2q_validate_gemm_fp8(h, d->a, d->w, d->m, d->n, d->k, d->fmt, d->scale_a, d->scale_a_kind, d->scale_w, d->scale_w_kind,
                                     d->out, d->out_type, d->epilogue == B2Q_EPI_SWIGLU ? d->n / 2 : 0);
  if (st != B2Q_OK) return st;
  const uint8_t* w = d->w;
  if (d->w_layout == B2Q_W_KN) {
    // the reference's operand B is [K x N] row-major (gemm_api.rs:126-231); the kernels read [N x K]: transpose it into the
    // workspace first (one pass over the codes; hold weights as [N x K] to avoid it)
    void* ws = nullptr;
    const size_t off = ((size_t)d->m * d->n * sizeof(float) + 255) & ~(size_t)255;     // in front: the plain result of an unfused epilogue
    st = b2q_workspace2(h, off + (size_t)d->n * d->k, &ws);
    if (st != B2Q_OK) return st;
    uint8_t* wt = reinterpret_cast<uint8_t*>(ws) + off;
    dim3 grid((unsigned)ceil_div64(d->n, 32), (unsigned)ceil_div64(d->k, 32));
    tc::transpose_u8_kernel<<<grid, 256, 0, h->stream>>>(d->w, wt, d->k, d->n);
    B2Q_LAUNCH_CHECK(h, "transpose_u8_kernel");
    w = wt;
  }
  tc::EpiArgs e{d->alpha, d->beta, needs_bias ? d->bias : nullptr,
                (d->epilogue == B2Q_EPI_RELU || d->epilogue == B2Q_EPI_BIAS_RELU) ? 1
                    : (d->epilogue == B2Q_EPI_GELU ? 2 : (d->epilogue == B2Q_EPI_SWIGLU ? 3 : 0))};
  const bool plain = d->alpha == 1.0f && d->beta == 0.0f && !e.bias && e.act == 0;
  return tc::gemm_fp8_impl(h, d->a, w, d->m, d->n, d->k, d->fmt, d->scale_a, d->scale_a_kind, d->scale_w, d->scale_w_kind, d->out,
                           d->out_type, plain ? nullptr : &e);
}
