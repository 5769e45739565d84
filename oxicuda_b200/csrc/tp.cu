// Tensor-parallel linears behind the C ABI: ColumnLinear / RowLinear of oxicuda-dist-infer
// (crates/oxicuda-dist-infer/src/tensor_parallel/column_parallel.rs:103-205, row_parallel.rs:97-224) and the
// SwiGLU MLP built from them (SwiGluExpert::forward, crates/oxicuda-moe/src/expert/ffn.rs:208-243), one rank per
// process and GPU.  The reference sums partials in rank order on the host; here the row-parallel boundary is
//   * for few tokens (partial sums up to 4 MiB of fp32): ONE kernel over peer-mapped memory.  Every rank pushes its
//     fp32 partial into the other ranks' inboxes with plain NVLink stores, signals per-CTA flags, waits (bounded)
//     for its peers and adds the inboxes IN RANK ORDER in fp32 (the reference's order, the same bits on every rank).
//     Above 256 KiB the exchange is two-shot: each rank reduces one slice and pushes the bf16 result to all.
//     The buffer parity and the flag epoch live in device memory, so the launch can be captured in a CUDA graph;
//   * for many tokens (bf16 results up to 64 MiB): the reduce-scatter is folded into the GEMM.  The epilogue of the
//     tcgen05 kernel stores every accumulator row block straight into the inbox of the rank that owns those rows (TMA
//     stores into peer-mapped memory), so the partial sums cross NVLink tile by tile while the MMAs run; one kernel
//     then waits for the peers, adds the tp slots of its own rows in rank order in fp32 and pushes the bf16 sums to
//     every rank.  The ranks walk the row blocks from different starting owners, so no inbox is the target of all the
//     others at once.  Optionally (b2q_tp_set_chunks) the GEMM is cut into column chunks and that kernel runs on a
//     second stream under the GEMM of the next chunk;
//   * beyond that, or without peer mappings: NCCL all-reduce (optionally per token chunk on the second stream).
// NCCL is resolved at run time from the library already loaded in the process (no link-time dependency).
#include "common.cuh"
#include <dlfcn.h>
#include <stdlib.h>

int32_t b2q_fp8_quantize_rows_bf16_scratch(b2q_handle h, const void* x, int64_t rows, int64_t cols, int fmt, int rounding, float* scales,
                                           uint8_t* codes);
extern "C" int32_t b2q_grouped_gemm_fp4_rows(b2q_handle h, const uint8_t* codes, const uint8_t* scales_e8m0, const void* x_bf16,
                                             const int32_t* row_offsets, int groups, int64_t capacity_rows, int64_t N, int64_t K, int act_mode,
                                             void* out, int out_type);
int32_t b2q_grouped_gemm_fp8_rows_act(b2q_handle h, const uint8_t* a, const float* scale_a, const uint8_t* w, const float* scale_w,
                                      const int32_t* row_offsets, const int32_t* row_counts, int groups, int64_t capacity_rows, int64_t N, int64_t K,
                                      int fmt, void* out, int out_type, int act);
int32_t b2q_swiglu_quantize_rows_interleaved(b2q_handle h, const float* gu, int64_t rows, int64_t cols, int fmt, int rounding, float* scales,
                                             uint8_t* codes);
namespace tc {
struct EpiArgs { float alpha, beta; const float* bias; int act; };
int32_t gemm_fp8_impl(b2q_handle h, const uint8_t* a, const uint8_t* w, int64_t M, int64_t N, int64_t K, int fmt, const float* scale_a,
                      int scale_a_kind, const float* scale_w, int scale_w_kind, void* out, int out_type, const EpiArgs* epi);
int32_t gemm_fp8_scatter(b2q_handle h, const uint8_t* a, const uint8_t* w, int64_t M, int64_t N, int64_t K, int fmt, const float* scale_a,
                         const float* scale_w, const float* bias, void* const* inbox, int tp, int rank);
}

namespace tpx {

// ---- NCCL entry points (declared here: the ABI of these calls is stable across NCCL 2.x) -------------------
typedef void* nccl_comm_t;
struct nccl_unique_id { char internal[128]; };
enum { kNcclUint8 = 1, kNcclFloat32 = 7, kNcclBfloat16 = 9, kNcclSum = 0 };
struct NcclApi {
  int (*GetUniqueId)(nccl_unique_id*);
  int (*CommInitRank)(nccl_comm_t*, int, nccl_unique_id, int);
  int (*CommDestroy)(nccl_comm_t);
  int (*AllReduce)(const void*, void*, size_t, int, int, nccl_comm_t, cudaStream_t);
  int (*AllGather)(const void*, void*, size_t, int, nccl_comm_t, cudaStream_t);
  const char* (*GetErrorString)(int);
  bool ok;
};
static NcclApi* nccl() {
  static NcclApi api = {};
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* lib = dlopen("libnccl.so.2", RTLD_NOW | RTLD_NOLOAD);     // the copy the process already uses (torch's, the caller's)
    if (!lib) lib = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!lib) lib = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
    if (lib) {
      api.GetUniqueId = (int (*)(nccl_unique_id*))dlsym(lib, "ncclGetUniqueId");
      api.CommInitRank = (int (*)(nccl_comm_t*, int, nccl_unique_id, int))dlsym(lib, "ncclCommInitRank");
      api.CommDestroy = (int (*)(nccl_comm_t))dlsym(lib, "ncclCommDestroy");
      api.AllReduce = (int (*)(const void*, void*, size_t, int, int, nccl_comm_t, cudaStream_t))dlsym(lib, "ncclAllReduce");
      api.AllGather = (int (*)(const void*, void*, size_t, int, nccl_comm_t, cudaStream_t))dlsym(lib, "ncclAllGather");
      api.GetErrorString = (const char* (*)(int))dlsym(lib, "ncclGetErrorString");
      api.ok = api.GetUniqueId && api.CommInitRank && api.CommDestroy && api.AllReduce && api.AllGather;
    }
  }
  return &api;
}

// ---- exchange buffer layout (one per rank, cudaMalloc'ed, mapped into every peer) ---------------------------
constexpr int kMaxRanks = 8;
constexpr int kMaxCtas = 128;                                 // CTAs of an exchange kernel (same on every rank)
constexpr size_t kFlagBytes = 16384;                          // flags[2 barriers][kMaxCtas][kMaxRanks] u32 = 8 KiB, then epoch[kMaxCtas] u32
constexpr size_t kOneShotMax = 256 << 10;                     // fp32 partial bytes up to which every rank receives every partial
constexpr size_t kTwoShotMax = 4 << 20;                       // fp32 partial bytes up to which the peer kernel is used at all
constexpr size_t kSlotBytes = kTwoShotMax / 2;                // inbox slot per (parity, source rank): a two-shot slice (<= 4 MiB / 2 ranks)
constexpr size_t kInboxBytes = 2 * kMaxRanks * kSlotBytes;    // 32 MiB
constexpr size_t kResultBytes = 2 * (kTwoShotMax / 2);        // bf16 result per parity
constexpr size_t kBigMax = 64ull << 20;                       // bf16 result bytes up to which the GEMM scatters its partials itself
constexpr size_t kBigInboxOff = kFlagBytes + kInboxBytes + kResultBytes;   // [chunk][tp slots][rows / tp][N] bf16
constexpr size_t kBigResultOff = kBigInboxOff + kBigMax;                   // [chunk][rows][N] bf16
constexpr size_t kXbufBytes = kBigResultOff + kBigMax;
constexpr uint64_t kWaitLimitNs = 1000000000ull;

struct Peers { uint8_t* base[kMaxRanks]; };

__device__ __forceinline__ uint64_t globaltimer_ns() { uint64_t t; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t)); return t; }
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) { asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory"); }
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) { uint32_t v; asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory"); return v; }

__device__ __forceinline__ uint32_t* flag_ptr(uint8_t* base, int which, int cta, int src) {
  return reinterpret_cast<uint32_t*>(base) + (which * kMaxCtas + cta) * kMaxRanks + src;
}
__device__ __forceinline__ uint32_t* epoch_ptr(uint8_t* base, int cta) { return reinterpret_cast<uint32_t*>(base + 8192) + cta; }
__device__ __forceinline__ float4* inbox_ptr(uint8_t* base, int parity, int src) {
  return reinterpret_cast<float4*>(base + kFlagBytes + ((size_t)parity * kMaxRanks + src) * kSlotBytes);
}
__device__ __forceinline__ uint2* result_ptr(uint8_t* base, int parity) {
  return reinterpret_cast<uint2*>(base + kFlagBytes + kInboxBytes + (size_t)parity * (kTwoShotMax / 2));
}

// CTA-level barrier with the same CTA of every peer: everything this CTA stored before is visible to the peers'
// CTA after their wait.  Returns false when a peer did not arrive within the limit.
__device__ __forceinline__ bool peer_barrier(const Peers& peers, int tp, int rank, int which, uint32_t e, int* s_abort) {
  __threadfence_system();
  __syncthreads();
  const int cta = blockIdx.x;
  if ((int)threadIdx.x < tp) {
    st_release_sys(flag_ptr(peers.base[threadIdx.x], which, cta, rank), e);
    const uint32_t* mine = flag_ptr(peers.base[rank], which, cta, threadIdx.x);
    const uint64_t t0 = globaltimer_ns();
    uint32_t spins = 0;
    while ((int32_t)(ld_acquire_sys(mine) - e) < 0) {
      if (((++spins) & 0xFF) == 0 && globaltimer_ns() - t0 > kWaitLimitNs) { *s_abort = 1; break; }
    }
  }
  __syncthreads();
  return *s_abort == 0;
}

__device__ __forceinline__ uint2 pack4_bf16(float4 v) {
  const __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
  return make_uint2(*reinterpret_cast<const uint32_t*>(&lo), *reinterpret_cast<const uint32_t*>(&hi));
}

// partial: this rank's fp32 partial sums, n4 float4 elements; y: bf16 result (n4 * 4 elements).
template <bool TWO_SHOT>
__global__ void __launch_bounds__(512, 1) tp_allreduce_push_kernel(const Peers peers, int tp, int rank, const float4* __restrict__ partial,
                                                                    int64_t n4, uint2* __restrict__ y, int32_t* status) {
  __shared__ int s_abort;
  b2q_pdl_entry();
  if (threadIdx.x == 0) s_abort = 0;
  const int cta = blockIdx.x, G = gridDim.x;
  uint8_t* my = peers.base[rank];
  const uint32_t e = *epoch_ptr(my, cta) + 1;                  // written only by this CTA of the previous launch
  const int parity = (int)(e & 1u);
  __syncthreads();
  bool ok = true;
  if constexpr (!TWO_SHOT) {
    const int64_t per = (n4 + G - 1) / G, i0 = cta * per, i1 = min(n4, i0 + per);
    for (int r = 0; r < tp; ++r) {                             // push this CTA's range into every rank's inbox (own rank: a local copy)
      float4* dst = inbox_ptr(peers.base[r], parity, rank);
      for (int64_t i = i0 + threadIdx.x; i < i1; i += blockDim.x) dst[i] = partial[i];
    }
    ok = peer_barrier(peers, tp, rank, 0, e, &s_abort);
    if (ok) {
      for (int64_t i = i0 + threadIdx.x; i < i1; i += blockDim.x) {
        float4 acc = __ldcg(inbox_ptr(my, parity, 0) + i);
        for (int r = 1; r < tp; ++r) {                         // rank order: the reference's summation order
          const float4 v = __ldcg(inbox_ptr(my, parity, r) + i);
          acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
        }
        y[i] = pack4_bf16(acc);
      }
    }
  } else {
    const int64_t slice = n4 / tp;                             // n4 is a multiple of tp (checked by the host)
    const int64_t per = (slice + G - 1) / G, i0 = cta * per, i1 = min(slice, i0 + per);
    for (int r = 0; r < tp; ++r) {                             // slice r of my partial -> rank r
      float4* dst = inbox_ptr(peers.base[r], parity, rank);
      const float4* src = partial + r * slice;
      for (int64_t i = i0 + threadIdx.x; i < i1; i += blockDim.x) dst[i] = src[i];
    }
    ok = peer_barrier(peers, tp, rank, 0, e, &s_abort);
    if (ok) {
      for (int64_t i = i0 + threadIdx.x; i < i1; i += blockDim.x) {
        float4 acc = __ldcg(inbox_ptr(my, parity, 0) + i);
        for (int r = 1; r < tp; ++r) {
          const float4 v = __ldcg(inbox_ptr(my, parity, r) + i);
          acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
        }
        const uint2 pk = pack4_bf16(acc);
        for (int r = 0; r < tp; ++r) result_ptr(peers.base[r], parity)[rank * slice + i] = pk;   // my slice of the result -> everyone
      }
      ok = peer_barrier(peers, tp, rank, 1, e, &s_abort);
    }
    if (ok) {
      const uint2* res = result_ptr(my, parity);
      for (int r = 0; r < tp; ++r)
        for (int64_t i = i0 + threadIdx.x; i < i1; i += blockDim.x) y[r * slice + i] = __ldcg(res + r * slice + i);
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    *epoch_ptr(my, cta) = e;
    if (!ok) atomicCAS(status, 0, (int)B2Q_ERR_TIMEOUT);
  }
}

__device__ __forceinline__ void add8_bf16(float (&acc)[8], const uint4 v, bool first) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float lo = __uint_as_float(w[j] << 16), hi = __uint_as_float(w[j] & 0xFFFF0000u);
    acc[2 * j] = first ? lo : acc[2 * j] + lo;
    acc[2 * j + 1] = first ? hi : acc[2 * j + 1] + hi;
  }
}

// Second half of the many-token boundary.  Every rank's GEMM has stored its bf16 partial of MY rows into slot `src` of
// my inbox (kernels that completed before this one was launched, on every rank: the first barrier orders them).  Sum the
// tp slots in rank order in fp32, write the bf16 sums into y and into every peer's result area, wait again, copy the
// peers' rows out of my result area.  inbox: [tp][slice16] 16-byte units, result: [tp * slice16], both rows of n16 units;
// y: the same rows at a pitch of y_pitch16 units (a column range of the full result).
// TPM: ranks the instance covers (2, 4 or 8); U: pieces per thread and round, chosen so that TPM * U = 8 loads of 16 bytes
// are in flight per thread whatever the group size (the kernel is bound by NVLink and HBM latency, not by arithmetic).
template <int TPM, int U>
__global__ void __launch_bounds__(512, 1) tp_reduce_gather_kernel(const Peers peers, int tp, int rank, size_t off_inbox, size_t off_result,
                                                                   int64_t slice16, int64_t n16, int64_t y_pitch16, uint4* __restrict__ y,
                                                                   int32_t* status) {
  __shared__ int s_abort;
  if (threadIdx.x == 0) s_abort = 0;
  const int cta = blockIdx.x, G = gridDim.x;
  uint8_t* my = peers.base[rank];
  const uint32_t e = *epoch_ptr(my, cta) + 1;
  __syncthreads();
  const int64_t per = (slice16 + G - 1) / G, i0 = cta * per, i1 = min(slice16, i0 + per);
  const int64_t rows_per = slice16 / n16;                                          // rows each rank owns
  auto y_at = [&](int r, int64_t i) { const int64_t row = i / n16; return y + (r * rows_per + row) * y_pitch16 + (i - row * n16); };
  const int64_t step = (int64_t)blockDim.x * U;
  bool ok = peer_barrier(peers, tp, rank, 0, e, &s_abort);
  if (ok) {
    const uint4* in = reinterpret_cast<const uint4*>(my + off_inbox);
    for (int64_t ib = i0 + threadIdx.x; ib < i1; ib += step) {
      uint4 v[U][TPM];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int64_t i = ib + (int64_t)u * blockDim.x;
#pragma unroll
        for (int r = 0; r < TPM; ++r)
          if (r < tp && i < i1) v[u][r] = __ldcg(in + r * slice16 + i);
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int64_t i = ib + (int64_t)u * blockDim.x;
        if (i >= i1) continue;
        float acc[8];
#pragma unroll
        for (int r = 0; r < TPM; ++r)
          if (r < tp) add8_bf16(acc, v[u][r], r == 0);             // rank order: the reference's summation order
        uint4 pk;
        __nv_bfloat162 h0 = __floats2bfloat162_rn(acc[0], acc[1]), h1 = __floats2bfloat162_rn(acc[2], acc[3]);
        __nv_bfloat162 h2 = __floats2bfloat162_rn(acc[4], acc[5]), h3 = __floats2bfloat162_rn(acc[6], acc[7]);
        pk.x = *reinterpret_cast<uint32_t*>(&h0); pk.y = *reinterpret_cast<uint32_t*>(&h1);
        pk.z = *reinterpret_cast<uint32_t*>(&h2); pk.w = *reinterpret_cast<uint32_t*>(&h3);
        *y_at(rank, i) = pk;
#pragma unroll
        for (int r = 0; r < TPM; ++r)
          if (r < tp && r != rank) reinterpret_cast<uint4*>(peers.base[r] + off_result)[rank * slice16 + i] = pk;
      }
    }
    ok = peer_barrier(peers, tp, rank, 1, e, &s_abort);
  }
  if (ok) {
    const uint4* res = reinterpret_cast<const uint4*>(my + off_result);
    for (int64_t ib = i0 + threadIdx.x; ib < i1; ib += step) {     // every peer's pieces in flight at once
      uint4 v[U][TPM];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int64_t i = ib + (int64_t)u * blockDim.x;
#pragma unroll
        for (int r = 0; r < TPM; ++r)
          if (r < tp && r != rank && i < i1) v[u][r] = __ldcg(res + r * slice16 + i);
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int64_t i = ib + (int64_t)u * blockDim.x;
#pragma unroll
        for (int r = 0; r < TPM; ++r)
          if (r < tp && r != rank && i < i1) *y_at(r, i) = v[u][r];
      }
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    *epoch_ptr(my, cta) = e;
    if (!ok) atomicCAS(status, 0, (int)B2Q_ERR_TIMEOUT);
  }
}

// Rows of a and b interleaved in blocks of `block` rows: out rows [2 j block, 2 j block + block) = a rows [j block, ...),
// the next `block` rows the same rows of b; 16-byte pieces of the rows.
__global__ void __launch_bounds__(256) interleave_rows_kernel(const uint4* __restrict__ a, const uint4* __restrict__ b, uint4* __restrict__ out,
                                                              int64_t rows, int64_t row16, int64_t block) {
  const int64_t total = 2 * rows * row16;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t orow = i / row16, c = i - orow * row16, blk = orow / (2 * block), in = orow - blk * 2 * block;
    const int64_t src = blk * block + (in < block ? in : in - block);
    out[i] = (in < block ? a : b)[src * row16 + c];
  }
}

// h[r, f] = silu(gu[r, f]) * gu[r, F + f] (bf16 in and out, fp32 inside), eight columns per thread
__global__ void __launch_bounds__(256) swiglu_bf16_kernel(const uint4* __restrict__ gu, uint4* __restrict__ hout, int64_t rows, int64_t F8) {
  const int64_t total = rows * F8;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / F8, c = i - r * F8;
    const uint4 g = gu[r * 2 * F8 + c], u = gu[r * 2 * F8 + F8 + c];
    const uint32_t gw[4] = {g.x, g.y, g.z, g.w}, uw[4] = {u.x, u.y, u.z, u.w};
    uint32_t o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float g0 = __uint_as_float(gw[j] << 16), g1 = __uint_as_float(gw[j] & 0xFFFF0000u);
      const float u0 = __uint_as_float(uw[j] << 16), u1 = __uint_as_float(uw[j] & 0xFFFF0000u);
      const __nv_bfloat162 hv = __floats2bfloat162_rn(__fdiv_rn(g0, 1.0f + expf(-g0)) * u0, __fdiv_rn(g1, 1.0f + expf(-g1)) * u1);
      o[j] = *reinterpret_cast<const uint32_t*>(&hv);
    }
    hout[i] = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

// y[t, c] += bias[c]  (bf16 rows, f32 bias)
__global__ void __launch_bounds__(256) bias_add_bf16_kernel(__nv_bfloat16* __restrict__ y, const float* __restrict__ bias, int64_t rows, int64_t cols) {
  const int64_t total = rows * cols;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x)
    y[i] = __float2bfloat16_rn(__bfloat162float(y[i]) + bias[i % cols]);
}
__global__ void __launch_bounds__(256) bias_add_f32_kernel(float* __restrict__ y, const float* __restrict__ bias, int64_t rows, int64_t cols) {
  const int64_t total = rows * cols;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) y[i] += bias[i % cols];
}
// gathered[t, r * local + c] = parts[r][t][c]  (16-byte pieces; local * 2 bytes is a multiple of 16)
__global__ void __launch_bounds__(256) gather_columns_kernel(const uint4* __restrict__ parts, uint4* __restrict__ out, int tp, int64_t rows,
                                                             int64_t local_vec) {
  const int64_t total = (int64_t)tp * rows * local_vec;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t c = i % local_vec, t = (i / local_vec) % rows, r = i / (local_vec * rows);
    out[(t * tp + r) * local_vec + c] = parts[i];
  }
}

}  // namespace tpx

struct b2q_tp_s {
  b2q_handle h;
  tpx::nccl_comm_t comm;
  int tp, rank;
  int chunks;                      // token chunks of the many-token path (0 = choose by size)
  int no_scatter;                  // B2Q_TP_SCATTER=0: many-token boundaries take NCCL (experiments, comparison runs)
  cudaStream_t comm_stream;
  cudaEvent_t ev_ready[16], ev_done;
  uint8_t* xbuf;                   // this rank's exchange buffer
  tpx::Peers peers;                // every rank's exchange buffer as mapped here
  int attached;
  // grow-only scratch of the MLP / linears
  void* scratch;
  size_t scratch_bytes;
};

namespace tpx {

static int32_t scratch(b2q_tp t, size_t bytes, uint8_t** out) {
  if (bytes > t->scratch_bytes) {
    b2q_handle h = t->h;
    B2Q_CUDA(h, cudaStreamSynchronize(h->stream));
    B2Q_CUDA(h, cudaStreamSynchronize(t->comm_stream));
    if (t->scratch) cudaFree(t->scratch);
    t->scratch = nullptr;
    t->scratch_bytes = 0;
    B2Q_CUDA(h, cudaMalloc(&t->scratch, bytes));
    t->scratch_bytes = bytes;
    // rows that no call ever writes (padding between experts) are read by the row quantizers: give them finite values
    B2Q_CUDA(h, cudaMemsetAsync(t->scratch, 0, bytes, h->stream));
  }
  *out = reinterpret_cast<uint8_t*>(t->scratch);
  return B2Q_OK;
}
static inline size_t align256(size_t v) { return (v + 255) & ~(size_t)255; }

// Sum of the ranks' fp32 partials [n floats] -> bf16 y on every rank, through the peer kernel.
static int32_t peer_allreduce(b2q_tp t, const float* partial, int64_t n, void* y) {
  b2q_handle h = t->h;
  const size_t bytes = (size_t)n * 4;
  const bool two = bytes > kOneShotMax;
  const int64_t n4 = n / 4;
  int grid = (int)((n4 + 511) / 512);
  if (two) grid = (int)((n4 / t->tp + 511) / 512);
  grid = grid < 1 ? 1 : (grid > kMaxCtas ? kMaxCtas : grid);
  if (two)
    B2Q_CUDA(h, b2q_pdl_launch(h->sw.chain_pdl != 0, tp_allreduce_push_kernel<true>, dim3(grid), dim3(512), 0, h->stream, t->peers, t->tp, t->rank,
                               (const float4*)partial, n4, (uint2*)y, h->d_status));
  else
    B2Q_CUDA(h, b2q_pdl_launch(h->sw.chain_pdl != 0, tp_allreduce_push_kernel<false>, dim3(grid), dim3(512), 0, h->stream, t->peers, t->tp, t->rank,
                               (const float4*)partial, n4, (uint2*)y, h->d_status));
  B2Q_LAUNCH_CHECK(h, "tp_allreduce_push_kernel");
  return B2Q_OK;
}
// Column chunk `chunk` of `chunks` of a row-parallel linear over all `tokens`: the scatter GEMM over rows
// [chunk * nc, (chunk + 1) * nc) of W (nc = N / chunks) and the kernel that sums and gathers those columns into y.
// With several chunks the second kernel runs on the exchange stream, under the GEMM of the next chunk.
static int32_t scatter_reduce_cols(b2q_tp t, const uint8_t* x_codes, const float* x_scales, const uint8_t* w_codes, const float* w_scales,
                                   const float* bias, int64_t tokens, int64_t in_local, int64_t N, void* y, int chunk, int chunks) {
  b2q_handle h = t->h;
  const int64_t nc = N / chunks;
  const size_t off = (size_t)chunk * tokens * nc * 2;
  void* inbox[kMaxRanks] = {};
  for (int r = 0; r < t->tp; ++r) inbox[r] = t->peers.base[r] + kBigInboxOff + off;
  int32_t st = tc::gemm_fp8_scatter(h, x_codes, w_codes + (size_t)chunk * nc * in_local, tokens, nc, in_local, B2Q_FP8_E4M3, x_scales,
                                    w_scales + chunk * nc, bias ? bias + chunk * nc : nullptr, inbox, t->tp, t->rank);
  if (st == B2Q_ERR_UNSUPPORTED)
    B2Q_FAIL(h, B2Q_ERR_UNSUPPORTED, "row-parallel scatter GEMM: shape %lld x %lld x %lld not covered", (long long)tokens, (long long)nc, (long long)in_local);
  if (st != B2Q_OK) return st;
  cudaStream_t rs = chunks > 1 ? t->comm_stream : h->stream;
  if (chunks > 1) {
    B2Q_CUDA(h, cudaEventRecord(t->ev_ready[chunk], h->stream));
    B2Q_CUDA(h, cudaStreamWaitEvent(rs, t->ev_ready[chunk], 0));
  }
  const int64_t n16 = nc * 2 / 16, slice16 = (tokens / t->tp) * n16;
  // alone on the stream: 512 threads per CTA; under the next chunk's GEMM: 256 threads and no shared memory beyond one word,
  // a CTA that fits beside a resident GEMM CTA
  const int threads = chunks > 1 ? 256 : 512;
  int grid = (int)((slice16 + threads - 1) / threads);
  grid = grid < 1 ? 1 : (grid > kMaxCtas ? kMaxCtas : grid);
  uint4* yc = reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(y) + (size_t)chunk * nc * 2);
#define B2Q_RG_LAUNCH(TPM, U)                                                                                                          \
  tp_reduce_gather_kernel<TPM, U><<<grid, threads, 0, rs>>>(t->peers, t->tp, t->rank, kBigInboxOff + off, kBigResultOff + off, slice16, n16, \
                                                            N * 2 / 16, yc, h->d_status)
  if (t->tp <= 2) B2Q_RG_LAUNCH(2, 4);
  else if (t->tp <= 4) B2Q_RG_LAUNCH(4, 2);
  else B2Q_RG_LAUNCH(8, 1);
#undef B2Q_RG_LAUNCH
  B2Q_LAUNCH_CHECK(h, "tp_reduce_gather_kernel");
  if (chunks > 1 && chunk == chunks - 1) {
    B2Q_CUDA(h, cudaEventRecord(t->ev_done, rs));
    B2Q_CUDA(h, cudaStreamWaitEvent(h->stream, t->ev_done, 0));
  }
  return B2Q_OK;
}
// Shapes the scatter GEMM and the 16-byte units of the reduce kernel cover (nc: the columns of one chunk).
static bool scatter_fits(int tp, int64_t tokens, int64_t nc, int64_t in_local) {
  return tokens > 128 && nc > 128 && tokens % (32 * tp) == 0 && nc % 8 == 0 && in_local % 16 == 0;
}

static bool peer_path_fits(b2q_tp t, int64_t n) {
  return t->attached && n % (4 * t->tp) == 0 && (size_t)n * 4 <= kTwoShotMax && ((size_t)n * 4 / t->tp) <= kSlotBytes;
}

static int32_t add_bias(b2q_handle h, void* y, int out_type, const float* bias, int64_t rows, int64_t cols) {
  if (!bias) return B2Q_OK;
  const int64_t total = rows * cols;
  int grid = (int)((total + 255) / 256);
  if (grid > h->sm_count * 8) grid = h->sm_count * 8;
  if (out_type == B2Q_OUT_BF16) bias_add_bf16_kernel<<<grid, 256, 0, h->stream>>>((__nv_bfloat16*)y, bias, rows, cols);
  else bias_add_f32_kernel<<<grid, 256, 0, h->stream>>>((float*)y, bias, rows, cols);
  B2Q_LAUNCH_CHECK(h, "bias_add_kernel");
  return B2Q_OK;
}

// The boundary of one call: the plan for the shape, the caller's chunk override, and the fall-back to NCCL when the
// operands do not suit the scatter GEMM (K pitch, alignment).
static void choose_boundary(b2q_tp t, int64_t tokens, int64_t out_features, int64_t in_local, const void* a, const void* w, int* mode,
                            int* chunks) {
  b2q_tp_plan(t->tp, t->attached, tokens, out_features, mode, chunks);
  if (*mode == 4 && (t->no_scatter || in_local % 16 != 0 || ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(w)) & 15) != 0)) {
    *mode = 3;
    *chunks = 1;
  }
  if (t->chunks > 0) {                                       // mode 3: token chunks; mode 4: column chunks
    if (*mode == 3 && tokens % t->chunks == 0 && (t->chunks == 1 || (tokens / t->chunks) % 256 == 0)) *chunks = t->chunks;
    if (*mode == 4 && out_features % (8 * t->chunks) == 0 && scatter_fits(t->tp, tokens, out_features / t->chunks, in_local)) *chunks = t->chunks;
  }
}

}  // namespace tpx

#define B2Q_REQUIRE_TP(t)                                                 \
  do {                                                                    \
    if (!(t) || !(t)->h) return (int32_t)B2Q_ERR_INVALID_ARGUMENT;        \
    B2Q_REQUIRE_HANDLE((t)->h);                                           \
  } while (0)
#define B2Q_NCCL(h, expr)                                                                                       \
  do {                                                                                                          \
    int _r = (expr);                                                                                            \
    if (_r != 0) B2Q_FAIL(h, B2Q_ERR_NCCL, "%s: %s", #expr, tpx::nccl()->GetErrorString ? tpx::nccl()->GetErrorString(_r) : "NCCL error"); \
  } while (0)

extern "C" {

int32_t b2q_tp_unique_id(uint8_t* id128) {
  if (!id128 || !tpx::nccl()->ok) return B2Q_ERR_NCCL;
  tpx::nccl_unique_id id;
  if (tpx::nccl()->GetUniqueId(&id) != 0) return B2Q_ERR_NCCL;
  memcpy(id128, id.internal, 128);
  return B2Q_OK;
}

int32_t b2q_tp_comm_init(const uint8_t* id128, int tp, int rank, void** comm) {
  if (!id128 || !comm || tp < 1 || rank < 0 || rank >= tp || !tpx::nccl()->ok) return B2Q_ERR_NCCL;
  tpx::nccl_unique_id id;
  memcpy(id.internal, id128, 128);
  tpx::nccl_comm_t c = nullptr;
  if (tpx::nccl()->CommInitRank(&c, tp, id, rank) != 0) return B2Q_ERR_NCCL;
  *comm = c;
  return B2Q_OK;
}

int32_t b2q_tp_comm_destroy(void* comm) {
  if (!comm) return B2Q_OK;
  return tpx::nccl()->ok && tpx::nccl()->CommDestroy(comm) == 0 ? B2Q_OK : B2Q_ERR_NCCL;
}

int32_t b2q_tp_create(b2q_handle h, void* nccl_comm, int tp, int rank, b2q_tp* out) {
  B2Q_REQUIRE_HANDLE(h);
  if (!out) B2Q_FAIL(h, B2Q_ERR_INVALID_ARGUMENT, "tp_create: null output");
  *out = nullptr;
  if (tp < 1 || tp > tpx::kMaxRanks || rank < 0 || rank >= tp)
    B2Q_FAIL(h, B2Q_ERR_INVALID_ARGUMENT, "tp_create: tp must be in [1, %d] and rank in [0, tp), got tp=%d rank=%d", tpx::kMaxRanks, tp, rank);
  if (tp > 1 && !nccl_comm) B2Q_FAIL(h, B2Q_ERR_INVALID_ARGUMENT, "tp_create: a communicator is required for tp > 1");
  if (tp > 1 && !tpx::nccl()->ok) B2Q_FAIL(h, B2Q_ERR_NCCL, "tp_create: libnccl.so.2 could not be resolved in this process");
  b2q_tp t = new b2q_tp_s();
  memset(t, 0, sizeof(*t));
  t->h = h; t->comm = nccl_comm; t->tp = tp; t->rank = rank;
  const char* ce = getenv("B2Q_TP_CHUNKS");
  t->chunks = ce ? atoi(ce) : 0;
  const char* se = getenv("B2Q_TP_SCATTER");
  t->no_scatter = se && atoi(se) == 0;
  // the exchange stream outranks the GEMM stream: its few CTAs are placed as soon as an SM has room for them
  int prio_lo = 0, prio_hi = 0;
  cudaDeviceGetStreamPriorityRange(&prio_lo, &prio_hi);
  bool ok = cudaStreamCreateWithPriority(&t->comm_stream, cudaStreamNonBlocking, prio_hi) == cudaSuccess;
  // an SM keeps one shared-memory split while CTAs are resident: the sum-and-gather kernel asks for the split the GEMM
  // CTAs run under (all of it shared), or it could not become resident beside them, nor they beside it
  ok = ok && cudaFuncSetAttribute(tpx::tp_reduce_gather_kernel<2, 4>, cudaFuncAttributePreferredSharedMemoryCarveout,
                                  (int)cudaSharedmemCarveoutMaxShared) == cudaSuccess;
  ok = ok && cudaFuncSetAttribute(tpx::tp_reduce_gather_kernel<4, 2>, cudaFuncAttributePreferredSharedMemoryCarveout,
                                  (int)cudaSharedmemCarveoutMaxShared) == cudaSuccess;
  ok = ok && cudaFuncSetAttribute(tpx::tp_reduce_gather_kernel<8, 1>, cudaFuncAttributePreferredSharedMemoryCarveout,
                                  (int)cudaSharedmemCarveoutMaxShared) == cudaSuccess;
  for (int i = 0; i < 16 && ok; ++i) ok = cudaEventCreateWithFlags(&t->ev_ready[i], cudaEventDisableTiming) == cudaSuccess;
  ok = ok && cudaEventCreateWithFlags(&t->ev_done, cudaEventDisableTiming) == cudaSuccess;
  if (ok && tp > 1) {
    ok = cudaMalloc(&t->xbuf, tpx::kXbufBytes) == cudaSuccess && cudaMemset(t->xbuf, 0, tpx::kFlagBytes) == cudaSuccess;
    t->peers.base[rank] = t->xbuf;
  }
  if (!ok) {
    b2q_tp_destroy(t);
    B2Q_FAIL(h, B2Q_ERR_CUDA, "tp_create: stream, event or exchange-buffer creation failed: %s", cudaGetErrorString(cudaGetLastError()));
  }
  *out = t;
  return B2Q_OK;
}

int32_t b2q_tp_destroy(b2q_tp t) {
  if (!t) return B2Q_OK;
  if (t->comm_stream) { cudaStreamSynchronize(t->comm_stream); cudaStreamDestroy(t->comm_stream); }
  for (int i = 0; i < 16; ++i) if (t->ev_ready[i]) cudaEventDestroy(t->ev_ready[i]);
  if (t->ev_done) cudaEventDestroy(t->ev_done);
  if (t->attached == 1) {
    for (int r = 0; r < t->tp; ++r) if (r != t->rank && t->peers.base[r]) cudaIpcCloseMemHandle(t->peers.base[r]);
  }
  if (t->xbuf) cudaFree(t->xbuf);
  if (t->scratch) cudaFree(t->scratch);
  delete t;
  return B2Q_OK;
}

int32_t b2q_tp_set_chunks(b2q_tp t, int chunks) {
  B2Q_REQUIRE_TP(t);
  if (chunks < 0 || chunks > 16) B2Q_FAIL(t->h, B2Q_ERR_INVALID_ARGUMENT, "tp_set_chunks: 0 (automatic) to 16, got %d", chunks);
  t->chunks = chunks;
  return B2Q_OK;
}

int32_t b2q_tp_exchange_buffer(b2q_tp t, void** ptr, uint8_t* ipc_handle64) {
  B2Q_REQUIRE_TP(t);
  if (t->tp == 1) B2Q_FAIL(t->h, B2Q_ERR_UNSUPPORTED, "tp_exchange_buffer: a single rank has no exchange buffer");
  if (ptr) *ptr = t->xbuf;
  if (ipc_handle64) {
    cudaIpcMemHandle_t hd;
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    B2Q_CUDA(t->h, cudaIpcGetMemHandle(&hd, t->xbuf));
    memcpy(ipc_handle64, &hd, 64);
  }
  return B2Q_OK;
}

int32_t b2q_tp_attach_peers(b2q_tp t, const uint8_t* ipc_handles, void* const* direct_ptrs) {
  B2Q_REQUIRE_TP(t);
  if (t->tp == 1) return B2Q_OK;
  if (t->attached) B2Q_FAIL(t->h, B2Q_ERR_INVALID_ARGUMENT, "tp_attach_peers: peers are attached already");
  if (!ipc_handles && !direct_ptrs) B2Q_FAIL(t->h, B2Q_ERR_INVALID_ARGUMENT, "tp_attach_peers: pass IPC handles or mapped pointers");
  for (int r = 0; r < t->tp; ++r) {
    if (r == t->rank) continue;
    if (direct_ptrs) {
      t->peers.base[r] = reinterpret_cast<uint8_t*>(direct_ptrs[r]);
    } else {
      cudaIpcMemHandle_t hd;
      memcpy(&hd, ipc_handles + 64 * r, 64);
      void* p = nullptr;
      B2Q_CUDA(t->h, cudaIpcOpenMemHandle(&p, hd, cudaIpcMemLazyEnablePeerAccess));
      t->peers.base[r] = reinterpret_cast<uint8_t*>(p);
    }
    if (!t->peers.base[r]) B2Q_FAIL(t->h, B2Q_ERR_INVALID_ARGUMENT, "tp_attach_peers: no mapping for rank %d", r);
  }
  t->attached = direct_ptrs ? 2 : 1;
  return B2Q_OK;
}

// Which boundary a row-parallel result of `tokens` x `out_features` takes: 0 none (tp = 1), 1 one-shot peer kernel,
// 2 two-shot peer kernel, 4 reduce-scatter stored by the GEMM epilogue into the owners' inboxes + one sum-and-gather
// kernel per token chunk, 3 NCCL all-reduce per token chunk.  `chunks` is the automatic choice; b2q_tp_set_chunks
// overrides it where the chunked shapes still fit.
int32_t b2q_tp_plan(int tp, int peers_attached, int64_t tokens, int64_t out_features, int* mode, int* chunks) {
  if (!mode || !chunks || tp < 1 || tokens < 1 || out_features < 1) return B2Q_ERR_INVALID_ARGUMENT;
  *chunks = 1;
  if (tp == 1) { *mode = 0; return B2Q_OK; }
  const int64_t n = tokens * out_features;
  const size_t bytes = (size_t)n * 4;
  if (peers_attached && n % (4 * tp) == 0 && bytes <= tpx::kTwoShotMax) {
    *mode = bytes <= tpx::kOneShotMax ? 1 : 2;
    return B2Q_OK;
  }
  if (peers_attached && (size_t)n * 2 <= tpx::kBigMax && tpx::scatter_fits(tp, tokens, out_features, 16)) {
    *mode = 4;                    // one chunk: at tp = 2 the sum-and-gather kernel adds 30-40 us to a 64 MiB result, and
    return B2Q_OK;                // a second GEMM launch plus the stream hand-over cost as much as overlapping half of it saves
  }
  *mode = 3;                      // one all-reduce after the GEMM measured fastest at tp = 2 and 4 (NCCL's CTAs wait for the
  return B2Q_OK;                  // persistent GEMM's SMs, so chunks do not overlap)
}

int32_t b2q_tp_all_reduce_f32_to_bf16(b2q_tp t, const float* partial, int64_t n, void* y_bf16) {
  B2Q_REQUIRE_TP(t);
  b2q_handle h = t->h;
  if (!partial || !y_bf16 || n <= 0) B2Q_FAIL(h, B2Q_ERR_INVALID_ARGUMENT, "tp_all_reduce: bad argument");
  if (t->tp == 1 || !tpx::peer_path_fits(t, n))
    B2Q_FAIL(h, B2Q_ERR_UNSUPPORTED, "tp_all_reduce_f32_to_bf16: needs attached peers, n %% (4 * tp) == 0 and at most %zu bytes of partials", tpx::kTwoShotMax);
  return tpx::peer_allreduce(t, partial, n, y_bf16);
}

int32_t b2q_tp_all_reduce_bf16(b2q_tp t, void* y_bf16, int64_t n) {
  B2Q_REQUIRE_TP(t);
  if (t->tp == 1) return B2Q_OK;
  if (!y_bf16 || n <= 0) B2Q_FAIL(t->h, B2Q_ERR_INVALID_ARGUMENT, "tp_all_reduce: bad argument");
  B2Q_NCCL(t->h, tpx::nccl()->AllReduce(y_bf16, y_bf16, (size_t)n, tpx::kNcclBfloat16, tpx::kNcclSum, t->comm, t->h->stream));
  return B2Q_OK;
}

// ColumnLinear::forward (column_parallel.rs:168-179): y_local = x W_s^T + b_s over this rank's out/tp rows of W;
// with y_gathered != NULL also ColumnLinear::all_gather (:181-204): shard r lands at columns [r * out_local, ...).
int32_t b2q_column_linear_forward(b2q_tp t, const uint8_t* x_codes, const float* x_scales, const uint8_t* w_codes, const float* w_scales,
                                  const float* bias, int64_t tokens, int64_t in_features, int64_t out_local, void* y_local,
                                  void* y_gathered) {
  B2Q_REQUIRE_TP(t);
  b2q_handle h = t->h;
  int32_t st = b2q_gemm_fp8(h, x_codes, w_codes, tokens, out_local, in_features, B2Q_FP8_E4M3, x_scales, B2Q_SCALE_PER_ROW, w_scales,
                            B2Q_SCALE_PER_ROW, y_local, B2Q_OUT_BF16);
  if (st != B2Q_OK) return st;
  st = tpx::add_bias(h, y_local, B2Q_OUT_BF16, bias, tokens, out_local);
  if (st != B2Q_OK || !y_gathered) return st;
  if (t->tp == 1) {
    B2Q_CUDA(h, cudaMemcpyAsync(y_gathered, y_local, (size_t)tokens * out_local * 2, cudaMemcpyDeviceToDevice, h->stream));
    return B2Q_OK;
  }
  if ((out_local * 2) % 16 != 0) B2Q_FAIL(h, B2Q_ERR_INVALID_DIMENSION, "column_linear_forward: out_local must be a multiple of 8 to gather");
  uint8_t* parts = nullptr;
  const size_t part_bytes = (size_t)tokens * out_local * 2;
  st = tpx::scratch(t, part_bytes * t->tp, &parts);
  if (st != B2Q_OK) return st;
  B2Q_NCCL(h, tpx::nccl()->AllGather(y_local, parts, part_bytes, tpx::kNcclUint8, t->comm, h->stream));
  const int64_t total = (int64_t)t->tp * tokens * (out_local * 2 / 16);
  int grid = (int)((total + 255) / 256);
  if (grid > h->sm_count * 8) grid = h->sm_count * 8;
  tpx::gather_columns_kernel<<<grid, 256, 0, h->stream>>>((const uint4*)parts, (uint4*)y_gathered, t->tp, tokens, out_local * 2 / 16);
  B2Q_LAUNCH_CHECK(h, "gather_columns_kernel");
  return B2Q_OK;
}

// One token range of a row-parallel linear and its boundary.  x_codes / x_scales / y point at the range.
static int32_t row_linear_range(b2q_tp t, const uint8_t* x_codes, const float* x_scales, const uint8_t* w_codes, const float* w_scales,
                                const float* bias, int64_t tokens, int64_t in_local, int64_t out_features, void* y, int mode,
                                float* partial_f32) {
  b2q_handle h = t->h;
  const float* b = t->rank == 0 ? bias : nullptr;             // RowLinear adds the bias on rank 0 only (row_parallel.rs:183-190)
  if (mode == 1 || mode == 2) {
    int32_t st = b2q_gemm_fp8(h, x_codes, w_codes, tokens, out_features, in_local, B2Q_FP8_E4M3, x_scales, B2Q_SCALE_PER_ROW, w_scales,
                              B2Q_SCALE_PER_ROW, partial_f32, B2Q_OUT_F32);
    if (st != B2Q_OK) return st;
    st = tpx::add_bias(h, partial_f32, B2Q_OUT_F32, b, tokens, out_features);
    if (st != B2Q_OK) return st;
    return tpx::peer_allreduce(t, partial_f32, tokens * out_features, y);
  }
  int32_t st = b2q_gemm_fp8(h, x_codes, w_codes, tokens, out_features, in_local, B2Q_FP8_E4M3, x_scales, B2Q_SCALE_PER_ROW, w_scales,
                            B2Q_SCALE_PER_ROW, y, B2Q_OUT_BF16);
  if (st != B2Q_OK) return st;
  return tpx::add_bias(h, y, B2Q_OUT_BF16, b, tokens, out_features);
}

// RowLinear::forward + all_reduce (row_parallel.rs:170-223): y = sum over ranks of x_s W_s^T (+ bias once).
int32_t b2q_row_linear_forward_allreduce(b2q_tp t, const uint8_t* x_codes, const float* x_scales, const uint8_t* w_codes,
                                         const float* w_scales, const float* bias, int64_t tokens, int64_t in_local, int64_t out_features,
                                         void* y) {
  B2Q_REQUIRE_TP(t);
  b2q_handle h = t->h;
  if (tokens <= 0 || in_local <= 0 || out_features <= 0)
    B2Q_FAIL(h, B2Q_ERR_INVALID_DIMENSION, "row_linear_forward: dimensions must be non-zero: tokens=%lld, in=%lld, out=%lld", (long long)tokens,
             (long long)in_local, (long long)out_features);
  int mode = 0, chunks = 1;
  tpx::choose_boundary(t, tokens, out_features, in_local, x_codes, w_codes, &mode, &chunks);
  uint8_t* ws = nullptr;
  if (mode == 1 || mode == 2) {
    int32_t st = tpx::scratch(t, (size_t)tokens * out_features * 4, &ws);
    if (st != B2Q_OK) return st;
  }
  if (mode < 3) return row_linear_range(t, x_codes, x_scales, w_codes, w_scales, bias, tokens, in_local, out_features, y, mode, (float*)ws);
  if (mode == 4) {
    const float* b = t->rank == 0 ? bias : nullptr;           // RowLinear adds the bias on rank 0 only (row_parallel.rs:183-190)
    for (int c = 0; c < chunks; ++c) {
      int32_t st = tpx::scatter_reduce_cols(t, x_codes, x_scales, w_codes, w_scales, b, tokens, in_local, out_features, y, c, chunks);
      if (st != B2Q_OK) return st;
    }
    return B2Q_OK;
  }
  const int64_t ct = tokens / chunks;
  for (int c = 0; c < chunks; ++c) {
    uint8_t* yc = reinterpret_cast<uint8_t*>(y) + (size_t)c * ct * out_features * 2;
    int32_t st = row_linear_range(t, x_codes + (size_t)c * ct * in_local, x_scales + c * ct, w_codes, w_scales, bias, ct, in_local,
                                  out_features, yc, 3, nullptr);
    if (st != B2Q_OK) return st;
    B2Q_CUDA(h, cudaEventRecord(t->ev_ready[c], h->stream));
    B2Q_CUDA(h, cudaStreamWaitEvent(t->comm_stream, t->ev_ready[c], 0));
    B2Q_NCCL(h, tpx::nccl()->AllReduce(yc, yc, (size_t)ct * out_features, tpx::kNcclBfloat16, tpx::kNcclSum, t->comm, t->comm_stream));
  }
  B2Q_CUDA(h, cudaEventRecord(t->ev_done, t->comm_stream));
  B2Q_CUDA(h, cudaStreamWaitEvent(h->stream, t->ev_done, 0));
  return B2Q_OK;
}

// The tensor-parallel SwiGLU MLP: per-token E4M3 quantization of x, gate|up column-parallel GEMM (one GEMM over the
// concatenated [2 * ffn_local x hidden] shard), SwiGLU + per-token re-quantization over this rank's columns, down
// row-parallel GEMM, sum over ranks.  y: bf16 [tokens x hidden], the same on every rank.
int32_t b2q_mlp_swiglu_fp8_forward(b2q_tp t, const void* x_bf16, const uint8_t* w_gate_up, const float* s_gate_up, const uint8_t* w_down,
                                   const float* s_down, int64_t tokens, int64_t hidden, int64_t ffn_local, int rounding, void* y_bf16) {
  return b2q_mlp_swiglu_fp8_forward_ex(t, x_bf16, w_gate_up, s_gate_up, w_down, s_down, tokens, hidden, ffn_local, rounding,
                                       B2Q_GATE_UP_CONCATENATED, y_bf16);
}

// out (2 * rows x row_bytes) = rows of a and b interleaved per 128: the gate | up weight layout whose GEMM tiles hold both
// projections of the same 128 hidden units (codes: row_bytes = in_features; scales: row_bytes = 4).
int32_t b2q_interleave_rows128(b2q_handle h, const void* a, const void* b, int64_t rows, int64_t row_bytes, void* out) {
  B2Q_REQUIRE_HANDLE(h);
  if (!a || !b || !out || rows <= 0 || row_bytes <= 0) B2Q_FAIL(h, B2Q_ERR_INVALID_ARGUMENT, "interleave_rows128: bad argument");
  if (rows % 128 != 0) B2Q_FAIL(h, B2Q_ERR_INVALID_DIMENSION, "interleave_rows128: rows must be a multiple of 128, got %lld", (long long)rows);
  if (row_bytes % 16 != 0 && row_bytes != 4) B2Q_FAIL(h, B2Q_ERR_INVALID_DIMENSION, "interleave_rows128: rows of 4 bytes or a multiple of 16 bytes");
  if (((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b) | reinterpret_cast<uintptr_t>(out)) & 15) != 0)
    B2Q_FAIL(h, B2Q_ERR_INVALID_ARGUMENT, "interleave_rows128: 16-byte aligned pointers");
  // 128 four-byte rows are one 512-byte row of a matrix interleaved per single row
  const int64_t krows = row_bytes == 4 ? rows / 128 : rows, row16 = row_bytes == 4 ? 32 : row_bytes / 16, block = row_bytes == 4 ? 1 : 128;
  const int64_t total = 2 * krows * row16;
  int grid = (int)((total + 255) / 256);
  if (grid > h->sm_count * 16) grid = h->sm_count * 16;
  tpx::interleave_rows_kernel<<<grid, 256, 0, h->stream>>>((const uint4*)a, (const uint4*)b, (uint4*)out, krows, row16, block);
  B2Q_LAUNCH_CHECK(h, "interleave_rows_kernel");
  return B2Q_OK;
}

int32_t b2q_mlp_swiglu_fp8_forward_ex(b2q_tp t, const void* x_bf16, const uint8_t* w_gate_up, const float* s_gate_up, const uint8_t* w_down,
                                      const float* s_down, int64_t tokens, int64_t hidden, int64_t ffn_local, int rounding, int gate_up_layout,
                                      void* y_bf16) {
  B2Q_REQUIRE_TP(t);
  b2q_handle h = t->h;
  if (gate_up_layout != B2Q_GATE_UP_CONCATENATED && gate_up_layout != B2Q_GATE_UP_INTERLEAVED128)
    B2Q_FAIL(h, B2Q_ERR_INVALID_ARGUMENT, "mlp_swiglu_fp8_forward: unknown gate | up layout %d", gate_up_layout);
  if (gate_up_layout == B2Q_GATE_UP_INTERLEAVED128 && ffn_local % 128 != 0)
    B2Q_FAIL(h, B2Q_ERR_INVALID_DIMENSION, "mlp_swiglu_fp8_forward: the interleaved layout needs ffn_local %% 128 == 0, got %lld", (long long)ffn_local);
  const bool inter = gate_up_layout == B2Q_GATE_UP_INTERLEAVED128;
  if (tokens <= 0 || hidden <= 0 || ffn_local <= 0)
    B2Q_FAIL(h, B2Q_ERR_INVALID_DIMENSION, "mlp_swiglu_fp8_forward: dimensions must be non-zero: tokens=%lld, hidden=%lld, ffn=%lld",
             (long long)tokens, (long long)hidden, (long long)ffn_local);
  if (!x_bf16 || !w_gate_up || !s_gate_up || !w_down || !s_down || !y_bf16) B2Q_FAIL(h, B2Q_ERR_INVALID_ARGUMENT, "mlp_swiglu_fp8_forward: null operand");
  int mode = 0, chunks = 1;
  tpx::choose_boundary(t, tokens, hidden, ffn_local, w_gate_up, w_down, &mode, &chunks);
  const int col_chunks = mode == 4 ? chunks : 1;             // mode 4 cuts the down projection's columns, mode 3 the tokens
  if (mode == 4) chunks = 1;
  const int64_t ct = tokens / chunks;
  const int64_t F = ffn_local;
  // scratch: x codes + scales (all tokens), then per chunk: gate|up bf16, h codes + scales, fp32 partial (peer modes)
  const size_t o_xc = 0, o_xs = o_xc + tpx::align256((size_t)tokens * hidden), o_gu = o_xs + tpx::align256((size_t)tokens * 4),
               o_hc = o_gu + tpx::align256((size_t)ct * 2 * F * (ct <= 128 ? 4 : 2)), o_hs = o_hc + tpx::align256((size_t)ct * F),
               o_pf = o_hs + tpx::align256((size_t)ct * 4),
               total = o_pf + ((mode == 1 || mode == 2) ? tpx::align256((size_t)tokens * hidden * 4) : 0);
  uint8_t* ws = nullptr;
  int32_t st = tpx::scratch(t, total, &ws);
  if (st != B2Q_OK) return st;
  uint8_t* xc = ws + o_xc; float* xs = (float*)(ws + o_xs);
  uint8_t* gu = ws + o_gu; uint8_t* hc = ws + o_hc; float* hs = (float*)(ws + o_hs); float* pf = (float*)(ws + o_pf);
  st = b2q_fp8_quantize_rows_bf16(h, x_bf16, tokens, hidden, B2Q_FP8_E4M3, rounding, xs, xc);
  if (st != B2Q_OK) return st;
  for (int c = 0; c < chunks; ++c) {
    const uint8_t* xcc = xc + (size_t)c * ct * hidden;
    uint8_t* yc = reinterpret_cast<uint8_t*>(y_bf16) + (size_t)c * ct * hidden * 2;
    if (inter && ct > 128) {
      // prefill: SwiGLU in the GEMM epilogue (the gate | up product never reaches memory), then the row quantizer over h
      const tc::EpiArgs e{1.0f, 0.0f, nullptr, 3};
      st = tc::gemm_fp8_impl(h, xcc, w_gate_up, ct, 2 * F, hidden, B2Q_FP8_E4M3, xs + c * ct, B2Q_SCALE_PER_ROW, s_gate_up, B2Q_SCALE_PER_ROW,
                             gu, B2Q_OUT_BF16, &e);
      if (st != B2Q_OK) return st;
      st = b2q_fp8_quantize_rows_bf16(h, gu, ct, F, B2Q_FP8_E4M3, rounding, hs, hc);
      if (st != B2Q_OK) return st;
    } else if (inter) {
      // few tokens: the f32 product of the interleaved rows, then h = bf16(silu(gate) * up) and its codes in one kernel
      // (the arithmetic of the epilogue above, so a layer gives the same numbers whatever the token count)
      st = b2q_gemm_fp8(h, xcc, w_gate_up, ct, 2 * F, hidden, B2Q_FP8_E4M3, xs + c * ct, B2Q_SCALE_PER_ROW, s_gate_up, B2Q_SCALE_PER_ROW, gu,
                        B2Q_OUT_F32);
      if (st != B2Q_OK) return st;
      st = b2q_swiglu_quantize_rows_interleaved(h, (const float*)gu, ct, F, B2Q_FP8_E4M3, rounding, hs, hc);
      if (st != B2Q_OK) return st;
    } else {
      st = b2q_gemm_fp8(h, xcc, w_gate_up, ct, 2 * F, hidden, B2Q_FP8_E4M3, xs + c * ct, B2Q_SCALE_PER_ROW, s_gate_up, B2Q_SCALE_PER_ROW, gu,
                        B2Q_OUT_BF16);
      if (st != B2Q_OK) return st;
      st = b2q_swiglu_quantize_rows_bf16(h, gu, gu + (size_t)F * 2, ct, F, 2 * F, B2Q_FP8_E4M3, rounding, hs, hc);
      if (st != B2Q_OK) return st;
    }
    if (mode == 4) {
      for (int j = 0; j < col_chunks; ++j)
        if ((st = tpx::scatter_reduce_cols(t, hc, hs, w_down, s_down, nullptr, ct, F, hidden, yc, j, col_chunks)) != B2Q_OK) return st;
      continue;
    }
    st = row_linear_range(t, hc, hs, w_down, s_down, nullptr, ct, F, hidden, yc, mode, pf);
    if (st != B2Q_OK) return st;
    if (mode == 3) {
      B2Q_CUDA(h, cudaEventRecord(t->ev_ready[c], h->stream));
      B2Q_CUDA(h, cudaStreamWaitEvent(t->comm_stream, t->ev_ready[c], 0));
      B2Q_NCCL(h, tpx::nccl()->AllReduce(yc, yc, (size_t)ct * hidden, tpx::kNcclBfloat16, tpx::kNcclSum, t->comm, t->comm_stream));
    }
  }
  if (mode == 3) {
    B2Q_CUDA(h, cudaEventRecord(t->ev_done, t->comm_stream));
    B2Q_CUDA(h, cudaStreamWaitEvent(h->stream, t->ev_done, 0));
  }
  return B2Q_OK;
}

// Expert-parallel mixture of SwiGLU experts: TopKRouter::route (crates/oxicuda-dist-infer/src/expert_parallel/router.rs:94-140),
// ExpertDispatcher::dispatch_and_gather (expert_parallel/dispatch.rs:99-219) and SwiGluExpert::forward
// (crates/oxicuda-moe/src/expert/ffn.rs:208-243) as one enqueue with no host synchronisation: route, count and slot the
// pairs of this rank's experts on the device, scatter the tokens, quantize per row, ONE grouped gate|up GEMM, SwiGLU +
// re-quantize, ONE grouped down GEMM, weighted gather; with several ranks the tokens are replicated and the ranks'
// contributions are added by one all-reduce.
int32_t b2q_moe_forward(b2q_tp t, const void* x_bf16, const float* logits, const uint8_t* w_gate_up, const float* s_gate_up,
                        const uint8_t* w_down, const float* s_down, int64_t tokens, int64_t hidden, int64_t ffn, int n_experts, int top_k,
                        int rounding, void* y_bf16, int32_t* counts_out) {
  return b2q_moe_forward_ex(t, x_bf16, logits, w_gate_up, s_gate_up, w_down, s_down, tokens, hidden, ffn, n_experts, top_k, rounding,
                            B2Q_GATE_UP_CONCATENATED, y_bf16, counts_out);
}

int32_t b2q_moe_forward_ex(b2q_tp t, const void* x_bf16, const float* logits, const uint8_t* w_gate_up, const float* s_gate_up,
                           const uint8_t* w_down, const float* s_down, int64_t tokens, int64_t hidden, int64_t ffn, int n_experts, int top_k,
                           int rounding, int gate_up_layout, void* y_bf16, int32_t* counts_out) {
  B2Q_REQUIRE_TP(t);
  b2q_handle h = t->h;
  if (gate_up_layout != B2Q_GATE_UP_CONCATENATED && gate_up_layout != B2Q_GATE_UP_INTERLEAVED128)
    B2Q_FAIL(h, B2Q_ERR_INVALID_ARGUMENT, "moe_forward: unknown gate | up layout %d", gate_up_layout);
  if (gate_up_layout == B2Q_GATE_UP_INTERLEAVED128 && ffn % 128 != 0)
    B2Q_FAIL(h, B2Q_ERR_INVALID_DIMENSION, "moe_forward: the interleaved layout needs ffn %% 128 == 0, got %lld", (long long)ffn);
  if (tokens <= 0 || hidden <= 0 || ffn <= 0)
    B2Q_FAIL(h, B2Q_ERR_INVALID_DIMENSION, "moe_forward: dimensions must be non-zero: tokens=%lld, hidden=%lld, ffn=%lld", (long long)tokens,
             (long long)hidden, (long long)ffn);
  if (!x_bf16 || !logits || !w_gate_up || !s_gate_up || !w_down || !s_down || !y_bf16) B2Q_FAIL(h, B2Q_ERR_INVALID_ARGUMENT, "moe_forward: null operand");
  if (n_experts < 1 || n_experts % t->tp != 0)
    B2Q_FAIL(h, B2Q_ERR_INVALID_DIMENSION, "n_experts %d not divisible by ep %d", n_experts, t->tp);
  const int n_local = n_experts / t->tp, first = t->rank * n_local;
  const int64_t pairs = tokens * top_k;
  const int64_t cap = (pairs + 255) / 256 * 256 + (int64_t)n_local * 256;      // upper bound of the padded row ranges
  const int64_t F = ffn;
  using tpx::align256;
  const size_t o_idx = 0, o_wgt = o_idx + align256((size_t)pairs * 4), o_cnt = o_wgt + align256((size_t)pairs * 4),
               o_off = o_cnt + 256, o_slot = o_off + 512, o_xb = o_slot + align256((size_t)pairs * 4),
               o_xc = o_xb + align256((size_t)cap * hidden * 2), o_xs = o_xc + align256((size_t)cap * hidden),
               o_gu = o_xs + align256((size_t)cap * 4), o_hc = o_gu + align256((size_t)cap * 2 * F * 2),
               o_hs = o_hc + align256((size_t)cap * F), o_yb = o_hs + align256((size_t)cap * 4),
               total = o_yb + align256((size_t)cap * hidden * 2);
  uint8_t* ws = nullptr;
  int32_t st = tpx::scratch(t, total, &ws);
  if (st != B2Q_OK) return st;
  int32_t* idx = (int32_t*)(ws + o_idx); float* wgt = (float*)(ws + o_wgt);
  int32_t* cnt = (int32_t*)(ws + o_cnt); int32_t* off = (int32_t*)(ws + o_off); int32_t* slot = (int32_t*)(ws + o_slot);
  uint8_t* xb = ws + o_xb; uint8_t* xc = ws + o_xc; float* xs = (float*)(ws + o_xs);
  uint8_t* gu = ws + o_gu; uint8_t* hc = ws + o_hc; float* hs = (float*)(ws + o_hs); uint8_t* yb = ws + o_yb;
  if ((st = b2q_moe_route_topk(h, logits, tokens, n_experts, top_k, idx, wgt)) != B2Q_OK) return st;
  if ((st = b2q_moe_assign_slots(h, idx, pairs, first, n_local, cnt, off, slot)) != B2Q_OK) return st;
  if (counts_out) B2Q_CUDA(h, cudaMemcpyAsync(counts_out, cnt, (size_t)n_local * 4, cudaMemcpyDeviceToDevice, h->stream));
  if ((st = b2q_moe_scatter(h, x_bf16, slot, pairs, top_k, hidden * 2, xb)) != B2Q_OK) return st;
  if ((st = b2q_fp8_quantize_rows_bf16_scratch(h, xb, cap, hidden, B2Q_FP8_E4M3, rounding, xs, xc)) != B2Q_OK) return st;
  if (gate_up_layout == B2Q_GATE_UP_INTERLEAVED128) {
    // silu(gate) * up in the epilogue of the grouped GEMM: gu receives h [cap x F] bf16
    if ((st = b2q_grouped_gemm_fp8_rows_act(h, xc, xs, w_gate_up, s_gate_up, off, cnt, n_local, cap, 2 * F, hidden, B2Q_FP8_E4M3, gu, B2Q_OUT_BF16,
                                            3)) != B2Q_OK)
      return st;
    if ((st = b2q_fp8_quantize_rows_bf16_scratch(h, gu, cap, F, B2Q_FP8_E4M3, rounding, hs, hc)) != B2Q_OK) return st;
  } else {
    if ((st = b2q_grouped_gemm_fp8_rows(h, xc, xs, w_gate_up, s_gate_up, off, cnt, n_local, cap, 2 * F, hidden, B2Q_FP8_E4M3, gu, B2Q_OUT_BF16)) != B2Q_OK)
      return st;
    if ((st = b2q_swiglu_quantize_rows_bf16(h, gu, gu + (size_t)F * 2, cap, F, 2 * F, B2Q_FP8_E4M3, rounding, hs, hc)) != B2Q_OK) return st;
  }
  if ((st = b2q_grouped_gemm_fp8_rows(h, hc, hs, w_down, s_down, off, cnt, n_local, cap, hidden, F, B2Q_FP8_E4M3, yb, B2Q_OUT_BF16)) != B2Q_OK) return st;
  if ((st = b2q_ep_token_gather_bf16(h, yb, slot, wgt, tokens, top_k, hidden, y_bf16)) != B2Q_OK) return st;
  if (t->tp > 1) B2Q_NCCL(h, tpx::nccl()->AllReduce(y_bf16, y_bf16, (size_t)tokens * hidden, tpx::kNcclBfloat16, tpx::kNcclSum, t->comm, h->stream));
  return B2Q_OK;
}

// The same layer over block-scaled FP4 experts (E2M1 codes, one E8M0 scale per 32 along K): the two grouped GEMMs run on
// tcgen05 kind::mxf8f6f4.block_scale with the scattered rows quantized per 32-block to E4M3 (act_mode, see
// b2q_gemm_fp4_blockscaled); gate | up is concatenated per expert, h = silu(gate) * up is formed in bf16 between them.
int32_t b2q_moe_forward_fp4(b2q_tp t, const void* x_bf16, const float* logits, const uint8_t* c_gate_up, const uint8_t* s_gate_up,
                            const uint8_t* c_down, const uint8_t* s_down, int64_t tokens, int64_t hidden, int64_t ffn, int n_experts, int top_k,
                            int act_mode, void* y_bf16, int32_t* counts_out) {
  B2Q_REQUIRE_TP(t);
  b2q_handle h = t->h;
  if (tokens <= 0 || hidden <= 0 || ffn <= 0)
    B2Q_FAIL(h, B2Q_ERR_INVALID_DIMENSION, "moe_forward_fp4: dimensions must be non-zero: tokens=%lld, hidden=%lld, ffn=%lld", (long long)tokens,
             (long long)hidden, (long long)ffn);
  if (!x_bf16 || !logits || !c_gate_up || !s_gate_up || !c_down || !s_down || !y_bf16) B2Q_FAIL(h, B2Q_ERR_INVALID_ARGUMENT, "moe_forward_fp4: null operand");
  if (n_experts < 1 || n_experts % t->tp != 0) B2Q_FAIL(h, B2Q_ERR_INVALID_DIMENSION, "n_experts %d not divisible by ep %d", n_experts, t->tp);
  if (hidden % 128 != 0 || ffn % 128 != 0)
    B2Q_FAIL(h, B2Q_ERR_UNSUPPORTED, "moe_forward_fp4: hidden and ffn must be multiples of 128, got %lld and %lld", (long long)hidden, (long long)ffn);
  const int n_local = n_experts / t->tp, first = t->rank * n_local;
  const int64_t pairs = tokens * top_k;
  const int64_t cap = (pairs + 255) / 256 * 256 + (int64_t)n_local * 256;
  const int64_t F = ffn;
  using tpx::align256;
  const size_t o_idx = 0, o_wgt = o_idx + align256((size_t)pairs * 4), o_cnt = o_wgt + align256((size_t)pairs * 4), o_off = o_cnt + 256,
               o_slot = o_off + 512, o_xb = o_slot + align256((size_t)pairs * 4), o_gu = o_xb + align256((size_t)cap * hidden * 2),
               o_hb = o_gu + align256((size_t)cap * 2 * F * 2), o_yb = o_hb + align256((size_t)cap * F * 2),
               total = o_yb + align256((size_t)cap * hidden * 2);
  uint8_t* ws = nullptr;
  int32_t st = tpx::scratch(t, total, &ws);
  if (st != B2Q_OK) return st;
  int32_t* idx = (int32_t*)(ws + o_idx); float* wgt = (float*)(ws + o_wgt);
  int32_t* cnt = (int32_t*)(ws + o_cnt); int32_t* off = (int32_t*)(ws + o_off); int32_t* slot = (int32_t*)(ws + o_slot);
  uint8_t* xb = ws + o_xb; uint8_t* gu = ws + o_gu; uint8_t* hb = ws + o_hb; uint8_t* yb = ws + o_yb;
  if ((st = b2q_moe_route_topk(h, logits, tokens, n_experts, top_k, idx, wgt)) != B2Q_OK) return st;
  if ((st = b2q_moe_assign_slots(h, idx, pairs, first, n_local, cnt, off, slot)) != B2Q_OK) return st;
  if (counts_out) B2Q_CUDA(h, cudaMemcpyAsync(counts_out, cnt, (size_t)n_local * 4, cudaMemcpyDeviceToDevice, h->stream));
  if ((st = b2q_moe_scatter(h, x_bf16, slot, pairs, top_k, hidden * 2, xb)) != B2Q_OK) return st;
  if ((st = b2q_grouped_gemm_fp4_rows(h, c_gate_up, s_gate_up, xb, off, n_local, cap, 2 * F, hidden, act_mode, gu, B2Q_OUT_BF16)) != B2Q_OK) return st;
  {
    const int64_t total8 = cap * (F / 8);
    int grid = (int)((total8 + 255) / 256);
    if (grid > h->sm_count * 16) grid = h->sm_count * 16;
    tpx::swiglu_bf16_kernel<<<grid, 256, 0, h->stream>>>((const uint4*)gu, (uint4*)hb, cap, F / 8);
    B2Q_LAUNCH_CHECK(h, "swiglu_bf16_kernel");
  }
  if ((st = b2q_grouped_gemm_fp4_rows(h, c_down, s_down, hb, off, n_local, cap, hidden, F, act_mode, yb, B2Q_OUT_BF16)) != B2Q_OK) return st;
  if ((st = b2q_ep_token_gather_bf16(h, yb, slot, wgt, tokens, top_k, hidden, y_bf16)) != B2Q_OK) return st;
  if (t->tp > 1) B2Q_NCCL(h, tpx::nccl()->AllReduce(y_bf16, y_bf16, (size_t)tokens * hidden, tpx::kNcclBfloat16, tpx::kNcclSum, t->comm, h->stream));
  return B2Q_OK;
}

}  // extern "C"
