// GPTQ / AWQ weight-only group quantization: low-bit codes packed 32 / bits to a u32 (element e of the flat row-major
// matrix in word e / epu, bits [(e % epu) * bits, +bits)), one f32 scale and optionally one f32 zero point per group of
// `group_size` columns of a row.  crates/oxicuda-dnn/src/quantize/gptq_awq.rs generates five kernels; each is restated
// here with its own arithmetic, operation for operation:
//   dnn_gptq_quantize_f32     (:329-499)  -> gptq_quantize_kernel + gptq_group_scales_kernel
//   dnn_gptq_dequantize_f32   (:509-616)  -> wq_dequantize_kernel
//   dnn_awq_scale_search_f32  (:626-713)  -> awq_scale_search_kernel
//   dnn_awq_quantize_f32      (:723-857)  -> awq_quantize_kernel
//   dnn_fused_dequant_gemv_f32 (:867-986) -> fused_dequant_gemv_kernel
// The reference packs with one atomic OR per element into a zeroed buffer; here one thread assembles a whole word, so the
// output needs no clearing and no atomics.  The reference GEMV runs one thread per row with a stride of cols / epu words
// between its loads (every load its own sector); here a CTA of 128 rows stages [128 rows x 32 words] tiles through shared
// memory with 16-byte asynchronous copies, two or four chunks deep, and every thread walks its own row in the reference's
// column order, so that the sum is the reference's bit for bit.  With split_k > 1 a cluster of CTAs cuts the columns into
// contiguous segments (each summed in order, the partial sums added in segment order through distributed shared memory):
// more threads per row for matrices with few rows, at the price of a different association of the sum.
#include "common.cuh"
#include <cooperative_groups.h>

namespace cg = cooperative_groups;

namespace wq {

constexpr int kThreads = 256;
constexpr float kMinDamp = 1e-6f;            // MIN_DAMP (:29)

__device__ __forceinline__ float rsqrt_approx(float a) {
  float r;
  asm("rsqrt.approx.f32 %0, %1;" : "=f"(r) : "f"(a));
  return r;
}

// The codes of one packed word as f32, without the conversion unit (a quarter-rate pipe that bounded the first version of
// the GEMV): a code q <= 255 placed in the low byte of 0x4B000000 is the float 8388608 + q, and subtracting 8388608 is
// exact.  2, 4 and 8 bits take the code bytes with one byte permutation each after 1, 2 or 4 masks of the word.
template <int BITS>
__device__ __forceinline__ void unpack_word_f32(uint32_t w, float (&qf)[32 / BITS]) {
  constexpr uint32_t kMagic = 0x4B000000u;
  constexpr int EPU = 32 / BITS;
  if constexpr (BITS == 8) {
#pragma unroll
    for (int i = 0; i < 4; ++i) qf[i] = __uint_as_float(__byte_perm(w, kMagic, 0x7540u + i)) - 8388608.0f;
  } else if constexpr (BITS == 4) {
    const uint32_t m[2] = {w & 0x0F0F0F0Fu, (w >> 4) & 0x0F0F0F0Fu};
#pragma unroll
    for (int i = 0; i < 8; ++i) qf[i] = __uint_as_float(__byte_perm(m[i & 1], kMagic, 0x7540u + (i >> 1))) - 8388608.0f;
  } else if constexpr (BITS == 2) {
    const uint32_t m[4] = {w & 0x03030303u, (w >> 2) & 0x03030303u, (w >> 4) & 0x03030303u, (w >> 6) & 0x03030303u};
#pragma unroll
    for (int i = 0; i < 16; ++i) qf[i] = __uint_as_float(__byte_perm(m[i & 3], kMagic, 0x7540u + (i >> 2))) - 8388608.0f;
  } else {
#pragma unroll
    for (int i = 0; i < EPU; ++i) qf[i] = __uint_as_float(((w >> (i * BITS)) & ((1u << BITS) - 1u)) | kMagic) - 8388608.0f;
  }
}

// dnn_gptq_quantize_f32: q = clamp(rni(w / max(h[col], 1e-6)) [+ 2^(bits-1), floored at 0, if symmetric], 0, 2^bits - 1)
__global__ void __launch_bounds__(kThreads) gptq_quantize_kernel(const float* __restrict__ w, const float* __restrict__ hdiag, int64_t total,
                                                                 int64_t cols, int bits, int symmetric, uint32_t* __restrict__ packed,
                                                                 int64_t words) {
  const int epu = 32 / bits;
  const float qmax = (float)((1u << bits) - 1u), half = (float)(1u << (bits - 1));
  for (int64_t wd = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; wd < words; wd += (int64_t)gridDim.x * blockDim.x) {
    const int64_t e0 = wd * epu;
    int64_t col = e0 % cols;
    uint32_t p = 0;
    for (int j = 0; j < epu; ++j) {
      const int64_t e = e0 + j;
      if (e >= total) break;
      const float safe_h = fmaxf(__ldg(hdiag + col), kMinDamp);
      float r = rintf(__fdiv_rn(__ldg(w + e), safe_h));
      if (symmetric) r = fmaxf(__fadd_rn(r, half), 0.0f);
      const float c = fmaxf(fminf(r, qmax), 0.0f);
      p |= __float2uint_rz(c) << (j * bits);
      if (++col == cols) col = 0;
    }
    packed[wd] = p;
  }
}
// The scale the reference leaves in scale[row, group]: every column of the group stores max(h[col], 1e-6) / qmax there,
// one thread per row walking the columns upwards, so the group's last column wins.
__global__ void __launch_bounds__(kThreads) gptq_group_scales_kernel(const float* __restrict__ hdiag, int64_t n, int64_t gpr, int64_t group, int bits,
                                                                     float* __restrict__ scales) {
  const float qmax = (float)((1u << bits) - 1u);
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t g = i % gpr;
    scales[i] = __fdiv_rn(fmaxf(__ldg(hdiag + g * group + group - 1), kMinDamp), qmax);
  }
}

// dnn_gptq_dequantize_f32: out = q * scale, or (q - zero) * scale with zero points.
template <typename TOut>
__global__ void __launch_bounds__(kThreads) wq_dequantize_kernel(const uint32_t* __restrict__ packed, const float* __restrict__ scales,
                                                                 const float* __restrict__ zeros, int64_t total, int64_t cols, int64_t group,
                                                                 int bits, TOut* __restrict__ out, int64_t words) {
  const int epu = 32 / bits;
  const uint32_t mask = (1u << bits) - 1u;
  const int64_t gpr = cols / group;
  for (int64_t wd = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; wd < words; wd += (int64_t)gridDim.x * blockDim.x) {
    const uint32_t p = __ldg(packed + wd);
    const int64_t e0 = wd * epu;
    int64_t row = e0 / cols, col = e0 - row * cols;
    int64_t g = col / group, cig = col - g * group;
    float s = __ldg(scales + row * gpr + g), z = zeros ? __ldg(zeros + row * gpr + g) : 0.0f;
    for (int j = 0; j < epu; ++j) {
      const int64_t e = e0 + j;
      if (e >= total) break;
      const float qf = __uint2float_rn((p >> (j * bits)) & mask);
      const float v = zeros ? __fmul_rn(__fsub_rn(qf, z), s) : __fmul_rn(qf, s);
      if constexpr (sizeof(TOut) == 2) out[e] = __float2bfloat16_rn(v); else out[e] = v;
      ++col; ++cig;
      bool reload = false;
      if (col == cols) { col = 0; cig = 0; g = 0; ++row; reload = true; }
      else if (cig == group) { cig = 0; ++g; reload = true; }
      if (reload && e + 1 < total) {
        s = __ldg(scales + row * gpr + g);
        if (zeros) z = __ldg(zeros + row * gpr + g);
      }
    }
  }
}

// The same for the common layout (a word never straddles a row or a group: cols % epu == 0, group % epu == 0, bits != 3):
// one thread per word, one scale / zero point load, the 4 / 8 / 16 results stored as 16-byte vectors.
template <int BITS, typename TOut>
__global__ void __launch_bounds__(kThreads) wq_dequantize_vec_kernel(const uint32_t* __restrict__ packed, const float* __restrict__ scales,
                                                                     const float* __restrict__ zeros, int64_t words, uint32_t words_per_row,
                                                                     uint32_t words_per_group, TOut* __restrict__ out) {
  constexpr int EPU = 32 / BITS;
  const uint32_t gpr = words_per_row / words_per_group;
  for (int64_t wd = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; wd < words; wd += (int64_t)gridDim.x * blockDim.x) {
    const uint32_t p = __ldg(packed + wd);
    int64_t row;
    uint32_t wj;
    if (words <= 0xFFFFFFFFll) { row = (uint32_t)wd / words_per_row; wj = (uint32_t)wd - (uint32_t)row * words_per_row; }
    else { row = wd / words_per_row; wj = (uint32_t)(wd - row * words_per_row); }
    const int64_t s_idx = row * gpr + wj / words_per_group;
    const float s = __ldg(scales + s_idx), z = zeros ? __ldg(zeros + s_idx) : 0.0f;
    float qf[EPU], v[EPU];
    unpack_word_f32<BITS>(p, qf);
#pragma unroll
    for (int i = 0; i < EPU; ++i) v[i] = zeros ? __fmul_rn(__fsub_rn(qf[i], z), s) : __fmul_rn(qf[i], s);
    TOut* o = out + wd * EPU;
    if constexpr (sizeof(TOut) == 4) {
#pragma unroll
      for (int i = 0; i < EPU / 4; ++i) reinterpret_cast<float4*>(o)[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
    } else {
      uint32_t h[EPU / 2];
#pragma unroll
      for (int i = 0; i < EPU / 2; ++i) {
        const __nv_bfloat162 b = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
        h[i] = *reinterpret_cast<const uint32_t*>(&b);
      }
      if constexpr (EPU == 4) *reinterpret_cast<uint2*>(o) = make_uint2(h[0], h[1]);
      else {
#pragma unroll
        for (int i = 0; i < EPU / 8; ++i) reinterpret_cast<uint4*>(o)[i] = make_uint4(h[4 * i], h[4 * i + 1], h[4 * i + 2], h[4 * i + 3]);
      }
    }
  }
}

// dnn_awq_scale_search_f32: a = max(|act|, 1e-7); scale = a * rsqrt.approx(a)  (the reference's stand-in for a^alpha)
__global__ void __launch_bounds__(kThreads) awq_scale_search_kernel(const float* __restrict__ act, int64_t n, float* __restrict__ out) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    const float a = fmaxf(fabsf(__ldg(act + i)), 1e-7f);
    out[i] = __fmul_rn(a, rsqrt_approx(a));
  }
}

// dnn_awq_quantize_f32: q = min(max(rni(w * channel_scale[col] / max(group_scale, 1e-12)), 0), 2^bits - 1)
__global__ void __launch_bounds__(kThreads) awq_quantize_kernel(const float* __restrict__ w, const float* __restrict__ ch_scales,
                                                                const float* __restrict__ g_scales, int64_t total, int64_t cols, int64_t group,
                                                                int bits, uint32_t* __restrict__ packed, int64_t words) {
  const int epu = 32 / bits;
  const float qmax = (float)((1u << bits) - 1u);
  const int64_t gpr = cols / group;
  for (int64_t wd = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; wd < words; wd += (int64_t)gridDim.x * blockDim.x) {
    const int64_t e0 = wd * epu;
    int64_t row = e0 / cols, col = e0 - row * cols;
    uint32_t p = 0;
    for (int j = 0; j < epu; ++j) {
      const int64_t e = e0 + j;
      if (e >= total) break;
      const float ws = __fmul_rn(__ldg(w + e), __ldg(ch_scales + col));
      const float safe = fmaxf(__ldg(g_scales + row * gpr + col / group), 1e-12f);
      const float r = rintf(__fdiv_rn(ws, safe));
      const float c = fminf(fmaxf(r, 0.0f), qmax);
      p |= __float2uint_rz(c) << (j * bits);
      if (++col == cols) { col = 0; ++row; }
    }
    packed[wd] = p;
  }
}

// ---------------------------------------------------------------------------
// dnn_fused_dequant_gemv_f32: y[row] = sum over the columns, upwards, of fma(float(q) * scale[row, col / group], x[col], acc)
// ---------------------------------------------------------------------------
constexpr int GV_ROWS = 128;      // rows per CTA, one thread each
constexpr int GV_WCH = 32;        // packed words of every row per staged chunk
constexpr int GV_STRIDE = 36;     // words between rows of the tile: 16-byte aligned, conflict-free for 16-byte reads
// STAGES chunks in shared memory, STAGES - 1 in flight while one is consumed.  One thread per row gives a matrix of 28672
// rows six warps per SM: four stages then keep enough bytes in flight (86 against 98 us); with the columns split there
// are CTAs to spare and two stages (five CTAs per SM instead of two) are faster (78 against 90 us).
constexpr size_t gv_smem_bytes(int stages, int epu) { return (size_t)stages * (GV_ROWS * GV_STRIDE * 4 + GV_WCH * epu * 4); }

__device__ __forceinline__ void cp_async4(void* smem, const void* g) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((uint32_t)__cvta_generic_to_shared(smem)), "l"(g) : "memory");
}
__device__ __forceinline__ void cp_async16(void* smem, const void* g) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(smem)), "l"(g) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// ALIGNED: group % epu == 0, so a word never straddles two groups and the group test runs once per word.
template <int BITS, bool HAS_ZERO, bool ALIGNED, int GV_STAGES>
__global__ void __launch_bounds__(GV_ROWS, 2) fused_dequant_gemv_kernel(const uint32_t* __restrict__ packed, const float* __restrict__ scales,
                                                                     const float* __restrict__ zeros, const float* __restrict__ x,
                                                                     float* __restrict__ y, int64_t rows, int64_t cols, int64_t group, int split,
                                                                     int chunks_per_split, int vec) {
  constexpr int EPU = 32 / BITS;
  // GV_STAGES buffers of [128 rows x 36 words] codes, then GV_STAGES buffers of the 32 * EPU activations of a chunk
  extern __shared__ __align__(16) uint8_t gv_smem[];
  uint32_t (*tile)[GV_ROWS * GV_STRIDE] = reinterpret_cast<uint32_t (*)[GV_ROWS * GV_STRIDE]>(gv_smem);
  float (*xs)[GV_WCH * EPU] = reinterpret_cast<float (*)[GV_WCH * EPU]>(gv_smem + (size_t)GV_STAGES * GV_ROWS * GV_STRIDE * 4);
  __shared__ float red[GV_ROWS];
  const int tid = threadIdx.x;
  const int ks = (int)(blockIdx.x % (unsigned)split);
  const int64_t row0 = (int64_t)(blockIdx.x / (unsigned)split) * GV_ROWS, row = row0 + tid;
  const int64_t P = cols / EPU, gpr = cols / group;
  const int chunks_total = (int)((P + GV_WCH - 1) / GV_WCH);
  const int c_begin = min(ks * chunks_per_split, chunks_total), c_end = min(c_begin + chunks_per_split, chunks_total);

  // 16-byte copies: thread tid moves words [sq, sq + 4) of rows sr, sr + 16, .. of every chunk
  const int sr = tid >> 3, sq = (tid & 7) * 4;
  const uint32_t* sbase = packed + (row0 + sr) * P + sq;
  auto stage = [&](int c, int buf) {
    const int64_t w0 = (int64_t)c * GV_WCH;
    if (vec) {
      if (w0 + sq < P) {
#pragma unroll
        for (int i = 0; i < GV_ROWS / 16; ++i)
          if (row0 + sr + 16 * i < rows) cp_async16(&tile[buf][(sr + 16 * i) * GV_STRIDE + sq], sbase + (int64_t)(16 * i) * P + w0);
      }
    } else {
      for (int u = tid; u < GV_ROWS * GV_WCH; u += GV_ROWS) {
        const int r = u >> 5, wj = u & 31;
        if (row0 + r < rows && w0 + wj < P) cp_async4(&tile[buf][r * GV_STRIDE + wj], packed + (row0 + r) * P + w0 + wj);
      }
    }
    const int64_t col0 = w0 * EPU;
    for (int i = tid; i < GV_WCH * EPU; i += GV_ROWS)
      if (col0 + i < cols) cp_async4(&xs[buf][i], x + col0 + i);
    cp_async_commit();
  };

  const bool live = row < rows && c_begin < c_end;
  // cursor over the groups of this row: g = current group, cig = columns of it already consumed; the scale (and zero
  // point) of the next group is fetched one group ahead, off the dependent chain of the sum
  const int64_t col_begin = (int64_t)c_begin * GV_WCH * EPU;
  int64_t g = live ? col_begin / group : 0, cig = live ? col_begin - g * group : 0;
  const float* srow = scales + (live ? row : 0) * gpr;
  const float* zrow = HAS_ZERO ? zeros + (live ? row : 0) * gpr : nullptr;
  float s = 0.0f, s_next = 0.0f, z = 0.0f, z_next = 0.0f;
  if (live) {
    s = __ldg(srow + g);
    if (g + 1 < gpr) s_next = __ldg(srow + g + 1);
    if (HAS_ZERO) {
      z = __ldg(zrow + g);
      if (g + 1 < gpr) z_next = __ldg(zrow + g + 1);
    }
  }
  auto next_group = [&]() {
    cig = 0;
    ++g;
    s = s_next;
    if (g + 1 < gpr) s_next = __ldg(srow + g + 1);
    if (HAS_ZERO) {
      z = z_next;
      if (g + 1 < gpr) z_next = __ldg(zrow + g + 1);
    }
  };

  float acc = 0.0f;
  // one commit group per chunk slot, empty past the last chunk, so that "all but the newest GV_STAGES - 2 groups are
  // complete" always means "this iteration's chunk has landed"
  for (int st = 0; st < GV_STAGES - 1; ++st) {
    if (c_begin + st < c_end) stage(c_begin + st, st); else cp_async_commit();
  }
  for (int c = c_begin; c < c_end; ++c) {
    const int buf = (c - c_begin) % GV_STAGES;
    cp_async_wait<GV_STAGES - 2>();
    __syncthreads();                                     // chunk c is visible; every row is done with the buffer of chunk c - 1
    if (c + GV_STAGES - 1 < c_end) stage(c + GV_STAGES - 1, (c - c_begin + GV_STAGES - 1) % GV_STAGES); else cp_async_commit();
    if (row < rows) {
      const int nw = (int)min((int64_t)GV_WCH, P - (int64_t)c * GV_WCH);
      const uint4* trow = reinterpret_cast<const uint4*>(&tile[buf][tid * GV_STRIDE]);
      bool done = false;
      if constexpr (ALIGNED && BITS != 3) {
        // Full chunk and groups that end on 16-byte reads of the tile: no test per word.  Up to 32 values at a time
        // are unpacked and scaled (independent work) before their fused multiply-adds join the sum one after another.
        if (nw == GV_WCH && group % (4 * EPU) == 0) {
          constexpr int STEP_WORDS = BITS == 2 ? 2 : 4;
          constexpr int NV = STEP_WORDS * EPU;
          // branch-free group step (selects and one clamped look-ahead load per 16-byte read), so that the whole chunk is
          // one basic block and the scheduler can overlap the unpacking of later values with the dependent sum
#pragma unroll
          for (int w4 = 0; w4 < GV_WCH / 4; ++w4) {
            {
              const bool adv = cig == group;
              const int64_t gn = min(g + 2, gpr - 1);
              const float s_ld = __ldg(srow + gn);
              s = adv ? s_next : s;
              s_next = adv ? s_ld : s_next;
              if (HAS_ZERO) {
                const float z_ld = __ldg(zrow + gn);
                z = adv ? z_next : z;
                z_next = adv ? z_ld : z_next;
              }
              g += adv ? 1 : 0;
              cig = adv ? 0 : cig;
            }
            const uint4 v = trow[w4];
            const uint32_t wv[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int st = 0; st < 4 / STEP_WORDS; ++st) {
              float xr[NV], dq[NV];
              const float4* xq = reinterpret_cast<const float4*>(&xs[buf][(w4 * 4 + st * STEP_WORDS) * EPU]);
#pragma unroll
              for (int i = 0; i < NV / 4; ++i) {
                const float4 f = xq[i];
                xr[4 * i] = f.x; xr[4 * i + 1] = f.y; xr[4 * i + 2] = f.z; xr[4 * i + 3] = f.w;
              }
#pragma unroll
              for (int k = 0; k < STEP_WORDS; ++k) {
                float qv[EPU];
                unpack_word_f32<BITS>(wv[st * STEP_WORDS + k], qv);
#pragma unroll
                for (int sub = 0; sub < EPU; ++sub)
                  dq[k * EPU + sub] = HAS_ZERO ? __fmul_rn(__fsub_rn(qv[sub], z), s) : __fmul_rn(qv[sub], s);
              }
#pragma unroll
              for (int j = 0; j < NV; ++j) acc = __fmaf_rn(dq[j], xr[j], acc);
            }
            cig += 4 * EPU;
          }
          done = true;
        }
      }
      for (int w4 = 0; !done && w4 * 4 < nw; ++w4) {
        const uint4 v = trow[w4];
        const uint32_t wv[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          if (w4 * 4 + k < nw) {
            float xr[EPU];
            const float* xp = &xs[buf][(w4 * 4 + k) * EPU];
            if constexpr (EPU % 4 == 0) {
#pragma unroll
              for (int i = 0; i < EPU / 4; ++i) {
                const float4 f = reinterpret_cast<const float4*>(xp)[i];
                xr[4 * i] = f.x; xr[4 * i + 1] = f.y; xr[4 * i + 2] = f.z; xr[4 * i + 3] = f.w;
              }
            } else {
#pragma unroll
              for (int i = 0; i < EPU; ++i) xr[i] = xp[i];
            }
            float qv[EPU];
            unpack_word_f32<BITS>(wv[k], qv);
            if (ALIGNED && cig == group) next_group();
#pragma unroll
            for (int sub = 0; sub < EPU; ++sub) {
              if (!ALIGNED && cig == group) next_group();
              const float qf = qv[sub];
              const float dq = HAS_ZERO ? __fmul_rn(__fsub_rn(qf, z), s) : __fmul_rn(qf, s);
              acc = __fmaf_rn(dq, xr[sub], acc);
              if (!ALIGNED) ++cig;
            }
            if (ALIGNED) cig += EPU;
          }
        }
      }
    }
  }

  if (split > 1) {
    cg::cluster_group cluster = cg::this_cluster();
    red[tid] = acc;
    cluster.sync();
    if (ks == 0 && row < rows) {
      float v = red[tid];
      for (int pr = 1; pr < split; ++pr) v = __fadd_rn(v, cluster.map_shared_rank(red, pr)[tid]);
      y[row] = v;
    }
    cluster.sync();                                      // the first CTA may still be reading this CTA's partial sums
  } else if (row < rows) {
    y[row] = acc;
  }
}

template <int BITS, bool HAS_ZERO, bool ALIGNED, int STAGES>
int32_t launch_gemv_s(b2q_handle h, const uint32_t* packed, const float* scales, const float* zeros, const float* x, float* y, int64_t rows,
                      int64_t cols, int64_t group, int split, int cps, int vec) {
  const int64_t row_tiles = ceil_div64(rows, GV_ROWS);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(row_tiles * split));
  cfg.blockDim = dim3(GV_ROWS);
  const size_t smem = gv_smem_bytes(STAGES, 32 / BITS);
  B2Q_SMEM_ATTR(h, (fused_dequant_gemv_kernel<BITS, HAS_ZERO, ALIGNED, STAGES>), smem);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = h->stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = (unsigned)split;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = split > 1 ? 1 : 0;
  B2Q_CUDA(h, cudaLaunchKernelEx(&cfg, fused_dequant_gemv_kernel<BITS, HAS_ZERO, ALIGNED, STAGES>, packed, scales, zeros, x, y, rows, cols, group, split, cps,
                                 vec));
  return B2Q_OK;
}
template <int BITS, bool HAS_ZERO, bool ALIGNED>
int32_t launch_gemv_t(b2q_handle h, const uint32_t* packed, const float* scales, const float* zeros, const float* x, float* y, int64_t rows,
                      int64_t cols, int64_t group, int split, int cps, int vec) {
  return split == 1 ? launch_gemv_s<BITS, HAS_ZERO, ALIGNED, 4>(h, packed, scales, zeros, x, y, rows, cols, group, split, cps, vec)
                    : launch_gemv_s<BITS, HAS_ZERO, ALIGNED, 2>(h, packed, scales, zeros, x, y, rows, cols, group, split, cps, vec);
}
template <int BITS>
int32_t launch_gemv(b2q_handle h, const uint32_t* packed, const float* scales, const float* zeros, const float* x, float* y, int64_t rows,
                    int64_t cols, int64_t group, int split, int cps, int vec) {
  const bool aligned = group % (32 / BITS) == 0;
  if (zeros) {
    return aligned ? launch_gemv_t<BITS, true, true>(h, packed, scales, zeros, x, y, rows, cols, group, split, cps, vec)
                   : launch_gemv_t<BITS, true, false>(h, packed, scales, zeros, x, y, rows, cols, group, split, cps, vec);
  }
  return aligned ? launch_gemv_t<BITS, false, true>(h, packed, scales, zeros, x, y, rows, cols, group, split, cps, vec)
                 : launch_gemv_t<BITS, false, false>(h, packed, scales, zeros, x, y, rows, cols, group, split, cps, vec);
}

// WeightQuantPlan::new (:254-283) plus the bit widths of GptqConfig::validate (:102-108)
int32_t validate(b2q_handle h, const char* what, int64_t rows, int64_t cols, int64_t group, int bits) {
  if (rows <= 0 || cols <= 0) B2Q_FAIL(h, B2Q_ERR_INVALID_DIMENSION, "%s: weight dimensions must be non-zero", what);
  if (bits != 2 && bits != 3 && bits != 4 && bits != 8) B2Q_FAIL(h, B2Q_ERR_INVALID_ARGUMENT, "%s: bits must be 2, 3, 4, or 8; got %d", what, bits);
  if (group <= 0) B2Q_FAIL(h, B2Q_ERR_INVALID_ARGUMENT, "%s: group_size must be non-zero", what);
  if (cols % group != 0)
    B2Q_FAIL(h, B2Q_ERR_INVALID_ARGUMENT, "%s: cols (%lld) must be divisible by group_size (%lld)", what, (long long)cols, (long long)group);
  return B2Q_OK;
}
inline int grid_words(b2q_handle h, int64_t n) {
  int64_t g = ceil_div64(n, kThreads);
  const int64_t cap = (int64_t)h->sm_count * 32;
  return (int)(g < 1 ? 1 : (g > cap ? cap : g));
}

}  // namespace wq

extern "C" {

int64_t b2q_wq_packed_words(int64_t rows, int64_t cols, int bits) {
  if (rows <= 0 || cols <= 0 || (bits != 2 && bits != 3 && bits != 4 && bits != 8)) return -1;
  const int64_t epu = 32 / bits;
  return (rows * cols + epu - 1) / epu;
}

int32_t b2q_gptq_quantize_f32(b2q_handle h, const float* weight, const float* hessian_diag, int64_t rows, int64_t cols, int64_t group_size, int bits,
                              int symmetric, uint32_t* packed, float* scales) {
  B2Q_REQUIRE_HANDLE(h);
  int32_t st = wq::validate(h, "gptq_quantize", rows, cols, group_size, bits);
  if (st != B2Q_OK) return st;
  if (!weight || !hessian_diag || !packed || !scales) B2Q_FAIL(h, B2Q_ERR_INVALID_ARGUMENT, "gptq_quantize: null pointer");
  const int64_t total = rows * cols, words = b2q_wq_packed_words(rows, cols, bits), gpr = cols / group_size;
  wq::gptq_quantize_kernel<<<wq::grid_words(h, words), wq::kThreads, 0, h->stream>>>(weight, hessian_diag, total, cols, bits, symmetric != 0, packed,
                                                                                    words);
  B2Q_LAUNCH_CHECK(h, "gptq_quantize_kernel");
  wq::gptq_group_scales_kernel<<<wq::grid_words(h, rows * gpr), wq::kThreads, 0, h->stream>>>(hessian_diag, rows * gpr, gpr, group_size, bits, scales);
  B2Q_LAUNCH_CHECK(h, "gptq_group_scales_kernel");
  return B2Q_OK;
}

int32_t b2q_wq_dequantize(b2q_handle h, const uint32_t* packed, const float* scales, const float* zeros, int64_t rows, int64_t cols,
                          int64_t group_size, int bits, void* out, int out_type) {
  B2Q_REQUIRE_HANDLE(h);
  int32_t st = wq::validate(h, "wq_dequantize", rows, cols, group_size, bits);
  if (st != B2Q_OK) return st;
  if (!packed || !scales || !out || out_type < 0 || out_type > 1) B2Q_FAIL(h, B2Q_ERR_INVALID_ARGUMENT, "wq_dequantize: bad argument");
  const int64_t total = rows * cols, words = b2q_wq_packed_words(rows, cols, bits);
  const int64_t epu = 32 / bits;
  if (bits != 3 && cols % epu == 0 && group_size % epu == 0 && cols / epu <= 0xFFFFFFFFll && (reinterpret_cast<uintptr_t>(out) & 15) == 0) {
    const uint32_t wpr = (uint32_t)(cols / epu), wpg = (uint32_t)(group_size / epu);
    const int grid = wq::grid_words(h, words);
#define WQ_DEQ(B)                                                                                                                          \
  do {                                                                                                                                     \
    if (out_type == B2Q_OUT_BF16)                                                                                                          \
      wq::wq_dequantize_vec_kernel<B, __nv_bfloat16><<<grid, wq::kThreads, 0, h->stream>>>(packed, scales, zeros, words, wpr, wpg, (__nv_bfloat16*)out); \
    else                                                                                                                                   \
      wq::wq_dequantize_vec_kernel<B, float><<<grid, wq::kThreads, 0, h->stream>>>(packed, scales, zeros, words, wpr, wpg, (float*)out);    \
  } while (0)
    if (bits == 2) WQ_DEQ(2);
    else if (bits == 4) WQ_DEQ(4);
    else WQ_DEQ(8);
#undef WQ_DEQ
    B2Q_LAUNCH_CHECK(h, "wq_dequantize_vec_kernel");
    return B2Q_OK;
  }
  if (out_type == B2Q_OUT_BF16)
    wq::wq_dequantize_kernel<__nv_bfloat16><<<wq::grid_words(h, words), wq::kThreads, 0, h->stream>>>(packed, scales, zeros, total, cols, group_size,
                                                                                                   bits, (__nv_bfloat16*)out, words);
  else
    wq::wq_dequantize_kernel<float><<<wq::grid_words(h, words), wq::kThreads, 0, h->stream>>>(packed, scales, zeros, total, cols, group_size, bits,
                                                                                           (float*)out, words);
  B2Q_LAUNCH_CHECK(h, "wq_dequantize_kernel");
  return B2Q_OK;
}

int32_t b2q_awq_scale_search_f32(b2q_handle h, const float* act_stats, int64_t num_channels, float* scale_out) {
  B2Q_REQUIRE_HANDLE(h);
  if (num_channels <= 0) return B2Q_OK;                      // the reference launches no thread
  if (!act_stats || !scale_out) B2Q_FAIL(h, B2Q_ERR_INVALID_ARGUMENT, "awq_scale_search: null pointer");
  wq::awq_scale_search_kernel<<<wq::grid_words(h, num_channels), wq::kThreads, 0, h->stream>>>(act_stats, num_channels, scale_out);
  B2Q_LAUNCH_CHECK(h, "awq_scale_search_kernel");
  return B2Q_OK;
}

int32_t b2q_awq_quantize_f32(b2q_handle h, const float* weight, const float* channel_scales, const float* group_scales, int64_t rows, int64_t cols,
                             int64_t group_size, int bits, uint32_t* packed, float* zeros) {
  B2Q_REQUIRE_HANDLE(h);
  int32_t st = wq::validate(h, "awq_quantize", rows, cols, group_size, bits);
  if (st != B2Q_OK) return st;
  if (bits != 4 && bits != 8) B2Q_FAIL(h, B2Q_ERR_INVALID_ARGUMENT, "awq_quantize: AWQ bits must be 4 or 8; got %d", bits);
  if (!weight || !channel_scales || !group_scales || !packed) B2Q_FAIL(h, B2Q_ERR_INVALID_ARGUMENT, "awq_quantize: null pointer");
  const int64_t total = rows * cols, words = b2q_wq_packed_words(rows, cols, bits);
  wq::awq_quantize_kernel<<<wq::grid_words(h, words), wq::kThreads, 0, h->stream>>>(weight, channel_scales, group_scales, total, cols, group_size, bits,
                                                                                   packed, words);
  B2Q_LAUNCH_CHECK(h, "awq_quantize_kernel");
  if (zeros) B2Q_CUDA(h, cudaMemsetAsync(zeros, 0, (size_t)(rows * (cols / group_size)) * sizeof(float), h->stream));   // the reference stores 0.0
  return B2Q_OK;
}

int32_t b2q_fused_dequant_gemv_f32(b2q_handle h, const uint32_t* packed, const float* scales, const float* zeros, const float* x, int64_t rows,
                                   int64_t cols, int64_t group_size, int bits, int split_k, float* y) {
  B2Q_REQUIRE_HANDLE(h);
  int32_t st = wq::validate(h, "fused_dequant_gemv", rows, cols, group_size, bits);
  if (st != B2Q_OK) return st;
  const int64_t epu = 32 / bits;
  if (cols % epu != 0)
    B2Q_FAIL(h, B2Q_ERR_INVALID_ARGUMENT, "fused_dequant_gemv: cols (%lld) must be a multiple of the %lld values of a packed word", (long long)cols,
             (long long)epu);
  if (!packed || !scales || !x || !y) B2Q_FAIL(h, B2Q_ERR_INVALID_ARGUMENT, "fused_dequant_gemv: null pointer");
  if (split_k < 0 || split_k > 8 || (split_k & (split_k - 1)) != 0)
    B2Q_FAIL(h, B2Q_ERR_INVALID_ARGUMENT, "fused_dequant_gemv: split_k must be 0 (library's choice), 1, 2, 4 or 8; got %d", split_k);
  const int64_t P = cols / epu, chunks = ceil_div64(P, wq::GV_WCH), row_tiles = ceil_div64(rows, wq::GV_ROWS);
  int split = split_k;
  if (split == 0) {                                          // about four warps per scheduler: 16 warps = 4 CTAs per SM
    split = 1;
    while (split < 8 && row_tiles * split < (int64_t)h->sm_count * 4 && split * 2 <= chunks) split *= 2;
  }
  while (split > 1 && split > chunks) split /= 2;
  const int cps = (int)ceil_div64(chunks, split);
  const int vec = P % 4 == 0 && (reinterpret_cast<uintptr_t>(packed) & 15) == 0;
  if (bits == 2) return wq::launch_gemv<2>(h, packed, scales, zeros, x, y, rows, cols, group_size, split, cps, vec);
  if (bits == 3) return wq::launch_gemv<3>(h, packed, scales, zeros, x, y, rows, cols, group_size, split, cps, vec);
  if (bits == 4) return wq::launch_gemv<4>(h, packed, scales, zeros, x, y, rows, cols, group_size, split, cps, vec);
  return wq::launch_gemv<8>(h, packed, scales, zeros, x, y, rows, cols, group_size, split, cps, vec);
}

}  // extern "C"
