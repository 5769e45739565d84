// Shared host/device helpers for libb2q: the handle, status plumbing and the
// bit-exact device codecs (E4M3/E5M2, E2M1, E8M0, NF4).
#pragma once

#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>
#include <atomic>

#include "../../include/b2q.h"

// ---------------------------------------------------------------------------
// Handle
// ---------------------------------------------------------------------------
struct b2q_handle_s {
  int device;
  int sm;            // 100 for compute capability 10.0
  int sm_count;
  cudaStream_t stream;
  // Device scratch owned by the handle (kept for its lifetime so that no call
  // allocates): [0] status word, [1..] reduction keys.
  int32_t* d_status;         // 1 x i32
  uint32_t* d_scratch;       // kScratchWords x u32
  int32_t* d_tile_counters;  // kTileCounters x i32, all zero between launches (split-K arrival counts; the last arriver resets its entry)
  void* ws;                  // grow-only workspace for calls that need temporaries (kept so steady-state calls never allocate)
  size_t ws_bytes;
  void* ws2;                 // second grow-only buffer: operands re-laid-out for a call whose kernel uses `ws` itself
  size_t ws2_bytes;
  int dynamic_weights;       // 1: weight operands may be written by the previous kernel of the stream (no early weight fetch)
  // Experiment switches (environment variables B2Q_*), read once when the handle is created: -1 = not set.
  struct Switches {
    int no_tail_split, force_tile, fp8_skinny, skinny_pdl, mx_streamk, mx_debug, mx_pdl, mx_inline, e8c_db, gemv_mx, gemv_cluster,
        gemv_exact, int4_small, gemv_stream, force_group_m, chain_pdl;
  } sw;
  // encoded TMA descriptors, direct-mapped by a hash of their key (128 bytes each; see b2q_tensor_map_2d)
  struct MapEntry { uint64_t key[4]; unsigned char map[128]; int valid; };
  MapEntry* map_cache;
  char err[512];
};
static const int kMapCacheEntries = 256;
// Returns a workspace of at least `bytes` (256-byte aligned); grows it when needed (synchronises the stream first).
int32_t b2q_workspace(b2q_handle h, size_t bytes, void** out);
int32_t b2q_workspace2(b2q_handle h, size_t bytes, void** out);
// b2q_select_tile with a switch that leaves the few-token tcgen05 kernels out of the table
int32_t b2q_select_tile_ex(int dtype, uint32_t m, uint32_t n, uint32_t k, b2q_tile_config* out, int* kernel_id, int few_token_kernels);
static const size_t kScratchWords = 1 << 16;   // 256 KiB of reduction keys / counters
static const size_t kTileCounters = 1 << 14;

#define B2Q_FAIL(h, code, ...)                                   \
  do {                                                           \
    if (h) snprintf((h)->err, sizeof((h)->err), __VA_ARGS__);    \
    return (int32_t)(code);                                      \
  } while (0)

#define B2Q_CUDA(h, expr)                                                              \
  do {                                                                                 \
    cudaError_t _e = (expr);                                                           \
    if (_e != cudaSuccess) B2Q_FAIL(h, B2Q_ERR_CUDA, "%s: %s", #expr, cudaGetErrorString(_e)); \
  } while (0)

#define B2Q_LAUNCH_CHECK(h, what)                                                      \
  do {                                                                                 \
    cudaError_t _e = cudaGetLastError();                                               \
    if (_e != cudaSuccess) B2Q_FAIL(h, B2Q_ERR_LAUNCH_FAILED, "%s: %s", what, cudaGetErrorString(_e)); \
  } while (0)

// cudaFuncSetAttribute(MaxDynamicSharedMemorySize) applies to the current device only: remember per kernel (one
// static mask per expansion site) which devices have been configured.  The handle's device must be current.
#define B2Q_SMEM_ATTR(h, kernel, bytes)                                                               \
  do {                                                                                                \
    static std::atomic<unsigned long long> _done{0};                                                  \
    const unsigned long long _bit = 1ull << ((h)->device & 63);                                       \
    if (!(_done.load(std::memory_order_acquire) & _bit)) {                                            \
      B2Q_CUDA(h, cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(bytes))); \
      _done.fetch_or(_bit, std::memory_order_release);                                                \
    }                                                                                                 \
  } while (0)

// Every entry point launches on the CURRENT device: a handle used while another device is current is refused.
#define B2Q_REQUIRE_HANDLE(h)                                                                          \
  do {                                                                                                 \
    if (!(h)) return (int32_t)B2Q_ERR_INVALID_ARGUMENT;                                                \
    (h)->err[0] = 0;                                                                                   \
    int _dev = -1;                                                                                     \
    if (cudaGetDevice(&_dev) != cudaSuccess || _dev != (h)->device)                                    \
      B2Q_FAIL(h, B2Q_ERR_INVALID_ARGUMENT, "the handle belongs to device %d but device %d is current", (h)->device, _dev); \
  } while (0)

static inline int64_t ceil_div64(int64_t a, int64_t b) { return (a + b - 1) / b; }

// ---------------------------------------------------------------------------
// Device codecs.  Integer-only where the reference is integer-only, explicit
// IEEE intrinsics (__fdiv_rn, __fmul_rn, __fadd_rn) where rounding order matters,
// so the results do not depend on -fmad or fast-math settings.
// ---------------------------------------------------------------------------
struct Fp8Fmt { int exp_bits, man_bits, bias; float max_val; uint32_t sat; };
__host__ __device__ inline Fp8Fmt fp8_fmt(int f) {
  return f == 0 ? Fp8Fmt{4, 3, 7, 448.0f, 0x7Eu} : Fp8Fmt{5, 2, 15, 57344.0f, 0x7Bu};
}

// Reference codec encode (truncating; saturates every biased exponent >= 2^eb-1;
// halves the subnormal mantissa): Fp8Codec::fp32_to_fp8.
__device__ __forceinline__ uint32_t fp8_encode_ref_dev(float v, const Fp8Fmt F) {
  uint32_t bits = __float_as_uint(v);
  uint32_t sign = bits >> 31;
  int exp32 = (int)((bits >> 23) & 0xFF);
  uint32_t man32 = bits & 0x007FFFFFu;
  if (v == 0.0f) return sign << 7;
  int exp8_raw = exp32 - 127 + F.bias;
  uint32_t man_shift = 23 - F.man_bits;
  uint32_t mmask = (1u << F.man_bits) - 1;
  if (exp8_raw <= 0) {
    uint32_t full_man = (man32 | 0x00800000u) >> 1;
    uint32_t shift = (uint32_t)(1 - exp8_raw) + man_shift;
    if (shift >= 24) return sign << 7;
    return (sign << 7) | ((full_man >> shift) & mmask);
  }
  if (exp8_raw >= (1 << F.exp_bits) - 1) return (sign << 7) | F.sat;
  return (sign << 7) | ((uint32_t)exp8_raw << F.man_bits) | ((man32 >> man_shift) & mmask);
}

// Round-to-nearest-even saturating encode == hardware conversion.
__device__ __forceinline__ uint32_t fp8_encode_rne_dev(float v, int fmt) {
  return (uint32_t)__nv_cvt_float_to_fp8(v, __NV_SATFINITE, fmt == 0 ? __NV_E4M3 : __NV_E5M2);
}

// Reference codec decode (subnormals decode as 2^(1-bias)*(1+m/2^mb)): Fp8Codec::fp8_to_fp32.
__device__ __forceinline__ float fp8_decode_ref_dev(uint32_t b, const Fp8Fmt F) {
  uint32_t sign = (b >> 7) & 1;
  uint32_t exp8 = (b >> F.man_bits) & ((1u << F.exp_bits) - 1);
  uint32_t man8 = b & ((1u << F.man_bits) - 1);
  uint32_t all_exp = (1u << F.exp_bits) - 1;
  if (F.exp_bits == 4) {
    if (exp8 == all_exp && man8 == 7) return __uint_as_float(0x7FC00000u);
  } else if (exp8 == all_exp) {
    return man8 == 0 ? __uint_as_float((sign << 31) | 0x7F800000u) : __uint_as_float(0x7FC00000u);
  }
  uint32_t man_shift = 23 - F.man_bits;
  if (exp8 == 0) {
    if (man8 == 0) return __uint_as_float(sign << 31);
    uint32_t exp32 = (uint32_t)(127 + 1 - F.bias);
    return __uint_as_float((sign << 31) | (exp32 << 23) | (man8 << man_shift));
  }
  uint32_t exp32 = (uint32_t)((int)exp8 - F.bias + 127);
  return __uint_as_float((sign << 31) | (exp32 << 23) | (man8 << man_shift));
}

// IEEE-style decode (true subnormals), what the tensor core multiplies with.
__device__ __forceinline__ float fp8_decode_ieee_dev(uint32_t b, const Fp8Fmt F) {
  uint32_t sign = (b >> 7) & 1;
  uint32_t exp8 = (b >> F.man_bits) & ((1u << F.exp_bits) - 1);
  uint32_t man8 = b & ((1u << F.man_bits) - 1);
  uint32_t all_exp = (1u << F.exp_bits) - 1;
  if (F.exp_bits == 4) {
    if (exp8 == all_exp && man8 == 7) return __uint_as_float(0x7FC00000u);
  } else if (exp8 == all_exp) {
    return man8 == 0 ? __uint_as_float((sign << 31) | 0x7F800000u) : __uint_as_float(0x7FC00000u);
  }
  float mag;
  if (exp8 == 0) mag = (float)man8 * __uint_as_float((uint32_t)(127 + 1 - F.bias - F.man_bits) << 23);
  else mag = __uint_as_float(((uint32_t)((int)exp8 - F.bias + 127) << 23) | (man8 << (23 - F.man_bits)));
  return sign ? -mag : mag;
}

// Fp4Quantizer::quantize_one (E2M1): round toward zero onto {0,.5,1,1.5,2,3,4,6},
// with |v| < 0.75 -> 0 and the sign bit kept for every non-zero input; -0.0 -> 0.
__device__ __forceinline__ uint32_t e2m1_encode_ref_dev(float value) {
  if (value == 0.0f) return 0;
  uint32_t sign = value < 0.0f ? 8u : 0u;
  float a = fminf(fabsf(value), 6.0f);          // NaN.min(6) == 6, as in the reference
  // thresholds 0.75, 1, 1.5, 2, 3, 4, 6: from 1 up they are the floats with one mantissa bit, so truncating the
  // float to that bit (bits >> 22) counts them: 1.0 -> 254 -> code 2, ..., 6.0 -> 259 -> code 7 (same codes as the
  // comparison chain for every float; NaN, which fminf turned into 6, ends at 7 either way)
  const uint32_t top = (__float_as_uint(a) >> 22) - 252u;
  uint32_t mag = a < 0.75f ? 0u : a < 1.0f ? 1u : (top < 7u ? top : 7u);
  return sign | mag;
}
__device__ __forceinline__ uint32_t int4_encode_ref_dev(float value) {
  float c = fminf(fmaxf(roundf(value), -8.0f), 7.0f);
  int q = isnan(value) ? 0 : (int)c;
  return (uint32_t)q & 0xFu;
}
__device__ __forceinline__ float e2m1_decode_dev(uint32_t raw) {
  uint32_t e = (raw >> 1) & 3, m = raw & 1;
  float v = e == 0 ? (float)m * 0.5f : __uint_as_float(((e + 126u) << 23) | (m << 22));
  return (raw & 8) ? -v : v;
}
__device__ __forceinline__ float int4_decode_dev(uint32_t raw) {
  return (float)((int)(raw << 28) >> 28);
}

// E8M0 block scale (no counterpart in the reference): smallest power of two >= absmax/6.
__device__ __forceinline__ uint32_t e8m0_from_absmax_dev(float absmax) {
  if (!(absmax > 0.0f)) return 127u;
  float s = __fdiv_rn(absmax, 6.0f);
  uint32_t u = __float_as_uint(s);
  int e = (int)((u >> 23) & 0xFF);
  uint32_t man = u & 0x007FFFFFu;
  int p;
  if (e == 0) {                                  // f32 subnormal: below 2^-126
    p = -127;                                    // clamped anyway
    if (man == 0) return 127u;
  } else {
    p = e - 127 + (man != 0 ? 1 : 0);            // ceil(log2 s)
  }
  p = min(127, max(-127, p));
  return (uint32_t)(p + 127);
}
__device__ __forceinline__ float e8m0_to_f32_dev(uint32_t b) {
  // 2^(b-127); b == 0 is 2^-127, an f32 subnormal
  return b == 0 ? __uint_as_float(0x00400000u) : __uint_as_float(b << 23);
}

// Orderable key for float atomics: non-negative floats compare as unsigned ints.
__device__ __forceinline__ uint32_t float_order_key(float f) {
  uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float float_from_order_key(uint32_t k) {
  return __uint_as_float((k & 0x80000000u) ? (k & 0x7FFFFFFFu) : ~k);
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_min(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fminf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Programmatic dependent launch for the small kernels of a decode step (row quantizer, SwiGLU quantizer, peer all-reduce):
// b2q_pdl_entry() is the first statement of such a kernel.  It waits for the previous kernel of the stream to complete
// (a no-op for a normal launch) and then lets the NEXT kernel start launching while this one runs; that kernel waits
// the same way before it touches memory, so the only thing that overlaps is launch latency.  B2Q_PDL_LAUNCH enqueues a
// kernel so (h->sw.chain_pdl = 0, B2Q_CHAIN_PDL=0, launches normally).
#ifdef __CUDACC__
__device__ __forceinline__ void b2q_pdl_entry() {
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
template <typename... KArgs, typename... Args>
static inline cudaError_t b2q_pdl_launch(bool pdl, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
#endif
