// Handle lifetime, status word and the host-side tile heuristics of libb2q.
#include "tc_common.cuh"
#include <stdlib.h>

int32_t b2q_workspace(b2q_handle h, size_t bytes, void** out) {
  if (bytes > h->ws_bytes) {
    B2Q_CUDA(h, cudaStreamSynchronize(h->stream));       // earlier calls may still be using the old buffer
    if (h->ws) cudaFree(h->ws);
    h->ws = nullptr;
    h->ws_bytes = 0;
    size_t want = bytes + bytes / 4;
    B2Q_CUDA(h, cudaMalloc(&h->ws, want));
    h->ws_bytes = want;
  }
  *out = h->ws;
  return B2Q_OK;
}

int32_t b2q_workspace2(b2q_handle h, size_t bytes, void** out) {
  if (bytes > h->ws2_bytes) {
    B2Q_CUDA(h, cudaStreamSynchronize(h->stream));
    if (h->ws2) cudaFree(h->ws2);
    h->ws2 = nullptr;
    h->ws2_bytes = 0;
    B2Q_CUDA(h, cudaMalloc(&h->ws2, bytes));
    h->ws2_bytes = bytes;
  }
  *out = h->ws2;
  return B2Q_OK;
}

int32_t b2q_tensor_map_2d(b2q_handle h, CUtensorMap* map, const void* ptr, int elem_bytes, uint64_t d0, uint64_t d1, uint32_t box0,
                          uint32_t box1) {
  static_assert(sizeof(CUtensorMap) == 128, "CUtensorMap size");
  const uint64_t key[4] = {(uint64_t)reinterpret_cast<uintptr_t>(ptr), d0, d1, ((uint64_t)box0 << 40) | ((uint64_t)box1 << 8) | (uint64_t)elem_bytes};
  uint64_t hsh = key[0] * 0x9E3779B97F4A7C15ull ^ key[1] * 0xC2B2AE3D27D4EB4Full ^ key[2] * 0x165667B19E3779F9ull ^ key[3];
  hsh ^= hsh >> 29;
  b2q_handle_s::MapEntry* e = h->map_cache ? &h->map_cache[hsh % kMapCacheEntries] : nullptr;
  if (e && e->valid && e->key[0] == key[0] && e->key[1] == key[1] && e->key[2] == key[2] && e->key[3] == key[3]) {
    memcpy(map, e->map, 128);
    return B2Q_OK;
  }
  tcx::EncodeTiledFn enc = tcx::get_encode_fn();
  if (!enc) B2Q_FAIL(h, B2Q_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  cuuint64_t dims[2] = {(cuuint64_t)d0, (cuuint64_t)d1};
  cuuint64_t strides[1] = {(cuuint64_t)(d0 * (uint64_t)elem_bytes)};
  cuuint32_t box[2] = {box0, box1};
  cuuint32_t estr[2] = {1, 1};
  const CUtensorMapDataType dt = elem_bytes == 1 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                                                                                   : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
  CUresult r = enc(map, dt, 2, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) B2Q_FAIL(h, B2Q_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
  if (e) {
    memcpy(e->key, key, sizeof(key));
    memcpy(e->map, map, 128);
    e->valid = 1;
  }
  return B2Q_OK;
}

extern "C" {

int32_t b2q_create(b2q_handle* out, int device) {
  if (!out) return B2Q_ERR_INVALID_ARGUMENT;
  *out = nullptr;
  int count = 0;
  if (cudaGetDeviceCount(&count) != cudaSuccess || count <= 0) return B2Q_ERR_CUDA;  // no CPU fallback
  if (device < 0 || device >= count) return B2Q_ERR_INVALID_ARGUMENT;
  b2q_handle h = new b2q_handle_s();
  memset(h, 0, sizeof(*h));
  h->device = device;
  int prev_device = -1;
  cudaGetDevice(&prev_device);
  struct RestoreDevice {                                 // the caller's current device is left as it was found
    int prev;
    ~RestoreDevice() { if (prev >= 0) cudaSetDevice(prev); }
  } restore{prev_device};
  cudaDeviceProp prop;
  if (cudaSetDevice(device) != cudaSuccess || cudaGetDeviceProperties(&prop, device) != cudaSuccess) {
    delete h;
    return B2Q_ERR_CUDA;
  }
  h->sm = prop.major * 10 + prop.minor;
  h->sm_count = prop.multiProcessorCount;
  if (h->sm != 100) {  // the kernels are built for sm_100a only
    delete h;
    return B2Q_ERR_UNSUPPORTED;
  }
  if (cudaMalloc(&h->d_status, sizeof(int32_t)) != cudaSuccess ||
      cudaMalloc(&h->d_scratch, kScratchWords * sizeof(uint32_t)) != cudaSuccess ||
      cudaMalloc(&h->d_tile_counters, kTileCounters * sizeof(int32_t)) != cudaSuccess ||
      cudaMemset(h->d_tile_counters, 0, kTileCounters * sizeof(int32_t)) != cudaSuccess ||
      cudaMemset(h->d_status, 0, sizeof(int32_t)) != cudaSuccess ||
      cudaMemset(h->d_scratch, 0, kScratchWords * sizeof(uint32_t)) != cudaSuccess) {
    cudaFree(h->d_status);
    cudaFree(h->d_scratch);
    cudaFree(h->d_tile_counters);
    delete h;
    return B2Q_ERR_CUDA;
  }
  h->stream = nullptr;
  h->map_cache = new b2q_handle_s::MapEntry[kMapCacheEntries]();
  // experiment switches: read here once, never on the dispatch path
  auto sw = [](const char* name) { const char* e = getenv(name); return e && e[0] ? (e[0] == 'p' ? 9 : atoi(e)) : -1; };
  h->sw.no_tail_split = getenv("B2Q_NO_TAIL_SPLIT") ? 1 : -1;
  h->sw.force_tile = sw("B2Q_FORCE_TILE_N");       // 128 | 256 | p(air)
  h->sw.fp8_skinny = sw("B2Q_FP8_SKINNY");
  h->sw.skinny_pdl = sw("B2Q_SKINNY_PDL");
  h->sw.mx_streamk = sw("B2Q_MX_STREAMK");
  h->sw.mx_debug = sw("B2Q_MX_DEBUG");
  h->sw.mx_pdl = sw("B2Q_MX_PDL");
  h->sw.mx_inline = sw("B2Q_MX_INLINE");
  h->sw.e8c_db = sw("B2Q_GEMV_E8C_DB");
  h->sw.gemv_mx = sw("B2Q_GEMV_MX");
  h->sw.gemv_cluster = sw("B2Q_GEMV_CLUSTER");
  h->sw.gemv_exact = sw("B2Q_GEMV_EXACT");
  h->sw.int4_small = sw("B2Q_INT4_SMALL");
  h->sw.gemv_stream = sw("B2Q_GEMV_STREAM");
  h->sw.force_group_m = sw("B2Q_GEMM_GROUP_M");
  h->sw.chain_pdl = sw("B2Q_CHAIN_PDL");            // 0: the small kernels of a decode step launch without programmatic dependent launch     // row tiles per raster group of the pair kernel (experiments)
  *out = h;
  return B2Q_OK;
}

int32_t b2q_destroy(b2q_handle h) {
  if (!h) return B2Q_OK;
  int prev_device = -1;
  cudaGetDevice(&prev_device);
  cudaSetDevice(h->device);
  cudaFree(h->d_status);
  cudaFree(h->d_scratch);
  cudaFree(h->d_tile_counters);
  if (h->ws) cudaFree(h->ws);
  if (h->ws2) cudaFree(h->ws2);
  delete[] h->map_cache;
  delete h;
  if (prev_device >= 0) cudaSetDevice(prev_device);
  return B2Q_OK;
}

int32_t b2q_set_static_weights(b2q_handle h, int static_weights) {
  B2Q_REQUIRE_HANDLE(h);
  h->dynamic_weights = static_weights ? 0 : 1;
  return B2Q_OK;
}

int32_t b2q_set_stream(b2q_handle h, void* stream) {
  B2Q_REQUIRE_HANDLE(h);
  h->stream = (cudaStream_t)stream;
  return B2Q_OK;
}

int32_t b2q_get_sm(b2q_handle h, int* sm) {
  B2Q_REQUIRE_HANDLE(h);
  if (!sm) B2Q_FAIL(h, B2Q_ERR_INVALID_ARGUMENT, "b2q_get_sm: null output");
  *sm = h->sm;
  return B2Q_OK;
}

int32_t b2q_get_sm_count(b2q_handle h, int* count) {
  B2Q_REQUIRE_HANDLE(h);
  if (!count) B2Q_FAIL(h, B2Q_ERR_INVALID_ARGUMENT, "b2q_get_sm_count: null output");
  *count = h->sm_count;
  return B2Q_OK;
}

const char* b2q_last_error(b2q_handle h) { return h ? h->err : "null handle"; }

int32_t b2q_check(b2q_handle h) {
  B2Q_REQUIRE_HANDLE(h);
  int32_t st = 0;
  B2Q_CUDA(h, cudaMemcpyAsync(&st, h->d_status, sizeof(st), cudaMemcpyDeviceToHost, h->stream));
  B2Q_CUDA(h, cudaStreamSynchronize(h->stream));
  if (st != 0) {
    // A kernel that gave up on a bounded wait may have left split-K arrival counters non-zero (its CTAs skip the
    // arrival): clear them with the status so that the next stream-K launch starts from a clean table.
    B2Q_CUDA(h, cudaMemsetAsync(h->d_tile_counters, 0, kTileCounters * sizeof(int32_t), h->stream));
    B2Q_CUDA(h, cudaMemsetAsync(h->d_status, 0, sizeof(int32_t), h->stream));
    B2Q_CUDA(h, cudaStreamSynchronize(h->stream));
    B2Q_FAIL(h, st, "device-side validation recorded status %d", (int)st);
  }
  return B2Q_OK;
}

// ---------------------------------------------------------------------------
// Tile heuristics (pure host functions)
// ---------------------------------------------------------------------------
int32_t b2q_classify_workload(uint32_t m, uint32_t n, uint32_t k) {
  uint64_t mn = (uint64_t)m * (uint64_t)n;
  if (mn < 8192) return 0;               // SmallSquare
  if (m < 128 && n >= 128) return 2;     // SkinnyM
  if (n < 128 && m >= 128) return 3;     // SkinnyN
  if (k < 64) return 4;                  // SkinnyK
  if (m >= 1024 && n >= 1024) return 1;  // LargeSquare
  return 5;                              // General
}

int32_t b2q_ref_tile_config(int dtype, uint32_t m, uint32_t n, uint32_t k, b2q_tile_config* out) {
  if (!out || dtype < 0 || dtype > 2) return B2Q_ERR_INVALID_ARGUMENT;
  if (m == 0 || n == 0 || k == 0) return B2Q_ERR_INVALID_DIMENSION;
  if (dtype == 2) {  // Int8GemmConfig::tile_config, Sm100 arm
    *out = b2q_tile_config{128, 128, 64, 64, 64, 4, 1, 1};
    return B2Q_OK;
  }
  const uint32_t stages = k < 64 ? 2u : 4u;
  b2q_tile_config t{0, 0, 128, 0, 0, stages, 1, 1};
  switch (b2q_classify_workload(m, n, k)) {
    case 0: t.tile_m = 64; t.tile_n = 64; t.tile_k = 64; t.warp_m = 32; t.warp_n = 32; break;
    case 2: t.tile_m = 64; t.tile_n = 256; t.warp_m = 32; t.warp_n = 128; break;
    case 3: t.tile_m = 256; t.tile_n = 64; t.warp_m = 128; t.warp_n = 32; break;
    case 1: t.tile_m = 256; t.tile_n = 256; t.warp_m = 64; t.warp_n = 128; break;
    case 4:
      t.tile_m = 256; t.tile_n = 256; t.warp_m = 64; t.warp_n = 128; t.stages = 2;
      if (dtype == 1) t.tile_k = 64;
      break;
    default:
      t.tile_m = dtype == 1 ? 128u : 256u; t.tile_n = 256; t.warp_m = 64; t.warp_n = 128;
      break;
  }
  *out = t;
  return B2Q_OK;
}

uint32_t b2q_fp8_compute_split_k(uint32_t m, uint32_t n, uint32_t k) {
  if (m * n < 2048 && k > 32768) {
    uint32_t f = k / 8192;
    return f < 2 ? 2 : (f > 64 ? 64 : f);
  }
  return 1;
}

// The static per-shape table: which kernel family and CTA tile each (dtype, shape)
// dispatches to.  dtype 0 fp8, 1 fp4 (weight-only), 2 int8.
int32_t b2q_select_tile(int dtype, uint32_t m, uint32_t n, uint32_t k, b2q_tile_config* out, int* kernel_id) {
  return b2q_select_tile_ex(dtype, m, n, k, out, kernel_id, 1);
}

}  // extern "C"

// few_token_kernels = 0 leaves the weight-stationary tcgen05 kernels (ids 6 and 7) out: what a call falls back to when
// its operands do not meet their alignment rules.
int32_t b2q_select_tile_ex(int dtype, uint32_t m, uint32_t n, uint32_t k, b2q_tile_config* out, int* kernel_id, int few_token_kernels) {
  if (!out || !kernel_id || dtype < 0 || dtype > 2) return B2Q_ERR_INVALID_ARGUMENT;
  if (m == 0 || n == 0 || k == 0) return B2Q_ERR_INVALID_DIMENSION;
  if (dtype == 1) {
    const uint64_t code_bytes = (uint64_t)n * (k / 2);
    if (few_token_kernels && m <= 32 && k % 512 == 0 && (code_bytes >= (40ull << 20) || (code_bytes >= (16ull << 20) && (m >= 4 || n >= 13312)))) {
      // FP4 weight-only with E8M0 scales, large matrix: tcgen05 block-scaled MMA, 128 weight rows x 128 K per stage
      *out = b2q_tile_config{m <= 8 ? 16u : (m <= 16 ? 32u : 64u), 128, 128, 128, m <= 8 ? 16u : (m <= 16 ? 32u : 64u), 8, 1, 1};
      *kernel_id = 7;
      return B2Q_OK;
    }
    // FP4 weight-only: warp-level mma GEMV, 16 output rows per warp
    uint32_t rows = n <= 2048 ? 64u : 128u;
    *out = b2q_tile_config{m <= 8 ? 8u : (m <= 16 ? 16u : 32u), rows, 512, 8, 16, 1, 1, 1};
    *kernel_id = 3;
    return B2Q_OK;
  }
  if (few_token_kernels && dtype == 0 && k % 128 == 0 &&
      ((m <= 64 && (uint64_t)n * k >= (32ull << 20)) || (m > 8 && m <= 32 && (uint64_t)n * k >= (16ull << 20)) ||
       (m > 32 && m < 64))) {   // 33..63 tokens: too many for the mma.sync GEMV, too few for a 128-row tile
    // FP8, few tokens against a large weight matrix: weight-stationary tcgen05 kernel (weights are the M = 128 operand)
    const uint32_t nb = m <= 16 ? 16u : (m <= 32 ? 32u : 64u);
    *out = b2q_tile_config{nb, 128, 128, 128, nb, 8, 1, 1};
    *kernel_id = 6;
    return B2Q_OK;
  }
  if (dtype == 0 && m <= 32 && k % 64 == 0) {  // FP8 decode: 16 weight rows per CTA, mma.sync.m16n8k32 over the codes
    *out = b2q_tile_config{m <= 8 ? 8u : (m <= 16 ? 16u : 32u), 16, 256, 8, 16, 2, 1, 1};
    *kernel_id = 5;
    return B2Q_OK;
  }
  if (m < 64 || k % 16 != 0) {  // TMA-incompatible pitch or too few rows for a tensor-core tile: SIMT path
    *out = b2q_tile_config{16, 16, 16, 16, 16, 1, 0, 1};
    *kernel_id = 0;
    return B2Q_OK;
  }
  // tcgen05.  Two-CTA 256x256 pair tiles whenever the problem has more than one 128-row block and more
  // than one 128-column block (measured 2.31 vs 2.13 PFLOP/s at 4096^3: shared-memory traffic per SM drops
  // by a third); otherwise one 128-row accumulator per CTA, 256 columns wide unless that wastes a wave.
  if (m > 128 && n > 128) {
    *out = b2q_tile_config{256, 256, 128, 128, 256, 6, 1, 1};
    *kernel_id = 4;
    return B2Q_OK;
  }
  const uint32_t tm = (m + 127) / 128;
  const uint32_t t256 = tm * ((n + 255) / 256), t128 = tm * ((n + 127) / 128);
  const uint32_t sms = 148;
  const double eff256 = (double)t256 / (double)(((t256 + sms - 1) / sms) * sms);
  const double eff128 = (double)t128 / (double)(((t128 + sms - 1) / sms) * sms) * 0.78;  // measured: N=128 MMAs reach ~0.8 of the N=256 rate
  const bool wide = n >= 256 && eff256 >= eff128;
  *out = b2q_tile_config{128, wide ? 256u : 128u, 128, 128, wide ? 256u : 128u, wide ? 4u : 6u, 1, 1};
  *kernel_id = wide ? 1 : 2;
  return B2Q_OK;
}
