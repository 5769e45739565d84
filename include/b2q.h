/*
 * b2q — B200-native (sm_100a) quantized linear-layer kernels behind a C ABI.
 *
 * Every entry point is the drop-in replacement for one item of the reference
 * (OxiCUDA, paths relative to its repository root) and cites it.  Conventions,
 * all taken from the reference's BLAS layer:
 *   - the caller owns every buffer; pointers are raw DEVICE pointers (the
 *     reference passes CUdeviceptr as u64, crates/oxicuda-blas/src/types.rs:540-552);
 *   - every call enqueues on the handle's stream and returns at once; the caller
 *     synchronises before reading (crates/oxicuda-blas/src/level3/gemm/dispatch.rs:1115-1117);
 *   - errors are int32 status codes, one per variant of BlasError
 *     (crates/oxicuda-blas/src/error.rs:17-60) / QuantError
 *     (crates/oxicuda-quant/src/error.rs:10-58); b2q_last_error() gives the text;
 *   - a handle is owned by one host thread (BlasHandle is Send, not Sync:
 *     crates/oxicuda-blas/src/handle.rs:39-42).
 * There is no CPU fallback: without a CUDA device b2q_create fails.
 */
#ifndef B2Q_H
#define B2Q_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct b2q_handle_s* b2q_handle;

typedef enum {
  B2Q_OK = 0,
  B2Q_ERR_CUDA = 1,                  /* BlasError::Cuda */
  B2Q_ERR_INVALID_DIMENSION = 2,     /* BlasError::InvalidDimension */
  B2Q_ERR_BUFFER_TOO_SMALL = 3,      /* BlasError::BufferTooSmall */
  B2Q_ERR_DIMENSION_MISMATCH = 4,    /* BlasError::DimensionMismatch / QuantError::DimensionMismatch */
  B2Q_ERR_UNSUPPORTED = 5,           /* BlasError::UnsupportedOperation */
  B2Q_ERR_LAUNCH_FAILED = 7,         /* BlasError::LaunchFailed */
  B2Q_ERR_INVALID_ARGUMENT = 8,      /* BlasError::InvalidArgument */
  B2Q_ERR_EMPTY_INPUT = 20,          /* QuantError::EmptyInput */
  B2Q_ERR_GROUP_SIZE_MISMATCH = 21,  /* QuantError::GroupSizeMismatch */
  B2Q_ERR_INVALID_SCALE = 22,        /* QuantError::InvalidScale */
  B2Q_ERR_NON_FINITE_FP8 = 23,       /* QuantError::NonFiniteFp8 */
  B2Q_ERR_INVALID_CONFIG = 24,       /* QuantError::InvalidConfig / InferError::InvalidConfig */
  B2Q_ERR_INVALID_BIT_WIDTH = 25,    /* QuantError::InvalidBitWidth */
  B2Q_ERR_TIMEOUT = 40,              /* a bounded device-side wait gave up */
  B2Q_ERR_NCCL = 41                  /* an NCCL call failed, or libnccl could not be resolved (DistInferError::Collective) */
} b2q_status;

typedef enum { B2Q_FP8_E4M3 = 0, B2Q_FP8_E5M2 = 1 } b2q_fp8_format;  /* Fp8Format, crates/oxicuda-quant/src/scheme/fp8.rs:32-37 */
/* B2Q_ROUND_REF reproduces Fp8Codec bit for bit (truncating mantissa, fp8.rs:163-208);
 * B2Q_ROUND_RNE is round-to-nearest-even saturating (== cvt.rn.satfinite.e4m3x2.f32 and the
 * encoder of crates/oxicuda-dnn/src/quantize/fp8_quantize.rs:325). */
typedef enum { B2Q_ROUND_REF = 0, B2Q_ROUND_RNE = 1 } b2q_rounding;
typedef enum { B2Q_FP4_E2M1 = 0, B2Q_FP4_INT4 = 1 } b2q_fp4_format;  /* Fp4Format, crates/oxicuda-blas/src/precision/fp4_fp6_ops.rs:107-114 */
/* Block-scale storage.  F32 is what every reference code path stores
 * (MicroScalingQuantizer::compute_scales, fp4_fp6_ops.rs:763-782); E8M0 has no
 * counterpart in the reference: scale = 2^ceil(log2(absmax/6)), byte = exponent+127. */
typedef enum { B2Q_SCALE_F32 = 0, B2Q_SCALE_E8M0 = 1 } b2q_scale_format;
typedef enum { B2Q_SYMMETRIC = 0, B2Q_ASYMMETRIC = 1 } b2q_quant_scheme; /* QuantScheme, crates/oxicuda-quant/src/scheme/minmax.rs:26-32 */
typedef enum { B2Q_OUT_BF16 = 0, B2Q_OUT_F32 = 1 } b2q_out_type;
typedef enum { B2Q_SCALE_SCALAR = 0, B2Q_SCALE_PER_ROW = 1 } b2q_scale_kind;

/* ---- handle: BlasHandle::{new,set_stream,sm_version} crates/oxicuda-blas/src/handle.rs:80-95, :243-255 ---- */
/* b2q_create / b2q_destroy leave the caller's current device as they found it.  Every other call launches on the
 * CURRENT device and returns B2Q_ERR_INVALID_ARGUMENT when that is not the handle's device. */
int32_t b2q_create(b2q_handle* out, int device);
int32_t b2q_destroy(b2q_handle h);
/* stream is a cudaStream_t passed as void*; NULL = the legacy default stream */
int32_t b2q_set_stream(b2q_handle h, void* stream);
/* The few-token tensor-core kernels (FP4 decode GEMV, FP8 GEMM with up to 64 tokens) are launched as programmatic
 * dependents of the previous kernel of the stream: they start while it drains and read everything it may have produced
 * only after it has completed.  With static_weights = 1 (the default: inference weights are written once) the weight
 * codes and weight scales are excepted: they are fetched before that point, which hides the first memory round trip.
 * Pass 0 when a call's weight operand may be written by the kernel that precedes it on the stream; the kernels then
 * read nothing before the previous kernel has completed.  No counterpart in the reference (it has no stream overlap). */
int32_t b2q_set_static_weights(b2q_handle h, int static_weights);
int32_t b2q_get_sm(b2q_handle h, int* sm);              /* 100 on a B200 */
int32_t b2q_get_sm_count(b2q_handle h, int* count);
const char* b2q_last_error(b2q_handle h);
/* Reads (and clears) the device-side status word written by kernels that validate
 * their input on the device (non-finite FP8 input, invalid scale, bounded waits).
 * Synchronises the handle stream.  Returns B2Q_OK or the recorded status. */
int32_t b2q_check(b2q_handle h);

/* ---- MinMaxQuantizer: crates/oxicuda-quant/src/scheme/minmax.rs ---- */
/* calibrate (:134-171), calibrate_2d (:179-207), calibrate_slice (:209-243): one (scale, zero point)
 * per slice of `cols` contiguous elements; rows=1 is PerTensor, rows=len/group is PerGroup. */
int32_t b2q_minmax_calibrate_f32(b2q_handle h, const float* x, int64_t rows, int64_t cols, int bits,
                                 int scheme, float* scales, int32_t* zero_points);
/* quantize (:252-268) / quantize_grouped (:275-299): codes are i32 as in the reference (Vec<i32>). */
int32_t b2q_minmax_quantize_f32(b2q_handle h, const float* x, int64_t rows, int64_t cols, const float* scales,
                                const int32_t* zero_points, int bits, int scheme, int32_t* codes);
/* dequantize (:302-306) / dequantize_grouped (:309-324) */
int32_t b2q_minmax_dequantize_f32(b2q_handle h, const int32_t* codes, int64_t rows, int64_t cols,
                                  const float* scales, const int32_t* zero_points, float* out);
/* fake_quant_inplace kernel (crates/oxicuda-quant/src/ptx_kernels.rs:55-121) with the rounding of its
 * CPU definition FakeQuantize::forward (crates/oxicuda-quant/src/qat/fake_quant.rs:118-133). */
int32_t b2q_fake_quant_inplace_f32(b2q_handle h, float* x, int64_t n, float scale, float zero_point,
                                   float qmin, float qmax);

/* ---- Fp8Codec: crates/oxicuda-quant/src/scheme/fp8.rs ---- */
/* encode (:135-137): clamp to +-max then encode.  A NaN/Inf input records B2Q_ERR_NON_FINITE_FP8 in the
 * device status word (encode_f32 :115-118); read it with b2q_check. */
int32_t b2q_fp8_encode_f32(b2q_handle h, const float* x, int64_t n, int fmt, int rounding, uint8_t* codes);
/* decode (:140-142).  rounding=B2Q_ROUND_REF decodes as the reference codec does (:210-261);
 * B2Q_ROUND_RNE decodes IEEE-style (true subnormals), which is what the tensor core computes with. */
int32_t b2q_fp8_decode_f32(b2q_handle h, const uint8_t* codes, int64_t n, int fmt, int rounding, float* out);
/* In place: rewrites each subnormal code (exponent field 0, mantissa m != 0) as exponent field 1 with the same
 * mantissa.  Fp8Codec::fp8_to_fp32 (fp8.rs:242-254) decodes a subnormal code as 2^(1-bias)*(1+m/2^mb), which is the
 * IEEE value of the rewritten code; b2q_gemm_fp8 over rewritten codes therefore multiplies exactly the values the
 * reference's decode -> f32 matmul composition multiplies. */
int32_t b2q_fp8_remap_ref_subnormals(b2q_handle h, uint8_t* codes, int64_t n, int fmt);
/* Absmax-scaled quantization of `rows` slices: scale = absmax/max_val (1.0 for an all-zero slice),
 * code = encode(x/scale).  The per-tensor rule of crates/oxicuda-dnn/src/quantize/fp8_quantize.rs:28-34
 * composed with the codec; rows=1 is per-tensor, rows>1 per-row (per-token / per-output-channel). */
int32_t b2q_fp8_quantize_rows_f32(b2q_handle h, const float* x, int64_t rows, int64_t cols, int fmt,
                                  int rounding, float* scales, uint8_t* codes);
/* Same, bf16 input (activations). */
int32_t b2q_fp8_quantize_rows_bf16(b2q_handle h, const void* x_bf16, int64_t rows, int64_t cols, int fmt,
                                   int rounding, float* scales, uint8_t* codes);

/* SwiGLU between the gate/up and down projections, fused with the per-token re-quantization of its result:
 * h = silu(gate) * up in fp32, silu(x) = x / (1 + exp(-x)) (crates/oxicuda-lm/src/layer/ffn.rs:25-27,
 * SwiGluExpert::forward crates/oxicuda-moe/src/expert/ffn.rs:208-243), then scale = absmax(h)/max_val per row and
 * code = encode(h/scale).  gate/up: bf16 [rows x cols] with leading dimension ld (they may be the two halves of one
 * [rows x 2*cols] GEMM output). */
int32_t b2q_swiglu_quantize_rows_bf16(b2q_handle h, const void* gate, const void* up, int64_t rows, int64_t cols,
                                      int64_t ld, int fmt, int rounding, float* scales, uint8_t* codes);

/* No counterpart in the reference.  The same quantizer for callers that cannot allocate device memory: a plugin
 * living inside a host process that has handed out all of its memory budget, or code in a region where the allocator
 * must not be touched.  It needs no handle (creating one allocates) and calls neither cudaMalloc nor cudaFree: the
 * reduction scratch is a fixed array inside the library (16.25 KiB per GPU for the life of the process), which limits
 * `rows` to 1024 slices per call (B2Q_ERR_BUFFER_TOO_SMALL beyond that, with the reason written to `err`).
 * The first call on each device looks up the array's address; make that call outside stream capture.  All calls on a
 * device share the array, so calls that may overlap on the GPU must be ordered by the caller.  `stream` is a
 * cudaStream_t; `device_status` (1 x int32 on the device, zeroed by the caller) receives
 * B2Q_ERR_NON_FINITE_FP8 if the input holds NaN/Inf; with NULL that detection is off (there is no handle whose status
 * word could hold it) and non-finite inputs are encoded silently; `err`/`err_len` (optional) receive a message on failure.
 * Same results as b2q_fp8_quantize_rows_f32. */
int32_t b2q_fp8_quantize_rows_f32_noalloc(const float* x, int64_t rows, int64_t cols, int fmt, int rounding,
                                          float* scales, uint8_t* codes, void* stream, int32_t* device_status,
                                          char* err, size_t err_len);

/* ---- MicroScalingQuantizer / Fp4Quantizer / PackedFp4: crates/oxicuda-blas/src/precision/fp4_fp6_ops.rs ---- */
/* quantize_fp4 (:849-876): blocks of `block` in {32,64,128} over the flat array (validate :205-214),
 * two codes per byte, element 2i in the low nibble (PackedFp4::pack :465-472).  n must be a multiple of
 * `block` on the device path.  scales: ceil(n/block) floats (B2Q_SCALE_F32) or bytes (B2Q_SCALE_E8M0). */
int32_t b2q_fp4_block_quantize_f32(b2q_handle h, const float* x, int64_t n, int block, int format,
                                   int scale_format, uint8_t* packed, void* scales);
/* dequantize_fp4 (:879-897) */
int32_t b2q_fp4_block_dequantize_f32(b2q_handle h, const uint8_t* packed, int64_t n, int block, int format,
                                     int scale_format, const void* scales, float* out);

/* ---- Nf4Quantizer::decode / nf4_dequant kernel: crates/oxicuda-quant/src/scheme/nf4.rs:127-150,
 *      crates/oxicuda-quant/src/ptx_kernels.rs:267-412 ---- */
int32_t b2q_nf4_decode_f32(b2q_handle h, const uint8_t* packed, int64_t nbytes, int block,
                           const float* absmaxs, float* out);
/* Nf4Quantizer::encode (nf4.rs:93-125) */
int32_t b2q_nf4_encode_f32(b2q_handle h, const float* x, int64_t n, int block, uint8_t* packed, float* absmaxs);

/* ---- int8_quant / int8_dequant kernels: crates/oxicuda-quant/src/ptx_kernels.rs:129-252 ----
 * out = i8(clamp(rni(x/scale), -127, 127)) (ties to even, as cvt.rni) ; out = f32(q)*scale */
int32_t b2q_int8_quant_f32(b2q_handle h, const float* x, int64_t n, float scale, int8_t* out);
int32_t b2q_int8_dequant_f32(b2q_handle h, const int8_t* q, int64_t n, float scale, float* out);

/* ---- dist-infer "FP8" (INT8 in a u8): crates/oxicuda-dist-infer/src/quantisation/fp8_infer.rs:61-142 ----
 * per-block absmax is stored; block >= n gives the per-tensor variant. */
int32_t b2q_distfp8_quantize_block_f32(b2q_handle h, const float* x, int64_t n, int64_t block, uint8_t* q,
                                       float* absmaxs);
int32_t b2q_distfp8_dequantize_block_f32(b2q_handle h, const uint8_t* q, int64_t n, int64_t block,
                                         const float* absmaxs, float* out);

/* ---- RMSNorm fused with the per-token FP8 quantizer of the next linear ----
 * y = x / sqrt(mean(x^2) + eps) * gamma per row (rms_norm, crates/oxicuda-dnn/src/norm/rms_norm.rs:29-33, CPU statement
 * :566-574), then the per-token rule of b2q_fp8_quantize_rows_bf16 on y in f32: scale = absmax(y)/max_val per row,
 * code = encode(y/scale).  x, gamma: bf16.  residual (optional, bf16 [rows x cols], updated in place) selects
 * fused_add_rms_norm (rms_norm.rs:98-103): residual = bf16(residual + x) and the norm is taken of the stored sum.
 * y_out (optional, bf16) also receives the normalised activations.  Floating-point path, not bit-exact: the f32 sum
 * of squares is a tree sum and the two divisions are multiplications by correctly rounded reciprocals (the
 * reference's own GPU kernel uses rsqrt.approx), so y is within a few f32 ulp of the CPU statement and a code can
 * differ from the two-kernel composition where y/scale falls on an FP8 rounding boundary. */
int32_t b2q_rms_norm_quantize_fp8_bf16(b2q_handle h, const void* x_bf16, void* residual_bf16, const void* gamma_bf16,
                                       int64_t rows, int64_t cols, float eps, int fmt, int rounding, float* scales,
                                       uint8_t* codes, void* y_out_bf16);

/* ---- KvCacheQuantizer: crates/oxicuda-quant/src/scheme/kv_cache.rs ---- */
typedef enum { B2Q_KV_PER_TOKEN = 0, B2Q_KV_PER_CHANNEL = 1 } b2q_kv_axis;  /* KvAxis, kv_cache.rs:33-38 */
/* quantize (:146-221): x is [n_tokens x head_dim] row-major; codes (one per byte, as the reference's Vec<u8>) lie in
 * [0, 2^bits-1], bits in [2, 8] (KvCacheConfig::new :59-64, else B2Q_ERR_INVALID_BIT_WIDTH); scales / zero_points hold
 * one f32 per group: n_tokens of them for B2Q_KV_PER_TOKEN, head_dim for B2Q_KV_PER_CHANNEL.  Bit-exact.
 * append_token (:254-282) is this call with n_tokens = 1 and the output pointers advanced to the new row. */
int32_t b2q_kv_cache_quantize_f32(b2q_handle h, const float* x, int64_t n_tokens, int64_t head_dim, int bits, int axis,
                                  uint8_t* codes, float* scales, float* zero_points);
int32_t b2q_kv_cache_quantize_bf16(b2q_handle h, const void* x_bf16, int64_t n_tokens, int64_t head_dim, int bits,
                                   int axis, uint8_t* codes, float* scales, float* zero_points);
/* dequantize (:224-238): code * scale + zero_point, unfused.  The bf16 form rounds that f32 value to nearest even. */
int32_t b2q_kv_cache_dequantize_f32(b2q_handle h, const uint8_t* codes, int64_t n_tokens, int64_t head_dim, int axis,
                                    const float* scales, const float* zero_points, float* out);
int32_t b2q_kv_cache_dequantize_bf16(b2q_handle h, const uint8_t* codes, int64_t n_tokens, int64_t head_dim, int axis,
                                     const float* scales, const float* zero_points, void* out_bf16);
/* ---- quantize_token: crates/oxicuda-infer/src/cache/kv_quant.rs:112-154, for n_tokens vectors of d channels ----
 * bits is 4 or 8 (KvQuantConfig::new :48-53, else B2Q_ERR_INVALID_CONFIG); symmetric codes lie in
 * [-(2^(bits-1)-1), 2^(bits-1)-1] and are stored as int8, asymmetric ones in [0, 2^bits-1] as uint8 (the reference
 * holds them as Vec<i32>; q_range :69-76).  An empty input is B2Q_ERR_INVALID_CONFIG as in the reference (:113-115). */
int32_t b2q_kv_quantize_tokens_f32(b2q_handle h, const float* x, int64_t n_tokens, int64_t d, int bits, int symmetric,
                                   uint8_t* codes, float* scales, float* zero_points);
int32_t b2q_kv_quantize_tokens_bf16(b2q_handle h, const void* x_bf16, int64_t n_tokens, int64_t d, int bits,
                                    int symmetric, uint8_t* codes, float* scales, float* zero_points);
/* QuantizedToken::dequantize (:94-100): scale * code + zero_point. */
int32_t b2q_kv_dequantize_tokens_f32(b2q_handle h, const uint8_t* codes, int64_t n_tokens, int64_t d, int symmetric,
                                     const float* scales, const float* zero_points, float* out);
int32_t b2q_kv_dequantize_tokens_bf16(b2q_handle h, const uint8_t* codes, int64_t n_tokens, int64_t d, int symmetric,
                                      const float* scales, const float* zero_points, void* out_bf16);

/* ---- oxicuda-dnn quantize: crates/oxicuda-dnn/src/quantize/ (the statements its GPU tests check bit for bit,
 * crates/oxicuda-dnn/src/gpu_tests/quantize.rs:184-325, :503-554) ---- */
/* quantize_to_fp8 (fp8_quantize.rs:45-122): scale[0] = max(absmax / 448, 1e-12); code = E4M3(clamp(x / scale, +-448))
 * with ties to even and saturation to 0x7E.  n = 0 is a no-op, as in the reference. */
int32_t b2q_dnn_quantize_to_fp8_f32(b2q_handle h, const float* x, int64_t n, uint8_t* codes, float* scale);
/* dequantize_from_fp8 (:125-170): out = e4m3(code) * scale[0]; subnormal codes are m / 512. */
int32_t b2q_dnn_dequantize_from_fp8_f32(b2q_handle h, const uint8_t* codes, const float* scale, int64_t n, float* out);
/* quantize_to_int8 (int8_quantize.rs:31-102): scale[0] = max(absmax / 127, 1e-12); q = rne(clamp(x / scale, +-127)). */
int32_t b2q_dnn_quantize_to_int8_f32(b2q_handle h, const float* x, int64_t n, int8_t* q, float* scale);
/* dequantize_from_int8 (:105-160): out = q * scale[0]. */
int32_t b2q_dnn_dequantize_from_int8_f32(b2q_handle h, const int8_t* q, const float* scale, int64_t n, float* out);
/* quantize_block_scaled (block_scale.rs:51-150): per block of block_size (a power of two >= 16, else
 * B2Q_ERR_INVALID_ARGUMENT) scale = max(absmax / 6, 1e-12); byte = clamp(rne(clamp(x / scale, +-6)) + 6, 0, 255);
 * ceil(n / block_size) scales. */
int32_t b2q_dnn_quantize_block_scaled_f32(b2q_handle h, const float* x, int64_t n, uint32_t block_size, uint8_t* out,
                                          float* scales);
/* BlockQuantizedInt8::{quantize,dequantize} (int8_quantize.rs:427-470): scale = absmax / 127 (1 for a zero block),
 * q = round_half_away(x / scale) clamped to [-128, 127]; the last block may be short. */
int32_t b2q_block_int8_quantize_f32(b2q_handle h, const float* x, int64_t n, int64_t block_size, int8_t* q, float* scales);
int32_t b2q_block_int8_dequantize_f32(b2q_handle h, const int8_t* q, const float* scales, int64_t n, int64_t block_size,
                                      float* out);
/* Fp4BlockQuantizer::compute_scale (block_scale.rs:437-444) for every block: absmax / max_val, 1 for a zero block. */
int32_t b2q_block_absmax_scale_f32(b2q_handle h, const float* x, int64_t n, int64_t block_size, float max_val,
                                   float* scales);

/* ---- INT4 group-scaled weight-only linear: crates/oxicuda-blas/src/precision/int_ops.rs ---- */
/* pack_int4 (:375-403): eight two's-complement nibbles per u32, value j in bits [4j, 4j+4).  n must be a multiple of 8
 * (B2Q_ERR_INVALID_ARGUMENT); a value outside [-8, 7] records B2Q_ERR_INVALID_ARGUMENT in the device status word
 * (read it with b2q_check).  values: int8 on the device, 8-byte aligned. */
int32_t b2q_pack_int4(b2q_handle h, const int8_t* values, int64_t n, uint32_t* packed);
/* unpack_int4 (:415-429) for `words` packed words -> 8 * words sign-extended int8. */
int32_t b2q_unpack_int4(b2q_handle h, const uint32_t* packed, int64_t words, int8_t* out);
/* The kernel of generate_int4_gemm_ptx (:602-757) with its own operand layout and summation order:
 * C[m x n] (f32) = dequant(A) * B, A packed [m x k/8] u32, scales f16 [m x k/group_size], B f32 [k x n] row-major;
 * acc = fma(float(int4) * scale, B[k, col], acc) for k ascending.  Bit-exact against that statement.
 * Validation as Int4GemmConfig::validate (:250-283). */
int32_t b2q_gemm_int4_f32(b2q_handle h, const uint32_t* a_packed, const void* scales_f16, const float* b, float* c,
                          int64_t m, int64_t n, int64_t k, int64_t group_size);
/* The decode form of the same linear: out[tokens x n] = x[tokens x k] (bf16) * dequant(W)^T, W packed [n x k/8],
 * scales f16 [n x k/group_size]; tokens <= 32, k % 128 == 0, group_size >= 32 (else B2Q_ERR_UNSUPPORTED).
 * Activations enter the tensor core as f16 (saturating at +-65504), fp32 accumulation. */
int32_t b2q_gemv_int4_wo(b2q_handle h, const uint32_t* packed, const void* scales_f16, int64_t group_size,
                         const void* x_bf16, int64_t tokens, int64_t n, int64_t k, void* out, int out_type);

/* ---- LlmInt8Quantizer::matmul: crates/oxicuda-quant/src/scheme/llm_int8.rs:175-288 ----
 * x [samples x cols] f32, w [rows x cols] f32 -> out [samples x rows] f32.  Per-row INT8 of W and per-token
 * (row_wise != 0) or per-tensor INT8 of X over the non-outlier columns, exact integer accumulation,
 * out = f32(acc)*(sx*sw[k]) + f32 dot over outlier columns (a column whose max |x| >= threshold).
 * Optional dumps for parity checks (each may be NULL): wq [rows x cols] i8, sw [rows], xq [samples x cols] i8,
 * sx [samples], acc [samples x rows] i32, n_outliers (1 x i32, device). */
int32_t b2q_llm_int8_linear_f32(b2q_handle h, const float* x, const float* w, int64_t samples, int64_t rows,
                                int64_t cols, float threshold, int row_wise, float* out, int8_t* wq, float* sw,
                                int8_t* xq, float* sx, int32_t* acc, int32_t* n_outliers);

/* ---- INT8 GEMM: Int8GemmConfig / generate_int8_gemm_ptx crates/oxicuda-blas/src/precision/int_ops.rs:78-189, :446-583 ----
 * C[m,n] = sum_k A[m,k]*B[n,k], exact s32.  A [M x K] row-major, B [N x K] row-major ("out x in" weights; the
 * reference's K-packed-by-4 [K/4 x N] u32 operand holds the same values).  K % 4 == 0 (validate :113-118).
 * c_s32 and/or c_f32 (AccType::F32: cvt.rn.f32.s32 times scale_a[m]*scale_b[n] when scales are given). */
int32_t b2q_gemm_i8(b2q_handle h, const int8_t* a, const int8_t* b, int64_t M, int64_t N, int64_t K,
                    int32_t* c_s32, float* c_f32, const float* scale_a, const float* scale_b);

/* ---- FP8 GEMM: gemm::<E4M3> crates/oxicuda-blas/src/level3/gemm_api.rs:82-231 (the reference's generator
 *      rejects FP8, crates/oxicuda-ptx/src/templates/gemm.rs:800-809; this is the working path) ----
 * out[m,n] = (sum_k A[m,k]*W[n,k]) * sa * sw, f32 accumulate in TMEM, bf16 (RNE) or f32 store.
 * A [M x K] codes row-major, W [N x K] codes row-major (K-major both: tcgen05 "TN").
 * scale_a: 1 float (B2Q_SCALE_SCALAR) or M floats (B2Q_SCALE_PER_ROW); scale_w: 1 or N floats.
 * Validation order follows gemm_impl: zero dims -> INVALID_DIMENSION (:142-146); K % 16 != 0 -> INVALID_DIMENSION
 * (TMA row pitch); C overlapping A/W -> INVALID_ARGUMENT (:189-195). */
int32_t b2q_gemm_fp8(b2q_handle h, const uint8_t* a, const uint8_t* w, int64_t M, int64_t N, int64_t K, int fmt,
                     const float* scale_a, int scale_a_kind, const float* scale_w, int scale_w_kind,
                     void* out, int out_type);
/* The general form, gemm_impl of crates/oxicuda-blas/src/level3/gemm_api.rs:126-231 with an EpilogueOp
 * (crates/oxicuda-blas/src/level3/gemm/epilogue.rs:29-120):
 *   out = act(alpha * (A W^T) * sa * sw + beta * out + bias[col])
 * in the reference's order (mul by alpha, fma with beta * C_old, add bias, then max(0, .) or gelu as x * sigmoid(1.702 x),
 * epilogue.rs:99-196).  w_layout = B2Q_W_KN takes the reference's row-major [K x N] operand B (transposed into the
 * handle's workspace on every call: hold weights as [N x K] where that matters).  The prefill tcgen05 kernels apply the
 * epilogue in their store path; few-token shapes run their kernel into the workspace and one elementwise pass. */
typedef enum { B2Q_EPI_LINEAR = 0, B2Q_EPI_RELU = 1, B2Q_EPI_GELU = 2, B2Q_EPI_BIAS = 3, B2Q_EPI_BIAS_RELU = 4,
               /* no counterpart in EpilogueOp: w holds gate and up rows interleaved per 128 (b2q_interleave_rows128), n % 256 == 0,
                * out is [m x n / 2] = silu(gate) * up (SwiGluExpert::forward, crates/oxicuda-moe/src/expert/ffn.rs:208-243);
                * alpha, beta and bias are not applied */
               B2Q_EPI_SWIGLU = 5 } b2q_epilogue_op;
typedef enum { B2Q_W_NK = 0, B2Q_W_KN = 1 } b2q_w_layout;
typedef struct {
  const uint8_t* a; const uint8_t* w; int64_t m, n, k; int32_t fmt;
  const float* scale_a; int32_t scale_a_kind; const float* scale_w; int32_t scale_w_kind;
  void* out; int32_t out_type;
  float alpha, beta; const float* bias; int32_t epilogue; int32_t w_layout;
} b2q_gemm_fp8_desc;
int32_t b2q_gemm_fp8_ex(b2q_handle h, const b2q_gemm_fp8_desc* d);
/* Checker path on the GPU: software decode (reference or IEEE), k-ascending fp32 FMA, one thread per output
 * — the arithmetic of the reference's naive kernel (crates/oxicuda-ptx/src/templates/gemm.rs:373-447). */
int32_t b2q_gemm_fp8_simt(b2q_handle h, const uint8_t* a, const uint8_t* w, int64_t M, int64_t N, int64_t K, int fmt,
                          int decode_mode, const float* scale_a, int scale_a_kind, const float* scale_w,
                          int scale_w_kind, void* out, int out_type);

/* ---- tensor-parallel linears: ColumnLinear / RowLinear crates/oxicuda-dist-infer/src/tensor_parallel/column_parallel.rs:103-205,
 *      row_parallel.rs:97-224; DistInferHandle crates/oxicuda-dist-infer/src/handle.rs:62-239.  One rank per process and GPU.
 * A b2q_tp binds a handle to an NCCL communicator of `tp` ranks (ncclComm_t passed as void*; NCCL is resolved at run
 * time from the libnccl.so.2 already loaded in the process).  It owns a second stream for overlapped collectives,
 * grow-only scratch (the first call with a larger shape allocates: warm up before capturing a CUDA graph) and, for
 * tp > 1, a 36 MiB exchange buffer for the peer-memory all-reduce of few-token results. ---- */
typedef struct b2q_tp_s* b2q_tp;
/* Helpers for callers without an NCCL binding of their own: ncclGetUniqueId / ncclCommInitRank (on the current
 * device) / ncclCommDestroy.  id128: 128 bytes, made on one rank and sent to the others by the caller. */
int32_t b2q_tp_unique_id(uint8_t* id128);
int32_t b2q_tp_comm_init(const uint8_t* id128, int tp, int rank, void** nccl_comm);
int32_t b2q_tp_comm_destroy(void* nccl_comm);
int32_t b2q_tp_create(b2q_handle h, void* nccl_comm, int tp, int rank, b2q_tp* out);   /* nccl_comm may be NULL for tp = 1 */
int32_t b2q_tp_destroy(b2q_tp t);
/* The exchange buffer of this rank: its device pointer and/or its 64-byte CUDA IPC handle.  Every rank sends its
 * handle to the others (any host channel) and passes the tp handles, in rank order, to b2q_tp_attach_peers; ranks
 * that share a process pass mapped pointers instead (direct_ptrs[r], peer access enabled by the caller).  Until peers
 * are attached every row-parallel boundary goes through NCCL. */
int32_t b2q_tp_exchange_buffer(b2q_tp t, void** ptr, uint8_t* ipc_handle64);
int32_t b2q_tp_attach_peers(b2q_tp t, const uint8_t* ipc_handles, void* const* direct_ptrs);
/* The row-parallel partial product with the reduce-scatter folded into its epilogue (the first half of boundary mode 4,
 * usable on its own): out = a [M x K] . w [N x K]^T with per-row scales (+ bias [N] on the rank that carries it), bf16;
 * rows [o * M / tp, (o + 1) * M / tp) are stored into inbox[o] -- rank o's buffer [tp][M / tp][N] bf16, a device pointer
 * valid on this GPU (peer-mapped, or local for o == rank) -- at slot `rank`.  Nothing waits in this kernel: the caller
 * orders the readers behind every rank's launch.  M > 128, N > 128, M % (32 * tp) == 0, N % 8 == 0, K % 16 == 0. */
int32_t b2q_gemm_fp8_scatter(b2q_handle h, const uint8_t* a, const uint8_t* w, int64_t M, int64_t N, int64_t K, int fmt,
                             const float* scale_a, const float* scale_w, const float* bias, void* const* inbox, int tp, int rank);
/* Chunks of the many-token paths (0 = automatic, see b2q_tp_plan). */
int32_t b2q_tp_set_chunks(b2q_tp t, int chunks);
/* The boundary a row-parallel result of tokens x out_features takes: mode 0 none (tp = 1); 1 one-shot and 2 two-shot
 * peer-memory kernel (fp32 partials up to 256 KiB / 4 MiB: every rank pushes its partial into its peers' inboxes over
 * NVLink, waits on per-CTA flags with a one-second limit (B2Q_ERR_TIMEOUT in the status word) and adds the partials in
 * rank order in fp32, the reference's order, row_parallel.rs:202-223); 4 (bf16 results up to 64 MiB, tokens a multiple
 * of 32 * tp) the reduce-scatter is part of the GEMM: its epilogue stores every row block as bf16 into the inbox of the
 * rank that owns those rows, then one kernel waits for the peers (same limit), adds the tp partials of its own rows in
 * rank order in fp32 and pushes the bf16 sums to every rank; with b2q_tp_set_chunks > 1 the GEMM is cut into column
 * chunks and that kernel runs on a second stream under the GEMM of the next chunk (the plan itself says 1);
 * 3 NCCL all-reduce of bf16 partials (anything else, or no peers attached), `chunks` token chunks.
 * Every rank gets the same bits in modes 1, 2 and 4.  Pure host function. */
int32_t b2q_tp_plan(int tp, int peers_attached, int64_t tokens, int64_t out_features, int* mode, int* chunks);
/* Sum over ranks of fp32 partials [n] -> bf16 on every rank through the peer kernel (n % (4 * tp) == 0, n * 4 <= 4 MiB,
 * peers attached); and the in-place NCCL sum of a bf16 buffer on the handle's stream. */
int32_t b2q_tp_all_reduce_f32_to_bf16(b2q_tp t, const float* partial, int64_t n, void* y_bf16);
int32_t b2q_tp_all_reduce_bf16(b2q_tp t, void* y_bf16, int64_t n);
/* ColumnLinear::forward (column_parallel.rs:168-179): y_local [tokens x out_local] bf16 = x W_s^T + bias_s over this
 * rank's out/tp rows of W (E4M3 codes, per-token and per-row scales); bias: f32 [out_local] or NULL.  With y_gathered
 * != NULL also ColumnLinear::all_gather (:181-204): [tokens x out_local * tp], shard r at columns [r * out_local, ...). */
int32_t b2q_column_linear_forward(b2q_tp t, const uint8_t* x_codes, const float* x_scales, const uint8_t* w_codes,
                                  const float* w_scales, const float* bias, int64_t tokens, int64_t in_features,
                                  int64_t out_local, void* y_local, void* y_gathered);
/* RowLinear::forward + all_reduce (row_parallel.rs:170-223): x_codes [tokens x in_local] is this rank's column slice of
 * the activations, w_codes [out x in_local] its columns of W; bias (f32 [out] or NULL) is added on rank 0 only (:183-190);
 * y [tokens x out] bf16 holds the sum over ranks on every rank. */
int32_t b2q_row_linear_forward_allreduce(b2q_tp t, const uint8_t* x_codes, const float* x_scales, const uint8_t* w_codes,
                                         const float* w_scales, const float* bias, int64_t tokens, int64_t in_local,
                                         int64_t out_features, void* y);
/* SwiGluExpert::forward (crates/oxicuda-moe/src/expert/ffn.rs:208-243) over ColumnLinear (gate | up, one GEMM over the
 * concatenated [2 * ffn_local x hidden] shard) and RowLinear (down [hidden x ffn_local]): x bf16 [tokens x hidden] is
 * quantized per token (absmax / 448), h = silu(gate) * up is re-quantized per token over this rank's columns,
 * y bf16 [tokens x hidden] is the sum over ranks. */
int32_t b2q_mlp_swiglu_fp8_forward(b2q_tp t, const void* x_bf16, const uint8_t* w_gate_up, const float* s_gate_up,
                                   const uint8_t* w_down, const float* s_down, int64_t tokens, int64_t hidden,
                                   int64_t ffn_local, int rounding, void* y_bf16);
/* The same layer with the layout of the gate | up shard stated.  B2Q_GATE_UP_INTERLEAVED128 (ffn_local % 128 == 0): rows
 * [256 j, 256 j + 128) are gate rows [128 j, ...), the next 128 the same up rows (and the scales likewise), as
 * b2q_interleave_rows128 writes them.  One accumulator tile of the gate | up GEMM then holds both projections of the same
 * hidden units, so above 128 tokens silu(gate) * up is formed in the GEMM epilogue and only h [tokens x ffn_local] bf16 is
 * written (the bf16 rounding of h, 2^-9, is far below the E4M3 step that follows); few-token steps read the interleaved
 * GEMM result directly.  No counterpart in the reference, which multiplies the three matrices one after the other. */
typedef enum { B2Q_GATE_UP_CONCATENATED = 0, B2Q_GATE_UP_INTERLEAVED128 = 1 } b2q_gate_up_layout;
int32_t b2q_mlp_swiglu_fp8_forward_ex(b2q_tp t, const void* x_bf16, const uint8_t* w_gate_up, const float* s_gate_up,
                                      const uint8_t* w_down, const float* s_down, int64_t tokens, int64_t hidden,
                                      int64_t ffn_local, int rounding, int gate_up_layout, void* y_bf16);
/* out [2 * rows x row_bytes] = the rows of a and of b interleaved per 128 rows (rows % 128 == 0; row_bytes a multiple of
 * 16, or 4 for a vector of per-row scales): a load-time step, one pass over the weights. */
int32_t b2q_interleave_rows128(b2q_handle h, const void* a, const void* b, int64_t rows, int64_t row_bytes, void* out);

/* ---- grouped GEMM: grouped_gemm / GroupedGemmProblem crates/oxicuda-blas/src/batched/grouped_gemm.rs:46-78 ----
 * One FP8 GEMM per entry of a host-side problem table (an expert and the tokens routed to it); entries with m == 0 are
 * skipped.  Problems are issued back to back on the handle's stream (the reference launches them one by one up to four
 * problems and uses a table-driven kernel beyond). */
typedef struct {
  const uint8_t* a; const uint8_t* w; int64_t m, n, k;
  const float* scale_a; int32_t scale_a_kind; const float* scale_w; int32_t scale_w_kind; void* out;
} b2q_gemm_fp8_problem;
int32_t b2q_grouped_gemm_fp8(b2q_handle h, const b2q_gemm_fp8_problem* problems, int count, int fmt, int out_type);

/* The table-driven form (what the reference uses above four problems, grouped_gemm.rs:46-78) with the table ON THE DEVICE,
 * for problems that share N and K and differ in their row count (experts of one layer): ONE launch, a persistent kernel
 * walks the 256 x 256 tiles of every problem.  Problem g multiplies rows [row_offsets[g], row_offsets[g] + row_counts[g])
 * of a [capacity_rows x K] (scale_a: one float per row) with rows [g * N, (g + 1) * N) of w [groups * N x K] (scale_w
 * likewise) and stores the same rows of out [capacity_rows x N].  row_offsets must be multiples of 256 with every
 * problem's rows inside [0, capacity_rows); the rows of a problem's last tile past its count are computed and stored
 * too (they belong to no other problem).  No host synchronisation: counts and offsets may come from the kernel before. */
int32_t b2q_grouped_gemm_fp8_rows(b2q_handle h, const uint8_t* a, const float* scale_a, const uint8_t* w, const float* scale_w,
                                  const int32_t* row_offsets, const int32_t* row_counts, int groups, int64_t capacity_rows,
                                  int64_t N, int64_t K, int fmt, void* out, int out_type);

/* ---- expert dispatch: ep_token_scatter / ep_token_gather crates/oxicuda-dist-infer/src/ptx_kernels.rs:46-469,
 *      ExpertDispatcher::{scatter,gather} crates/oxicuda-dist-infer/src/expert_parallel/dispatch.rs:99-219 ----
 * scatter: expert_buf[slot[i]] = in[token[i]] for each routed pair i (rows of row_bytes bytes, a multiple of 16);
 * gather: out[t] = sum_j weight[t*top_k+j] * expert_out[slot[t*top_k+j]] in fp32, j ascending, bf16 in and out;
 * a negative slot marks a pair served by another rank and contributes nothing. */
int32_t b2q_ep_token_scatter(b2q_handle h, const void* in, const int32_t* token, const int32_t* slot, int64_t pairs,
                             int64_t row_bytes, void* expert_buf);
int32_t b2q_ep_token_gather_bf16(b2q_handle h, const void* expert_out, const int32_t* slot, const float* weight,
                                 int64_t tokens, int top_k, int64_t hidden, void* out);

/* Device-side routing and slotting (no host synchronisation), the pieces b2q_moe_forward is made of:
 * TopKRouter::route (expert_parallel/router.rs:94-140): per token the top_k experts by descending logit (equal logits
 * keep index order, as the reference's stable sort) and the softmax of those k logits; at most 64 experts, top_k <= 8. */
int32_t b2q_moe_route_topk(b2q_handle h, const float* logits, int64_t tokens, int n_experts, int top_k, int32_t* expert_idx,
                           float* weight);
/* Counts the pairs routed to experts [first_local, first_local + n_local), lays the experts out at row offsets padded to
 * multiples of 256 (offsets[n_local + 1], the layout b2q_grouped_gemm_fp8_rows takes) and gives every such pair a row
 * (slot_of_pair, -1 for pairs of other ranks).  Rows within an expert are handed out in arrival order. */
int32_t b2q_moe_assign_slots(b2q_handle h, const int32_t* expert_idx, int64_t pairs, int first_local, int n_local,
                             int32_t* counts, int32_t* offsets, int32_t* slot_of_pair);
/* expert_buf[slot_of_pair[i]] = x[i / top_k] for every pair with a slot (ExpertDispatcher::scatter, dispatch.rs:99-150). */
int32_t b2q_moe_scatter(b2q_handle h, const void* x, const int32_t* slot_of_pair, int64_t pairs, int top_k, int64_t row_bytes,
                        void* expert_buf);
/* ExpertDispatcher::dispatch_and_gather (dispatch.rs:99-219) over SwiGluExpert::forward (crates/oxicuda-moe/src/expert/ffn.rs:208-243)
 * with FP8 weights, experts sharded over the ranks of `t` (expert parallel: rank r owns experts [r * E / ep, ...)):
 * x bf16 [tokens x hidden] and logits f32 [tokens x n_experts] are replicated; w_gate_up [E/ep][2 * ffn][hidden] and
 * w_down [E/ep][hidden][ffn] are this rank's experts (E4M3 codes, one scale per row); y bf16 [tokens x hidden] is the
 * weighted sum over each token's top_k experts, on every rank (one all-reduce adds the ranks' contributions).
 * Everything is enqueued without reading anything back: routing, slotting, scatter, per-row quantization, one grouped
 * gate|up GEMM, SwiGLU + re-quantization, one grouped down GEMM, gather.  counts_out (optional, device int32 [E/ep])
 * receives the number of pairs each local expert served. */
int32_t b2q_moe_forward(b2q_tp t, const void* x_bf16, const float* logits, const uint8_t* w_gate_up, const float* s_gate_up,
                        const uint8_t* w_down, const float* s_down, int64_t tokens, int64_t hidden, int64_t ffn, int n_experts,
                        int top_k, int rounding, void* y_bf16, int32_t* counts_out);
/* The same with the layout of every expert's gate | up block stated (see b2q_mlp_swiglu_fp8_forward_ex): with
 * B2Q_GATE_UP_INTERLEAVED128 (ffn % 128 == 0) silu(gate) * up is formed in the epilogue of the grouped GEMM. */
/* The layer over block-scaled FP4 experts (config 5's FP4 runs): c_gate_up [E/ep][2 * ffn][hidden / 2] and c_down
 * [E/ep][hidden][ffn / 2] are E2M1 codes (PackedFp4 bytes), s_* one E8M0 byte per 32 codes along K
 * (MicroScalingQuantizer, fp4_fp6_ops.rs:746-898, with the power-of-two scale rule of b2q_fp4_block_quantize_f32); gate rows
 * then up rows per expert.  Both grouped GEMMs are ONE launch each of the tcgen05 block-scaled kernel
 * (b2q_grouped_gemm_fp4_rows); act_mode as in b2q_gemm_fp4_blockscaled; hidden and ffn multiples of 128. */
int32_t b2q_moe_forward_fp4(b2q_tp t, const void* x_bf16, const float* logits, const uint8_t* c_gate_up, const uint8_t* s_gate_up,
                            const uint8_t* c_down, const uint8_t* s_down, int64_t tokens, int64_t hidden, int64_t ffn, int n_experts,
                            int top_k, int act_mode, void* y_bf16, int32_t* counts_out);
int32_t b2q_moe_forward_ex(b2q_tp t, const void* x_bf16, const float* logits, const uint8_t* w_gate_up, const float* s_gate_up,
                           const uint8_t* w_down, const float* s_down, int64_t tokens, int64_t hidden, int64_t ffn, int n_experts,
                           int top_k, int rounding, int gate_up_layout, void* y_bf16, int32_t* counts_out);

/* ---- FP4 weight-only decode GEMV: Fp4GemmConfig / generate_fp4_gemm_ptx
 *      crates/oxicuda-blas/src/precision/fp4_fp6_ops.rs:337-395, :1237-1362; semantics = dequantize_fp4 (:879-897)
 *      followed by a dot product.  The reference's M (quantized rows) is `N` here, its N (columns of dense B) is
 *      `tokens`; activations are taken token-major [tokens x K] bf16 instead of [K x tokens] f32.
 * codes [N x K/2] (E2M1, low nibble first), scales [N x K/32] f32 or E8M0 bytes, x [tokens x K] bf16,
 * out [tokens x N] bf16 or f32.  tokens <= 32, K % 128 == 0, block == 32.
 * With E8M0 scales, K % 512 == 0, codes 32-byte aligned and scales 16-byte aligned, matrices from 16 MiB of codes run on
 * the block-scaled tensor-core kernel (weights and scales as stored; each bf16 activation enters as the sum of two E4M3
 * terms under a power-of-two scale per 32 values, absolute error below 2^-18 of the largest of the 32); it uses the
 * handle's workspace, and consecutive calls on the stream overlap (programmatic dependent launch).  Everything else
 * runs kernels that use the activations exactly. */
int32_t b2q_gemv_fp4_wo(b2q_handle h, const uint8_t* codes, const void* scales, int scale_format, int block,
                        const void* x_bf16, int64_t tokens, int64_t N, int64_t K, void* out, int out_type);

/* Weight-only FP4 GEMM for any token count (prefill): same operands and semantics as b2q_gemv_fp4_wo plus `format`
 * (B2Q_FP4_E2M1 or B2Q_FP4_INT4) and blocks of 32, 64 or 128.  32 tokens or fewer go to the decode GEMV; above that E2M1
 * codes with E8M0 scales of block 32 run on the block-scaled tensor-core GEMM (b2q_gemm_fp4_blockscaled, split
 * activations); what that instruction cannot express (f32 scales, INT4 codes, blocks of 64 / 128) is expanded to bf16 in
 * the handle's workspace (N*K*2 bytes) and multiplied on tcgen05 (kind::f16, fp32 accumulation).  Fp4GemmConfig::validate order: zero dims, odd K, block size
 * (crates/oxicuda-blas/src/precision/fp4_fp6_ops.rs:354-376). */
int32_t b2q_gemm_fp4_wo(b2q_handle h, const uint8_t* codes, const void* scales, int scale_format, int block, int format,
                        const void* x_bf16, int64_t tokens, int64_t N, int64_t K, void* out, int out_type);

/* The same product on the block-scaled tensor-core instruction (tcgen05.mma kind::mxf8f6f4.block_scale): E2M1 codes and
 * E8M0 block scales (block 32) feed the MMA as stored, nothing is expanded in HBM.  K % 128 == 0, codes 32-byte aligned.
 * act_mode: B2Q_FP4_ACT_SPLIT keeps weight-only semantics (every bf16 activation enters as the sum of two E4M3 codes under
 * its 32-block's power-of-two scale, exact to 2^-18 of the block maximum; 64 tokens per 128-row tile);
 * B2Q_FP4_ACT_MXFP8 quantizes the activations to one E4M3 code under an E8M0 scale per 32 values (the MX W4A8 recipe,
 * twice the rate): the result is that of the quantized activations -- no counterpart in the reference, whose
 * activations stay f32 (parity by composition: the same activation quantizer, then dequantize_fp4 and an f32 matmul).
 * b2q_gemm_fp4_wo takes this path (SPLIT) for E2M1 codes with E8M0 scales of block 32 and more than 32 tokens. */
typedef enum { B2Q_FP4_ACT_SPLIT = 0, B2Q_FP4_ACT_MXFP8 = 1 } b2q_fp4_act_mode;
int32_t b2q_gemm_fp4_blockscaled(b2q_handle h, const uint8_t* codes, const uint8_t* scales_e8m0, const void* x_bf16,
                                 int64_t tokens, int64_t N, int64_t K, int act_mode, void* out, int out_type);
/* grouped_gemm (crates/oxicuda-blas/src/batched/grouped_gemm.rs:46-78) for FP4 weights, table on the device, ONE launch:
 * problem g multiplies rows [row_offsets[g], row_offsets[g + 1]) of x_bf16 [capacity_rows x K] (offsets multiples of 256;
 * the last problem runs to capacity_rows) with weights [g * N, (g + 1) * N) of the stacked codes [groups * N x K / 2] and
 * scales [groups * N x K / 32]; out [capacity_rows x N].  Rows behind a problem's real row count are padding: they are
 * computed like any other and never read back by the caller. */
int32_t b2q_grouped_gemm_fp4_rows(b2q_handle h, const uint8_t* codes, const uint8_t* scales_e8m0, const void* x_bf16,
                                  const int32_t* row_offsets, int groups, int64_t capacity_rows, int64_t N, int64_t K,
                                  int act_mode, void* out, int out_type);

/* ---- GGML block codecs, the weight formats of GGUF files: crates/oxicuda-quant/src/scheme/ggml.rs
 *      quantize_q8_0 :243-262, quantize_q4_0 :284-316, quantize_q4_1 :342-372, quantize_q4_k :404-472, dequantize_* :265-506,
 *      GgmlType :147-185.  Blocks are packed little-endian records in the field order of the reference's structs:
 *      Q8_0 {d f16, qs i8[32]} 34 bytes; Q4_0 {d, qs u8[16]} 18 (byte i = code i | code i+16 << 4); Q4_1 {d, m, qs[16]} 20;
 *      Q4_K {d, dmin, scales u8[8], mins u8[8], qs u8[128]} 148 bytes for 256 weights (byte i = code 2i | code 2i+1 << 4).
 *      Bit-exact with the reference's arithmetic (binary16 scales rounded to nearest even).  Errors as check_block
 *      (:522-534): EMPTY_INPUT, GROUP_SIZE_MISMATCH. ---- */
typedef enum { B2Q_GGML_Q8_0 = 0, B2Q_GGML_Q4_0 = 1, B2Q_GGML_Q4_1 = 2, B2Q_GGML_Q4_K = 3 } b2q_ggml_type;
int64_t b2q_ggml_block_bytes(int type);   /* bytes of one record; -1 for an unknown type */
int64_t b2q_ggml_block_size(int type);    /* weights per record: 32, or 256 for Q4_K */
/* w [n] f32 -> blocks [n / block_size records]. */
int32_t b2q_ggml_quantize_f32(b2q_handle h, int type, const float* w, int64_t n, uint8_t* blocks);
/* blocks -> out [n] f32 or bf16 (B2Q_OUT_F32 / B2Q_OUT_BF16; bf16 is the f32 value rounded to nearest even). */
int32_t b2q_ggml_dequantize(b2q_handle h, int type, const uint8_t* blocks, int64_t n, void* out, int out_type);

/* ---- GPTQ / AWQ weight-only group quantization: crates/oxicuda-dnn/src/quantize/gptq_awq.rs.  The five kernels that
 *      WeightQuantPlan generates, each with the reference kernel's own arithmetic.  Layout (QuantizedWeight :210-232):
 *      codes packed 32 / bits to a u32 over the FLAT row-major matrix (element e in word e / epu at bits
 *      [(e % epu) * bits, +bits); epu = 16, 10, 8, 4 for bits = 2, 3, 4, 8), scales and zero points f32
 *      [rows x cols / group_size].  Validation as WeightQuantPlan::new (:254-283) and GptqConfig::validate (:102-127):
 *      INVALID_DIMENSION for an empty matrix, INVALID_ARGUMENT for bits outside {2, 3, 4, 8}, a zero group size or
 *      cols % group_size != 0. ---- */
/* quantized_weight_info().packed_weight_elements (:996-1027): ceil(rows * cols / epu); -1 for a bad argument. */
int64_t b2q_wq_packed_words(int64_t rows, int64_t cols, int bits);
/* dnn_gptq_quantize_f32 (:329-499), the reference's simplified quantizer (no inverse-Hessian update):
 * q = clamp(rni(w / max(hessian_diag[col], 1e-6)) (+ 2^(bits-1), floored at 0, when symmetric), 0, 2^bits - 1);
 * scales[row, group] = max(hessian_diag[last column of the group], 1e-6) / (2^bits - 1) (the value the reference's
 * column loop leaves there).  packed needs no clearing (the reference ORs into a zeroed buffer).  Bit-exact. */
int32_t b2q_gptq_quantize_f32(b2q_handle h, const float* weight, const float* hessian_diag, int64_t rows, int64_t cols,
                              int64_t group_size, int bits, int symmetric, uint32_t* packed, float* scales);
/* dnn_gptq_dequantize_f32 (:509-616): out[e] = q * scale (zeros == NULL: the symmetric kernel) or (q - zero) * scale;
 * out f32 or bf16 (the f32 value rounded to nearest even).  Bit-exact. */
int32_t b2q_wq_dequantize(b2q_handle h, const uint32_t* packed, const float* scales, const float* zeros, int64_t rows,
                          int64_t cols, int64_t group_size, int bits, void* out, int out_type);
/* dnn_awq_scale_search_f32 (:626-713): scale_out[c] = a * rsqrt.approx(a), a = max(|act_stats[c]|, 1e-7) (the
 * reference's stand-in for act^alpha: its alpha grid and weight operand are not read, best_alpha is not written). */
int32_t b2q_awq_scale_search_f32(b2q_handle h, const float* act_stats, int64_t num_channels, float* scale_out);
/* dnn_awq_quantize_f32 (:723-857): q = min(max(rni(w * channel_scales[col] / max(group_scales[row, group], 1e-12)), 0),
 * 2^bits - 1); group_scales is an INPUT; zeros (may be NULL: AwqConfig.zero_point = false) is filled with 0.0 as the
 * reference does.  bits 4 or 8 (AwqConfig::validate :174-199).  Bit-exact. */
int32_t b2q_awq_quantize_f32(b2q_handle h, const float* weight, const float* channel_scales, const float* group_scales,
                             int64_t rows, int64_t cols, int64_t group_size, int bits, uint32_t* packed, float* zeros);
/* dnn_fused_dequant_gemv_f32 (:867-986): y[row] = sum over col = 0 .. cols-1, in that order, of
 * fma(float(q) * scales[row, col / group_size], x[col], acc), f32.  The reference reads row r at word r * (cols / epu),
 * which agrees with the flat packing of the kernels above only when epu divides cols: that is required here
 * (INVALID_ARGUMENT otherwise).  zeros == NULL is the reference kernel (it ignores zero points); with zeros the term
 * is (float(q) - zero) * scale, as b2q_wq_dequantize has it.
 * split_k = 1: the reference's summation order, bit-exact.  2, 4, 8: the columns are cut into that many contiguous
 * segments, each summed in order by its own thread, the partial sums added in segment order (deterministic; differs
 * from split_k = 1 by rounding only) - more threads for matrices with few rows.  0: the library's choice. */
int32_t b2q_fused_dequant_gemv_f32(b2q_handle h, const uint32_t* packed, const float* scales, const float* zeros,
                                   const float* x, int64_t rows, int64_t cols, int64_t group_size, int bits, int split_k,
                                   float* y);

/* ---- tile heuristics: classify_workload / Fp8TileHeuristic::select crates/oxicuda-blas/src/precision/fp8_ops.rs:67-107,
 *      :239-304; select_fp4_tile fp4_fp6_ops.rs:996-1075; Int8GemmConfig::tile_config int_ops.rs:141-176 ---- */
typedef struct {
  uint32_t tile_m, tile_n, tile_k, warp_m, warp_n, stages, use_tensor_core, split_k;
} b2q_tile_config;  /* TileConfig, crates/oxicuda-blas/src/level3/gemm/dispatch.rs:57-107 */
/* 0 SmallSquare, 1 LargeSquare, 2 SkinnyM, 3 SkinnyN, 4 SkinnyK, 5 General */
int32_t b2q_classify_workload(uint32_t m, uint32_t n, uint32_t k);
/* The reference's Blackwell heuristic (what Fp8Config::tile_config(Sm100, ..) returns); dtype 0 fp8, 1 fp4, 2 int8. */
int32_t b2q_ref_tile_config(int dtype, uint32_t m, uint32_t n, uint32_t k, b2q_tile_config* out);
/* Fp8Config::compute_split_k (fp8_ops.rs:389-396) */
uint32_t b2q_fp8_compute_split_k(uint32_t m, uint32_t n, uint32_t k);
/* The static per-shape table this library actually dispatches with (replaces the autotuner role,
 * crates/oxicuda-autotune/src/dispatch.rs:36-196): the CTA tile, pipeline depth and kernel family chosen for
 * (dtype, m, n, k).  kernel_id: 0 simt, 1 tcgen05 128x256, 2 tcgen05 128x128, 3 warp gemv,
 * 4 tcgen05 two-CTA 256x256, 5 fp8 decode gemv (mma.sync), 6 fp8 few-token weight-stationary tcgen05,
 * 7 fp4 block-scaled tcgen05 gemv (E8M0 scales; f32 scales take 3). */
int32_t b2q_select_tile(int dtype, uint32_t m, uint32_t n, uint32_t k, b2q_tile_config* out, int* kernel_id);

#ifdef __cplusplus
}
#endif
#endif /* B2Q_H */
