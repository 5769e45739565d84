"""ctypes binding of libb2q.so — the C ABI declared in include/b2q.h.

The library is the product; this module only loads it and maps status codes to
exceptions named after the reference's error variants
(crates/oxicuda-blas/src/error.rs:17-60, crates/oxicuda-quant/src/error.rs:10-58).
There is no fallback: if the shared library is missing, importing a symbol fails
loudly, and without a CUDA device `Handle()` raises.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

_PKG = Path(__file__).resolve().parent
LIB_PATH = _PKG / "libb2q.so"

# status codes (include/b2q.h)
OK = 0
ERR_CUDA, ERR_INVALID_DIMENSION, ERR_BUFFER_TOO_SMALL, ERR_DIMENSION_MISMATCH = 1, 2, 3, 4
ERR_UNSUPPORTED, ERR_LAUNCH_FAILED, ERR_INVALID_ARGUMENT = 5, 7, 8
ERR_EMPTY_INPUT, ERR_GROUP_SIZE_MISMATCH, ERR_INVALID_SCALE, ERR_NON_FINITE_FP8, ERR_INVALID_CONFIG = 20, 21, 22, 23, 24
ERR_INVALID_BIT_WIDTH = 25
ERR_TIMEOUT = 40
ERR_NCCL = 41

FP8_E4M3, FP8_E5M2 = 0, 1
ROUND_REF, ROUND_RNE = 0, 1
FP4_E2M1, FP4_INT4 = 0, 1
SCALE_F32, SCALE_E8M0 = 0, 1
SYMMETRIC, ASYMMETRIC = 0, 1
OUT_BF16, OUT_F32 = 0, 1
GATE_UP_CONCATENATED, GATE_UP_INTERLEAVED128 = 0, 1
SCALE_SCALAR, SCALE_PER_ROW = 0, 1


class B2qError(RuntimeError):
    """Base of every error raised for a non-zero b2q status."""
    status = -1

    def __init__(self, status: int, message: str):
        super().__init__(f"[b2q status {status}] {message}")
        self.status = status
        self.message = message


class CudaError(B2qError): pass
class InvalidDimension(B2qError): pass
class BufferTooSmall(B2qError): pass
class DimensionMismatch(B2qError): pass
class UnsupportedOperation(B2qError): pass
class LaunchFailed(B2qError): pass
class InvalidArgument(B2qError): pass
class EmptyInput(B2qError): pass
class GroupSizeMismatch(B2qError): pass
class InvalidScale(B2qError): pass
class NonFiniteFp8(B2qError): pass
class InvalidConfig(B2qError): pass
class InvalidBitWidth(B2qError): pass
class DeviceTimeout(B2qError): pass
class CollectiveError(B2qError): pass


_ERRORS = {
    ERR_CUDA: CudaError, ERR_INVALID_DIMENSION: InvalidDimension, ERR_BUFFER_TOO_SMALL: BufferTooSmall,
    ERR_DIMENSION_MISMATCH: DimensionMismatch, ERR_UNSUPPORTED: UnsupportedOperation, ERR_LAUNCH_FAILED: LaunchFailed,
    ERR_INVALID_ARGUMENT: InvalidArgument, ERR_EMPTY_INPUT: EmptyInput, ERR_GROUP_SIZE_MISMATCH: GroupSizeMismatch,
    ERR_INVALID_SCALE: InvalidScale, ERR_NON_FINITE_FP8: NonFiniteFp8, ERR_INVALID_CONFIG: InvalidConfig,
    ERR_INVALID_BIT_WIDTH: InvalidBitWidth, ERR_TIMEOUT: DeviceTimeout, ERR_NCCL: CollectiveError,
}


class GemmFp8Problem(C.Structure):
    """b2q_gemm_fp8_problem (include/b2q.h): one entry of a grouped-GEMM problem table."""
    _fields_ = [("a", C.c_void_p), ("w", C.c_void_p), ("m", C.c_int64), ("n", C.c_int64), ("k", C.c_int64),
                ("scale_a", C.c_void_p), ("scale_a_kind", C.c_int32), ("scale_w", C.c_void_p), ("scale_w_kind", C.c_int32),
                ("out", C.c_void_p)]


class GemmFp8Desc(C.Structure):
    """b2q_gemm_fp8_desc (include/b2q.h): operands, scales and the epilogue of b2q_gemm_fp8_ex."""
    _fields_ = [("a", C.c_void_p), ("w", C.c_void_p), ("m", C.c_int64), ("n", C.c_int64), ("k", C.c_int64), ("fmt", C.c_int32),
                ("scale_a", C.c_void_p), ("scale_a_kind", C.c_int32), ("scale_w", C.c_void_p), ("scale_w_kind", C.c_int32),
                ("out", C.c_void_p), ("out_type", C.c_int32), ("alpha", C.c_float), ("beta", C.c_float), ("bias", C.c_void_p),
                ("epilogue", C.c_int32), ("w_layout", C.c_int32)]


class TileConfig(C.Structure):
    """TileConfig, crates/oxicuda-blas/src/level3/gemm/dispatch.rs:57-107."""
    _fields_ = [(n, C.c_uint32) for n in
                ("tile_m", "tile_n", "tile_k", "warp_m", "warp_n", "stages", "use_tensor_core", "split_k")]

    def as_tuple(self):
        return tuple(getattr(self, n) for n, _ in self._fields_)


_H = C.c_void_p
_P = C.c_void_p
_I64 = C.c_int64
_I = C.c_int
_F = C.c_float
_U32 = C.c_uint32

# name -> (restype, argtypes); must list every symbol include/b2q.h declares
SIGNATURES = {
    "b2q_create": (C.c_int32, [C.POINTER(_H), _I]),
    "b2q_destroy": (C.c_int32, [_H]),
    "b2q_set_stream": (C.c_int32, [_H, _P]),
    "b2q_set_static_weights": (C.c_int32, [_H, C.c_int]),
    "b2q_get_sm": (C.c_int32, [_H, C.POINTER(_I)]),
    "b2q_get_sm_count": (C.c_int32, [_H, C.POINTER(_I)]),
    "b2q_last_error": (C.c_char_p, [_H]),
    "b2q_check": (C.c_int32, [_H]),
    "b2q_minmax_calibrate_f32": (C.c_int32, [_H, _P, _I64, _I64, _I, _I, _P, _P]),
    "b2q_minmax_quantize_f32": (C.c_int32, [_H, _P, _I64, _I64, _P, _P, _I, _I, _P]),
    "b2q_minmax_dequantize_f32": (C.c_int32, [_H, _P, _I64, _I64, _P, _P, _P]),
    "b2q_fake_quant_inplace_f32": (C.c_int32, [_H, _P, _I64, _F, _F, _F, _F]),
    "b2q_fp8_encode_f32": (C.c_int32, [_H, _P, _I64, _I, _I, _P]),
    "b2q_fp8_decode_f32": (C.c_int32, [_H, _P, _I64, _I, _I, _P]),
    "b2q_fp8_remap_ref_subnormals": (C.c_int32, [_H, _P, _I64, _I]),
    "b2q_fp8_quantize_rows_f32": (C.c_int32, [_H, _P, _I64, _I64, _I, _I, _P, _P]),
    "b2q_fp8_quantize_rows_bf16": (C.c_int32, [_H, _P, _I64, _I64, _I, _I, _P, _P]),
    "b2q_swiglu_quantize_rows_bf16": (C.c_int32, [_H, _P, _P, _I64, _I64, _I64, _I, _I, _P, _P]),
    "b2q_rms_norm_quantize_fp8_bf16": (C.c_int32, [_H, _P, _P, _P, _I64, _I64, _F, _I, _I, _P, _P, _P]),
    "b2q_kv_cache_quantize_f32": (C.c_int32, [_H, _P, _I64, _I64, _I, _I, _P, _P, _P]),
    "b2q_kv_cache_quantize_bf16": (C.c_int32, [_H, _P, _I64, _I64, _I, _I, _P, _P, _P]),
    "b2q_kv_cache_dequantize_f32": (C.c_int32, [_H, _P, _I64, _I64, _I, _P, _P, _P]),
    "b2q_kv_cache_dequantize_bf16": (C.c_int32, [_H, _P, _I64, _I64, _I, _P, _P, _P]),
    "b2q_kv_quantize_tokens_f32": (C.c_int32, [_H, _P, _I64, _I64, _I, _I, _P, _P, _P]),
    "b2q_kv_quantize_tokens_bf16": (C.c_int32, [_H, _P, _I64, _I64, _I, _I, _P, _P, _P]),
    "b2q_kv_dequantize_tokens_f32": (C.c_int32, [_H, _P, _I64, _I64, _I, _P, _P, _P]),
    "b2q_kv_dequantize_tokens_bf16": (C.c_int32, [_H, _P, _I64, _I64, _I, _P, _P, _P]),
    "b2q_dnn_quantize_to_fp8_f32": (C.c_int32, [_H, _P, _I64, _P, _P]),
    "b2q_dnn_dequantize_from_fp8_f32": (C.c_int32, [_H, _P, _P, _I64, _P]),
    "b2q_dnn_quantize_to_int8_f32": (C.c_int32, [_H, _P, _I64, _P, _P]),
    "b2q_dnn_dequantize_from_int8_f32": (C.c_int32, [_H, _P, _P, _I64, _P]),
    "b2q_dnn_quantize_block_scaled_f32": (C.c_int32, [_H, _P, _I64, _U32, _P, _P]),
    "b2q_block_int8_quantize_f32": (C.c_int32, [_H, _P, _I64, _I64, _P, _P]),
    "b2q_block_int8_dequantize_f32": (C.c_int32, [_H, _P, _P, _I64, _I64, _P]),
    "b2q_block_absmax_scale_f32": (C.c_int32, [_H, _P, _I64, _I64, _F, _P]),
    "b2q_pack_int4": (C.c_int32, [_H, _P, _I64, _P]),
    "b2q_unpack_int4": (C.c_int32, [_H, _P, _I64, _P]),
    "b2q_gemm_int4_f32": (C.c_int32, [_H, _P, _P, _P, _P, _I64, _I64, _I64, _I64]),
    "b2q_gemv_int4_wo": (C.c_int32, [_H, _P, _P, _I64, _P, _I64, _I64, _I64, _P, _I]),
    "b2q_fp8_quantize_rows_f32_noalloc": (C.c_int32, [_P, _I64, _I64, _I, _I, _P, _P, _P, _P, C.c_char_p, C.c_size_t]),
    "b2q_fp4_block_quantize_f32": (C.c_int32, [_H, _P, _I64, _I, _I, _I, _P, _P]),
    "b2q_fp4_block_dequantize_f32": (C.c_int32, [_H, _P, _I64, _I, _I, _I, _P, _P]),
    "b2q_nf4_decode_f32": (C.c_int32, [_H, _P, _I64, _I, _P, _P]),
    "b2q_nf4_encode_f32": (C.c_int32, [_H, _P, _I64, _I, _P, _P]),
    "b2q_int8_quant_f32": (C.c_int32, [_H, _P, _I64, _F, _P]),
    "b2q_int8_dequant_f32": (C.c_int32, [_H, _P, _I64, _F, _P]),
    "b2q_distfp8_quantize_block_f32": (C.c_int32, [_H, _P, _I64, _I64, _P, _P]),
    "b2q_distfp8_dequantize_block_f32": (C.c_int32, [_H, _P, _I64, _I64, _P, _P]),
    "b2q_llm_int8_linear_f32": (C.c_int32, [_H, _P, _P, _I64, _I64, _I64, _F, _I, _P, _P, _P, _P, _P, _P, _P]),
    "b2q_gemm_i8": (C.c_int32, [_H, _P, _P, _I64, _I64, _I64, _P, _P, _P, _P]),
    "b2q_gemm_fp8": (C.c_int32, [_H, _P, _P, _I64, _I64, _I64, _I, _P, _I, _P, _I, _P, _I]),
    "b2q_gemm_fp8_ex": (C.c_int32, [_H, _P]),
    "b2q_gemm_fp8_simt": (C.c_int32, [_H, _P, _P, _I64, _I64, _I64, _I, _I, _P, _I, _P, _I, _P, _I]),
    "b2q_grouped_gemm_fp8": (C.c_int32, [_H, _P, _I, _I, _I]),
    "b2q_grouped_gemm_fp8_rows": (C.c_int32, [_H, _P, _P, _P, _P, _P, _P, _I, _I64, _I64, _I64, _I, _P, _I]),
    "b2q_moe_route_topk": (C.c_int32, [_H, _P, _I64, _I, _I, _P, _P]),
    "b2q_moe_assign_slots": (C.c_int32, [_H, _P, _I64, _I, _I, _P, _P, _P]),
    "b2q_moe_scatter": (C.c_int32, [_H, _P, _P, _I64, _I, _I64, _P]),
    "b2q_moe_forward": (C.c_int32, [_P, _P, _P, _P, _P, _P, _P, _I64, _I64, _I64, _I, _I, _I, _P, _P]),
    "b2q_gemm_fp8_scatter": (C.c_int32, [_H, _P, _P, _I64, _I64, _I64, _I, _P, _P, _P, _P, _I, _I]),
    "b2q_ggml_block_bytes": (C.c_int64, [_I]),
    "b2q_ggml_block_size": (C.c_int64, [_I]),
    "b2q_ggml_quantize_f32": (C.c_int32, [_H, _I, _P, _I64, _P]),
    "b2q_ggml_dequantize": (C.c_int32, [_H, _I, _P, _I64, _P, _I]),
    "b2q_wq_packed_words": (C.c_int64, [_I64, _I64, _I]),
    "b2q_gptq_quantize_f32": (C.c_int32, [_H, _P, _P, _I64, _I64, _I64, _I, _I, _P, _P]),
    "b2q_wq_dequantize": (C.c_int32, [_H, _P, _P, _P, _I64, _I64, _I64, _I, _P, _I]),
    "b2q_awq_scale_search_f32": (C.c_int32, [_H, _P, _I64, _P]),
    "b2q_awq_quantize_f32": (C.c_int32, [_H, _P, _P, _P, _I64, _I64, _I64, _I, _P, _P]),
    "b2q_fused_dequant_gemv_f32": (C.c_int32, [_H, _P, _P, _P, _P, _I64, _I64, _I64, _I, _I, _P]),
    "b2q_moe_forward_fp4": (C.c_int32, [_P, _P, _P, _P, _P, _P, _P, _I64, _I64, _I64, _I, _I, _I, _P, _P]),
    "b2q_grouped_gemm_fp4_rows": (C.c_int32, [_H, _P, _P, _P, _P, _I, _I64, _I64, _I64, _I, _P, _I]),
    "b2q_moe_forward_ex": (C.c_int32, [_P, _P, _P, _P, _P, _P, _P, _I64, _I64, _I64, _I, _I, _I, _I, _P, _P]),
    "b2q_ep_token_scatter": (C.c_int32, [_H, _P, _P, _P, _I64, _I64, _P]),
    "b2q_ep_token_gather_bf16": (C.c_int32, [_H, _P, _P, _P, _I64, _I, _I64, _P]),
    "b2q_gemv_fp4_wo": (C.c_int32, [_H, _P, _P, _I, _I, _P, _I64, _I64, _I64, _P, _I]),
    "b2q_gemm_fp4_wo": (C.c_int32, [_H, _P, _P, _I, _I, _I, _P, _I64, _I64, _I64, _P, _I]),
    "b2q_tp_unique_id": (C.c_int32, [_P]),
    "b2q_tp_comm_init": (C.c_int32, [_P, _I, _I, C.POINTER(_P)]),
    "b2q_tp_comm_destroy": (C.c_int32, [_P]),
    "b2q_tp_create": (C.c_int32, [_H, _P, _I, _I, C.POINTER(_P)]),
    "b2q_tp_destroy": (C.c_int32, [_P]),
    "b2q_tp_exchange_buffer": (C.c_int32, [_P, C.POINTER(_P), _P]),
    "b2q_tp_attach_peers": (C.c_int32, [_P, _P, _P]),
    "b2q_tp_set_chunks": (C.c_int32, [_P, _I]),
    "b2q_tp_plan": (C.c_int32, [_I, _I, _I64, _I64, C.POINTER(_I), C.POINTER(_I)]),
    "b2q_tp_all_reduce_f32_to_bf16": (C.c_int32, [_P, _P, _I64, _P]),
    "b2q_tp_all_reduce_bf16": (C.c_int32, [_P, _P, _I64]),
    "b2q_column_linear_forward": (C.c_int32, [_P, _P, _P, _P, _P, _P, _I64, _I64, _I64, _P, _P]),
    "b2q_row_linear_forward_allreduce": (C.c_int32, [_P, _P, _P, _P, _P, _P, _I64, _I64, _I64, _P]),
    "b2q_mlp_swiglu_fp8_forward": (C.c_int32, [_P, _P, _P, _P, _P, _P, _I64, _I64, _I64, _I, _P]),
    "b2q_mlp_swiglu_fp8_forward_ex": (C.c_int32, [_P, _P, _P, _P, _P, _P, _I64, _I64, _I64, _I, _I, _P]),
    "b2q_interleave_rows128": (C.c_int32, [_H, _P, _P, _I64, _I64, _P]),
    "b2q_gemm_fp4_blockscaled": (C.c_int32, [_H, _P, _P, _P, _I64, _I64, _I64, _I, _P, _I]),
    "b2q_classify_workload": (C.c_int32, [_U32, _U32, _U32]),
    "b2q_ref_tile_config": (C.c_int32, [_I, _U32, _U32, _U32, C.POINTER(TileConfig)]),
    "b2q_fp8_compute_split_k": (_U32, [_U32, _U32, _U32]),
    "b2q_select_tile": (C.c_int32, [_I, _U32, _U32, _U32, C.POINTER(TileConfig), C.POINTER(_I)]),
}

_lib = None


def lib() -> C.CDLL:
    """The loaded shared library; raises if it has not been built."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python -m oxicuda_b200._build` "
                "(there is no CPU or PyTorch fallback for the CUDA kernels)")
        L = C.CDLL(str(LIB_PATH))
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(L, name)           # AttributeError if the library lacks a declared symbol
            fn.restype = res
            fn.argtypes = args
        _lib = L
    return _lib


def ptr(t) -> C.c_void_p:
    """Device (or host) address of a torch tensor / numpy array / None."""
    if t is None:
        return C.c_void_p(0)
    if hasattr(t, "data_ptr"):
        return C.c_void_p(t.data_ptr())
    return C.c_void_p(t.ctypes.data)


class Handle:
    """BlasHandle equivalent (crates/oxicuda-blas/src/handle.rs:43-264): one per host thread."""

    def __init__(self, device: int = 0):
        self._h = _H()
        st = lib().b2q_create(C.byref(self._h), device)
        if st != OK:
            raise _ERRORS.get(st, B2qError)(st, "b2q_create failed (no CUDA device, or not an sm_100 GPU)")
        self.device = device

    def close(self):
        if getattr(self, "_h", None):
            lib().b2q_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def call(self, name: str, *args):
        st = getattr(lib(), name)(self._h, *args)
        if st != OK:
            msg = lib().b2q_last_error(self._h)
            raise _ERRORS.get(st, B2qError)(st, msg.decode() if msg else name)

    def set_stream(self, stream_ptr: int):
        self.call("b2q_set_stream", C.c_void_p(stream_ptr))

    def set_static_weights(self, static_weights: bool):
        """False: weight operands may be produced by the kernel right before a call (see include/b2q.h)."""
        self.call("b2q_set_static_weights", 1 if static_weights else 0)

    def sm_version(self) -> int:
        v = _I()
        self.call("b2q_get_sm", C.byref(v))
        return v.value

    def sm_count(self) -> int:
        v = _I()
        self.call("b2q_get_sm_count", C.byref(v))
        return v.value

    def check(self):
        """Synchronise and raise what the kernels recorded on the device (NonFiniteFp8, InvalidScale, timeout)."""
        self.call("b2q_check")


_default = {}


def reset_default_handles():
    """Drops the cached per-device handles: the next default_handle() creates a new one, which re-reads the B2Q_*
    experiment switches from the environment (a handle reads them once, when it is created)."""
    import torch
    if torch.cuda.is_available():
        torch.cuda.synchronize()
    for h in _default.values():
        h.close()
    _default.clear()


def default_handle(device: int | None = None) -> Handle:
    import torch
    if device is None:
        device = torch.cuda.current_device()
    h = _default.get(device)
    if h is None:
        h = _default[device] = Handle(device)
    h.set_stream(torch.cuda.current_stream(device).cuda_stream)
    return h
