"""ctypes binding of the tvk C-ABI (include/tvk.h).

This is the only place Python touches ``libtvk.so``. Loading fails loudly when the library has
not been built: there is no Python or CPU fallback behind any of these calls.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

_LIB_PATH = Path(__file__).resolve().parent / "lib" / "libtvk.so"
_lib = None

# enums (keep in step with include/tvk.h)
OK, ERR_INVALID, ERR_UNSUPPORTED, ERR_OOM, ERR_CUDA, ERR_TIMEOUT, ERR_BAD_FORK, ERR_NO_DEVICE = range(8)
F32, F16, BF16, I64, I32, U8, F64 = range(7)
ACT_NONE, ACT_RELU, ACT_GELU = range(3)
(U_NEG, U_EXP, U_LOG, U_SQRT, U_RSQRT, U_SIGMOID, U_RELU, U_GELU, U_TANH, U_ABS, U_SILU, U_RECIPROCAL, U_SQUARE,
 U_SIN, U_COS, U_GELU_TANH, U_FLOOR, U_CEIL, U_ROUND, U_TRUNC, U_SIGN, U_LOG2, U_LOG10, U_LOG1P, U_EXPM1, U_EXP2, U_TAN, U_SINH, U_COSH, U_ASIN, U_ACOS,
 U_ATAN, U_ERF, U_ERFC, U_HARDSIGMOID, U_HARDSWISH, U_MISH, U_LOGSIGMOID, U_ASINH, U_ACOSH, U_ATANH, U_ERFINV, U_LGAMMA, U_FRAC, U_SINC) = range(45)
(B_ADD, B_SUB, B_MUL, B_DIV, B_MAXIMUM, B_MINIMUM, B_POW, B_GELU_BACKWARD, B_THRESHOLD_BACKWARD, B_SILU_BACKWARD,
 B_SIGMOID_BACKWARD, B_TANH_BACKWARD, B_GELU_TANH_BACKWARD, B_ADD_RELU, B_FMOD, B_REMAINDER, B_ATAN2, B_FLOOR_DIVIDE, B_CLAMP, B_LEAKY_RELU, B_ELU,
 B_SOFTPLUS, B_LEAKY_RELU_BACKWARD, B_ELU_BACKWARD, B_HARDSWISH_BACKWARD, B_HARDSIGMOID_BACKWARD, B_MISH_BACKWARD, B_LOGSIGMOID_BACKWARD,
 B_SOFTPLUS_BACKWARD, B_HYPOT, B_COPYSIGN, B_LOGADDEXP, B_LOGADDEXP2, B_FMAX, B_FMIN, B_HEAVISIDE) = range(36)
(L_AND, L_OR, L_XOR, L_NOT) = range(4)
C_EQ, C_NE, C_LT, C_LE, C_GT, C_GE = range(6)
T_ADDCMUL, T_ADDCDIV, T_LERP, T_WHERE = range(4)
R_SUM, R_MEAN, R_AMAX, R_AMIN = range(4)
MAX_DIMS = 8


class TvkError(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(message or f"tvk error {code}")
        self.code = code


class DeviceProps(C.Structure):
    _fields_ = [("name", C.c_char * 256), ("total_memory", C.c_uint64), ("vendor_id", C.c_uint32),
                ("device_id", C.c_uint32), ("cc_major", C.c_int32), ("cc_minor", C.c_int32),
                ("driver_version", C.c_int32), ("runtime_version", C.c_int32), ("sm_count", C.c_int32),
                ("warp_size", C.c_int32), ("l2_bytes", C.c_int32), ("max_smem_per_block", C.c_int32)]


class MemStats(C.Structure):
    _fields_ = [(n, C.c_uint64) for n in (
        "allocated_bytes", "peak_allocated_bytes", "reserved_bytes", "cached_bytes", "total_allocated_bytes",
        "total_freed_bytes", "num_device_mallocs", "num_cache_hits", "num_oom_retries")]


class GemmDesc(C.Structure):
    _fields_ = [("dtype", C.c_int32), ("activation", C.c_int32),
                ("batch", C.c_int64), ("m", C.c_int64), ("n", C.c_int64), ("k", C.c_int64),
                ("a", C.c_void_p), ("a_rs", C.c_int64), ("a_cs", C.c_int64), ("a_bs", C.c_int64),
                ("b", C.c_void_p), ("b_rs", C.c_int64), ("b_cs", C.c_int64), ("b_bs", C.c_int64),
                ("c", C.c_void_p), ("c_rs", C.c_int64), ("c_bs", C.c_int64),
                ("bias", C.c_void_p), ("bias_rs", C.c_int64), ("bias_cs", C.c_int64), ("bias_bs", C.c_int64),
                ("alpha", C.c_float), ("beta", C.c_float), ("force_path", C.c_int32), ("c_f32", C.c_int32),
                ("n_peer_c", C.c_int32), ("reserved_", C.c_int32), ("peer_c", C.c_void_p * 7),
                ("c2", C.c_void_p), ("aux", C.c_void_p), ("aux_rs", C.c_int64), ("aux_bs", C.c_int64),
                ("aux_op", C.c_int32), ("reserved2_", C.c_int32)]


class ScaledMmDesc(C.Structure):
    _fields_ = [("a_kind", C.c_int32), ("b_kind", C.c_int32), ("out_kind", C.c_int32), ("bias_dtype", C.c_int32),
                ("m", C.c_int64), ("n", C.c_int64), ("k", C.c_int64),
                ("a", C.c_void_p), ("a_rs", C.c_int64), ("a_cs", C.c_int64),
                ("b", C.c_void_p), ("b_rs", C.c_int64), ("b_cs", C.c_int64),
                ("out", C.c_void_p),
                ("scale_a", C.c_void_p), ("sa_stride", C.c_int64),
                ("scale_b", C.c_void_p), ("sb_stride", C.c_int64),
                ("bias", C.c_void_p), ("scale_result", C.c_void_p)]


F8_E4M3, F8_E5M2 = 0, 1
SCALED_OUT_F32, SCALED_OUT_F16, SCALED_OUT_BF16, SCALED_OUT_E4M3, SCALED_OUT_E5M2 = range(5)
AUX_NONE, AUX_GELU_BACKWARD, AUX_RELU_BACKWARD = 0, 1, 2
SCAN_SUM, SCAN_PROD, SCAN_LOGADDEXP = 0, 1, 2


class MultiItem(C.Structure):
    _fields_ = [("ptr", C.c_void_p * 4), ("numel", C.c_int64), ("step", C.c_void_p)]


class IpcHandle(C.Structure):
    _fields_ = [("reserved", C.c_ubyte * 64), ("offset", C.c_uint64)]


class Conv2dDesc(C.Structure):
    _fields_ = [("dtype", C.c_int32)] + [(n, C.c_int64) for n in (
        "n", "cin", "h", "w", "cout", "kh", "kw", "stride_h", "stride_w", "pad_h", "pad_w", "dilation_h", "dilation_w", "groups", "layout")]


CONV_X_CHANNELS_LAST, CONV_Y_CHANNELS_LAST, CONV_W_CHANNELS_LAST = 1, 2, 4


class Pool2dDesc(C.Structure):
    _fields_ = [("dtype", C.c_int32)] + [(n, C.c_int64) for n in (
        "planes", "h", "w", "ho", "wo", "kh", "kw", "stride_h", "stride_w", "pad_h", "pad_w", "dilation_h", "dilation_w")] + [
        ("count_include_pad", C.c_int32), ("divisor_override", C.c_int64)]


class Iter(C.Structure):
    _fields_ = [("ndim", C.c_int32), ("noperands", C.c_int32), ("sizes", C.c_int64 * MAX_DIMS),
                ("strides", (C.c_int64 * MAX_DIMS) * 4)]


RAW_ALLOC_FN = C.CFUNCTYPE(C.c_int, C.POINTER(C.c_void_p), C.c_uint64)
RAW_FREE_FN = C.CFUNCTYPE(C.c_int, C.c_void_p)

_i, _i64, _u64, _p, _d = C.c_int, C.c_int64, C.c_uint64, C.c_void_p, C.c_double
_P = C.POINTER

# name -> (restype, argtypes); every symbol declared in include/tvk.h appears here.
SIGNATURES = {
    "tvk_last_error": (C.c_char_p, []),
    "tvk_version": (C.c_char_p, []),
    "tvk_device_count": (_i, [_P(_i)]),
    "tvk_is_initialized": (_i, []),
    "tvk_init": (_i, []),
    "tvk_is_in_bad_fork": (_i, []),
    "tvk_set_device": (_i, [_i]),
    "tvk_get_device": (_i, [_P(_i)]),
    "tvk_get_device_props": (_i, [_i, _P(DeviceProps)]),
    "tvk_get_stream": (_i, [_i, _P(_p)]),
    "tvk_synchronize": (_i, [_i]),
    "tvk_check_device_status": (_i, [_i]),
    "tvk_round_size": (_u64, [_u64]),
    "tvk_malloc": (_i, [_i, _u64, _P(_p)]),
    "tvk_free": (_i, [_i, _p]),
    "tvk_empty_cache": (_i, [_i]),
    "tvk_mem_info": (_i, [_i, _P(_u64), _P(_u64)]),
    "tvk_mem_get_stats": (_i, [_i, _P(MemStats)]),
    "tvk_mem_reset_peak": (_i, [_i]),
    "tvk_host_alloc": (_i, [_u64, _P(_p)]),
    "tvk_host_free": (_i, [_p]),
    "tvk_debug_set_raw_allocator": (_i, [_p, _p, _i]),
    "tvk_debug_bounded_wait": (_i, [_i, _i, _p]),
    "tvk_memcpy_h2d": (_i, [_i, _p, _p, _u64]),
    "tvk_memcpy_d2h": (_i, [_i, _p, _p, _u64]),
    "tvk_memcpy_d2d": (_i, [_i, _p, _p, _u64]),
    "tvk_memcpy_peer": (_i, [_i, _p, _i, _p, _u64]),
    "tvk_memcpy_async": (_i, [_p, _p, _u64, _p]),
    "tvk_pointer_device": (_i, [_p, _P(_i)]),
    "tvk_event_create": (_i, [_P(_p)]),
    "tvk_event_destroy": (_i, [_p]),
    "tvk_event_record": (_i, [_i, _p]),
    "tvk_event_synchronize": (_i, [_p]),
    "tvk_event_wait": (_i, [C.c_int, _p]),
    "tvk_event_query": (_i, [_p, _P(_i)]),
    "tvk_event_elapsed_ms": (_i, [_p, _p, _P(C.c_float)]),
    "tvk_graph_begin_capture": (_i, [_i]),
    "tvk_graph_end_capture": (_i, [_i, _P(_p)]),
    "tvk_graph_launch": (_i, [_i, _p]),
    "tvk_graph_destroy": (_i, [_p]),
    "tvk_rng_set_seed": (_i, [_i, _u64]),
    "tvk_rng_get_state": (_i, [_i, _P(_u64), _P(_u64)]),
    "tvk_rng_set_state": (_i, [_i, _u64, _u64]),
    "tvk_rng_reserve": (_i, [_i, _u64, _P(_u64), _P(_u64)]),
    "tvk_max_pool2d_forward": (_i, [_p, _p, _p, _p, _p]),
    "tvk_max_pool2d_backward": (_i, [_p, _p, _p, _p, _p]),
    "tvk_avg_pool2d_forward": (_i, [_p, _p, _p, _p]),
    "tvk_avg_pool2d_backward": (_i, [_p, _p, _p, _p]),
    "tvk_random_fill": (_i, [_i, _i, _p, _i64, _d, _d, _u64, _u64, _p, _p]),
    "tvk_dropout": (_i, [_i, _p, _p, _p, _i64, _d, _u64, _u64, _p, _p]),
    "tvk_rng_reserve_state": (_i, [_i, _u64, _P(_u64), _P(_u64), _P(_p)]),
    "tvk_gemm_workspace_size": (_i, [_P(GemmDesc), _P(_u64)]),
    "tvk_gemm_splits": (_i, [_P(GemmDesc), _P(C.c_int)]),
    "tvk_gemm": (_i, [_P(GemmDesc), _p, _u64, _p]),
    "tvk_gemm_path": (_i, [_P(GemmDesc), _P(_i)]),
    "tvk_debug_gemm_tuning": (_i, [_i, _i, _i, _i, _i]),
    "tvk_unary": (_i, [_i, _i, _p, _p, _i64, _p]),
    "tvk_binary": (_i, [_i, _i, _p, _p, _p, _d, _d, _i64, _p]),
    "tvk_compare": (_i, [_i, _i, _p, _p, _p, _d, _i64, _p]),
    "tvk_logical": (_i, [_i, _p, _p, _p, _i64, _p]),
    "tvk_ternary": (_i, [_i, _i, _p, _p, _p, _p, _d, _i64, _p]),
    "tvk_unary_strided": (_i, [_i, _i, _p, _p, _P(Iter), _p]),
    "tvk_binary_strided": (_i, [_i, _i, _p, _p, _p, _d, _P(Iter), _p]),
    "tvk_compare_strided": (_i, [_i, _i, _p, _p, _p, _P(Iter), _p]),
    "tvk_ternary_strided": (_i, [_i, _i, _p, _p, _p, _p, _d, _P(Iter), _p]),
    "tvk_fill": (_i, [_i, _p, _d, _i64, _p]),
    "tvk_cast": (_i, [_i, _p, _i, _p, _i64, _p]),
    "tvk_copy_strided": (_i, [_i, _p, _i, _p, _P(Iter), _p]),
    "tvk_reduce_workspace_size": (_i, [_i64, _i64, _i64, _P(_u64)]),
    "tvk_reduce": (_i, [_i, _i, _i, _p, _p, _i64, _i64, _i64, _p, _u64, _p]),
    "tvk_reduce_noalloc": (_i, [_i, _i, _i, _p, _p, _i64, _i64, _i64, _p]),
    "tvk_argreduce": (_i, [_i, _i, _p, _p, _i64, _i64, _i64, _p, _u64, _p]),
    "tvk_softmax_forward": (_i, [_i, _i, _i, _p, _p, _i64, _i64, _p]),
    "tvk_softmax_backward": (_i, [_i, _i, _p, _p, _p, _i64, _i64, _p]),
    "tvk_nll_loss_forward": (_i, [_i, _p, _p, _p, _p, _p, _i64, _i64, _i, _i64, _p]),
    "tvk_nll_loss_backward": (_i, [_i, _p, _p, _p, _p, _p, _i64, _i64, _i, _i64, _p]),
    "tvk_rmsnorm_forward": (_i, [_i, _p, _p, _p, _p, _i64, _i64, _d, _p]),
    "tvk_rmsnorm_backward_workspace_size": (_i, [_i64, _i64, _P(_u64)]),
    "tvk_rmsnorm_backward": (_i, [_i, _p, _p, _p, _p, _p, _p, _i64, _i64, _p, _u64, _p]),
    "tvk_layernorm_forward": (_i, [_i, _p, _p, _p, _p, _p, _p, _i64, _i64, _d, _p]),
    "tvk_layernorm_backward_workspace_size": (_i, [_i64, _i64, _P(_u64)]),
    "tvk_layernorm_backward": (_i, [_i, _p, _p, _p, _p, _p, _p, _p, _p, _i64, _i64, _p, _u64, _p]),
    "tvk_groupnorm_forward": (_i, [_i, _p, _p, _p, _p, _p, _p, _i64, _i64, _i64, _i64, _d, _p]),
    "tvk_groupnorm_backward": (_i, [_i, _p, _p, _p, _p, _p, _p, _p, _p, _i64, _i64, _i64, _i64, _p]),
    "tvk_cross_entropy_workspace_size": (_i, [_i64, _P(_u64)]),
    "tvk_cross_entropy_forward": (_i, [_i, _p, _p, _p, _p, _p, _p, _i64, _i64, _i, _i64, _p, _u64, _p]),
    "tvk_cross_entropy_backward": (_i, [_i, _p, _p, _p, _p, _p, _p, _p, _i64, _i64, _i, _i64, _p]),
    "tvk_scan": (_i, [_i, _i, _p, _p, _i64, _i64, _i64, _p]),
    "tvk_embedding_forward": (_i, [_i, _p, _p, _p, _i64, _i64, _i64, _p]),
    "tvk_embedding_backward": (_i, [_i, _p, _p, _p, _i64, _i64, _i64, _i64, _p]),
    "tvk_batchnorm_workspace_size": (_i, [_i64, _i64, _i64, _P(_u64)]),
    "tvk_batchnorm_forward": (_i, [_i, _p, _p, _p, _p, _p, _p, _i, _p, _p, _i64, _i64, _i64, _d, _d, _p, _u64, _p]),
    "tvk_batchnorm_backward": (_i, [_i, _p, _p, _p, _p, _p, _p, _p, _p, _i64, _i64, _i64, _p, _u64, _p]),
    "tvk_batchnorm_cl_workspace_size": (_i, [_i64, _i64, _P(_u64)]),
    "tvk_batchnorm_inference": (_i, [_i, _p, _p, _p, _p, _i, _p, _p, _i64, _i64, _i64, _i, _d, _p]),
    "tvk_batchnorm_forward_cl": (_i, [_i, _p, _p, _p, _p, _p, _p, _i, _p, _p, _i64, _i64, _d, _d, _p, _u64, _p]),
    "tvk_batchnorm_backward_cl": (_i, [_i, _p, _p, _p, _p, _p, _p, _p, _p, _i64, _i64, _p, _u64, _p]),
    "tvk_ipc_export": (_i, [_p, _P(IpcHandle)]),
    "tvk_ipc_open": (_i, [_P(IpcHandle), _P(_p)]),
    "tvk_ipc_close": (_i, [_p]),
    "tvk_conv2d_workspace_size": (_i, [_P(Conv2dDesc), _i, _P(_u64)]),
    "tvk_conv2d_forward": (_i, [_P(Conv2dDesc), _p, _p, _p, _p, _u64, _p]),
    "tvk_conv2d_backward_input": (_i, [_P(Conv2dDesc), _p, _p, _p, _p, _u64, _p]),
    "tvk_conv2d_backward_weight": (_i, [_P(Conv2dDesc), _p, _p, _p, _p, _u64, _p]),
    "tvk_conv2d_backward": (_i, [_P(Conv2dDesc), _p, _p, _p, _p, _p, _p, _u64, _p]),
    "tvk_scaled_mm_workspace_size": (_i, [_P(ScaledMmDesc), _P(_u64)]),
    "tvk_scaled_mm": (_i, [_P(ScaledMmDesc), _p, _u64, _p]),
    "tvk_depthwise_conv2d_forward": (_i, [_P(Conv2dDesc), _p, _p, _p, _p]),
    "tvk_depthwise_conv2d_backward_input": (_i, [_P(Conv2dDesc), _p, _p, _p, _p]),
    "tvk_depthwise_conv2d_backward_weight": (_i, [_P(Conv2dDesc), _p, _p, _p, _p]),
    "tvk_attention_workspace_size": (_i, [_i, _i64, _i64, _i64, _i64, _i64, _i64, _i, _P(_u64)]),
    "tvk_attention_forward": (_i, [_i, _p, _p, _p, _p, _p, _i64, _i64, _i64, _i64, _i64, _i64, _d, _i, _p, _u64, _p]),
    "tvk_attention_backward": (_i, [_i, _p, _p, _p, _p, _p, _p, _p, _p, _p, _i64, _i64, _i64, _i64, _i64, _i64, _d, _i, _p, _u64, _p]),
    "tvk_sort_workspace_size": (_i, [_i, _i64, _i64, _P(_u64)]),
    "tvk_topk": (_i, [_i, _p, _p, _p, _i64, _i64, _i64, _i, _p, _u64, _p]),
    "tvk_adam_step": (_i, [_i, _p, _p, _p, _p, _i64, _d, _d, _d, _d, _d, _i64, _i, _i, _p]),
    "tvk_sgd_step": (_i, [_i, _p, _p, _p, _i64, _d, _d, _d, _d, _i, _i, _i, _p]),
    "tvk_adam_step_multi": (_i, [_i, _P(MultiItem), _i, _d, _d, _d, _d, _d, _i64, _i, _i, _p]),
    "tvk_sgd_step_multi": (_i, [_i, _P(MultiItem), _i, _d, _d, _d, _d, _i, _i, _i, _p]),
    "tvk_foreach_axpby": (_i, [_i, _P(MultiItem), _i, _d, _d, _d, _i, _p]),
}


def library_path() -> Path:
    return _LIB_PATH


def lib() -> C.CDLL:
    """Loads libtvk.so once. Raises ImportError when it has not been built."""
    global _lib
    if _lib is None:
        if not _LIB_PATH.exists():
            raise ImportError(
                f"{_LIB_PATH} is missing: build it with `python -m torchvulkan_b200.build` "
                "(nvcc, sm_100a). There is no fallback implementation.")
        handle = C.CDLL(str(_LIB_PATH))
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)  # AttributeError here means the header and the library disagree
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


def last_error() -> str:
    return lib().tvk_last_error().decode("utf-8", "replace")


def check(rc: int) -> None:
    if rc != OK:
        raise TvkError(rc, last_error())


def call(name: str, *args) -> None:
    """Calls an int-returning entry point and raises TvkError on a non-zero status."""
    check(getattr(lib(), name)(*args))
