"""ctypes binding of libtmq_b200.so: the only bridge between Python and the CUDA kernels.

The library is required.  There is no CPU or PyTorch fallback: if the shared object is missing or a call
returns an error status, the caller gets an exception.
"""
import ctypes
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "_build", "libtmq_b200.so")

_lib = None

c_int, c_size_t, c_double, c_float, c_void_p, c_int64 = (ctypes.c_int, ctypes.c_size_t, ctypes.c_double, ctypes.c_float,
                                                         ctypes.c_void_p, ctypes.c_int64)


class MtTensor(ctypes.Structure):
    _fields_ = [("w", c_void_p), ("out", c_void_p), ("n", ctypes.c_uint64), ("out_offset", ctypes.c_uint64)]


_SIGNATURES = {
    "tmq_status_string": (ctypes.c_char_p, [c_int]),
    "tmq_last_cuda_error": (c_int, []),
    "tmq_abi_version": (c_int, []),
    "tmq_softstep_fwd": (c_int, [c_void_p, c_void_p, c_size_t, c_double, c_void_p]),
    "tmq_softstep_bwd": (c_int, [c_void_p, c_void_p, c_void_p, c_size_t, c_double, c_double, c_void_p]),
    "tmq_softstep_deriv_fwd": (c_int, [c_void_p, c_void_p, c_size_t, c_double, c_double, c_void_p]),
    "tmq_softstep_deriv_bwd": (c_int, [c_void_p, c_void_p, c_void_p, c_size_t, c_double, c_double, c_void_p]),
    "tmq_clamp": (c_int, [c_void_p, c_void_p, c_size_t, c_float, c_float, c_void_p]),
    "tmq_reduce_scratch_bytes": (c_size_t, []),
    "tmq_qloss_sum": (c_int, [c_void_p, c_size_t, c_double, c_double, c_void_p, c_void_p, c_size_t, c_void_p]),
    "tmq_qloss_sum_noalloc": (c_int, [c_void_p, c_size_t, c_double, c_double, c_void_p, c_void_p]),
    "tmq_softstep_fused_step": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_size_t, c_double,
                                        c_double, c_double, c_double, c_float, c_float, c_float, c_void_p, c_size_t,
                                        c_void_p]),
    "tmq_mt_plan_bytes": (c_size_t, [ctypes.POINTER(MtTensor), c_int]),
    "tmq_mt_plan_build": (c_int, [ctypes.POINTER(MtTensor), c_int, c_void_p, c_size_t, ctypes.POINTER(c_int)]),
    "tmq_mt_qloss": (c_int, [c_void_p, c_int, c_int, c_double, c_double, c_void_p, c_void_p, c_size_t, c_void_p]),
    "tmq_mt_qloss_bwd": (c_int, [c_void_p, c_int, c_int, c_double, c_double, c_void_p, c_void_p, c_void_p]),
    "tmq_mt_adam_clamp": (c_int, [c_void_p, c_int, c_int, c_void_p, c_void_p, c_double, c_double, c_double, c_double,
                                  ctypes.c_longlong, c_int, c_float, c_float, c_void_p]),
    "tmq_mt_clamp": (c_int, [c_void_p, c_int, c_int, c_float, c_float, c_void_p]),
    "tmq_selftest_wait_timeout": (c_int, [ctypes.c_longlong, c_void_p, c_void_p, c_void_p]),
    "tmq_selftest_div": (c_int, [ctypes.c_uint, ctypes.c_uint64, ctypes.c_uint64, c_void_p, c_void_p]),
    "tmq_selftest_const_div": (c_int, [c_double, c_void_p, c_void_p]),
    "tmq_pack2b_f32": (c_int, [c_void_p, c_void_p, c_int64, c_int64, c_void_p]),
    "tmq_pack2b_i32": (c_int, [c_void_p, c_void_p, c_int64, c_int64, c_void_p]),
    "tmq_pack2b_i8": (c_int, [c_void_p, c_void_p, c_int64, c_int64, c_void_p]),
    "tmq_unpack2b_f32": (c_int, [c_void_p, c_void_p, c_int64, c_int64, c_void_p]),
    "tmq_ternary_conv2d_stem_bf16": (c_int, [c_void_p] * 5 + [c_int] * 13 + [c_void_p, c_void_p]),
    "tmq_maxpool2d_nhwc_bf16": (c_int, [c_void_p, c_void_p] + [c_int] * 8 + [c_void_p]),
    "tmq_ternary_dwconv2d_f32": (c_int, [c_void_p] * 5 + [c_int] * 12 + [c_void_p]),
    "tmq_maxpool2d_nhwc_f32_fwd": (c_int, [c_void_p, c_void_p, c_void_p] + [c_int] * 7 + [c_void_p]),
    "tmq_maxpool2d_nhwc_f32_bwd": (c_int, [c_void_p, c_void_p, c_void_p] + [c_int] * 7 + [c_void_p]),
    "tmq_ternary_dwconvtrans2d_f32": (c_int, [c_void_p] * 5 + [c_int] * 14 + [c_void_p]),
    "tmq_ternary_dwconv_patches_f32": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_void_p]),
    "tmq_ternary_dwconvtrans_patches_f32": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p]),
    "tmq_rc_encode_bound": (c_size_t, [c_int64, c_int64]),
    "tmq_rc_encode": (c_int, [c_void_p, c_int64, c_int64, c_void_p, c_size_t, ctypes.POINTER(c_size_t)]),
    "tmq_rc_decode": (c_int, [c_void_p, c_size_t, c_void_p, c_int64, c_int64]),
    "tmq_prepack_row_words": (c_size_t, [c_int64, c_int]),
    "tmq_prepack_words": (c_size_t, [c_int64, c_int64, c_int]),
    "tmq_prepack": (c_int, [c_void_p, c_void_p, c_int64, c_int64, c_int, c_void_p]),
    "tmq_ternary_gemm_bf16": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64,
                                      c_int64, c_int, c_void_p, c_void_p]),
    "tmq_ternary_gemm_workspace_bytes": (c_size_t, [c_int64, c_int64, c_int64, c_int]),
    "tmq_ternary_gemm_bf16_splitk": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64,
                                             c_int64, c_int, c_void_p, c_size_t, c_void_p, c_void_p]),
    "tmq_ternary_gemm_i8_splitk": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64, c_void_p,
                                           c_size_t, c_void_p, c_void_p]),
    "tmq_ternary_gemm_bf16_bcast": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int64, c_int64,
                                            c_int64, c_int64, c_void_p, c_void_p]),
    "tmq_ternary_gemv_bf16": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64,
                                      c_int64, c_int, c_void_p, c_void_p]),
    "tmq_ternary_gemv_i8": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64, c_void_p,
                                    c_void_p]),
    "tmq_ternary_gemv_batched_bf16": (c_int, [c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int64,
                                              c_int64, c_int64, c_int64, c_int, c_void_p, c_void_p]),
    "tmq_ternary_gemv_batched_i8": (c_int, [c_void_p, c_int64, c_void_p, c_void_p, c_int, c_int64, c_int64, c_int64,
                                            c_int64, c_void_p, c_void_p]),
    "tmq_qat_linear_workspace_bytes": (c_size_t, [c_int64, c_int64, c_int64]),
    "tmq_qat_linear_fwd_bf16": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64,
                                        ctypes.c_double, c_void_p, c_size_t, c_void_p, c_void_p]),
    "tmq_ternary_conv2d_bf16": (c_int, [c_void_p] * 6 + [c_int] * 14 + [c_void_p, c_void_p]),
    "tmq_ternary_conv2d_bf16_f32out": (c_int, [c_void_p] * 6 + [c_int] * 14 + [c_void_p, c_void_p]),
    "tmq_ternary_conv2d_s1_bf16": (c_int, [c_void_p] * 6 + [c_int] * 12 + [c_void_p, c_void_p]),
    "tmq_stem_rows_k": (c_int, [c_int, c_int, c_int, c_int]),
    "tmq_ternary_conv2d_stem_rows_bf16": (c_int, [c_void_p] * 5 + [c_int] * 12 + [c_void_p, c_void_p]),
    "tmq_ternary_conv2d_stem_rows_pool_bf16": (c_int, [c_void_p] * 5 + [c_int] * 11 + [c_void_p, c_void_p]),
    "tmq_ternary_conv2d_i8": (c_int, [c_void_p] * 3 + [c_int] * 13 + [c_void_p, c_void_p]),
    "tmq_split_f32_bf16": (c_int, [c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int, c_void_p]),
    "tmq_nchw_f32_to_nhwc_bf16": (c_int, [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p]),
    "tmq_avgpool_nhwc_bf16": (c_int, [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]),
    "tmq_conv_patches_bf16": (c_int, [c_void_p, c_void_p] + [c_int] * 13 + [c_void_p]),
    "tmq_ternary_gemm_i8": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64, c_void_p,
                                    c_void_p]),
}


class TmqError(RuntimeError):
    pass


def exported_symbols():
    """Names include/tmq_b200.h declares (kept in step with it by tests/test_abi.py)."""
    return sorted(_SIGNATURES)


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise TmqError(f"tmq_b200: {LIB_PATH} is missing; build it with `python -m tmq_b200.build` "
                           "(there is no fallback path)")
        L = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in _SIGNATURES.items():
            fn = getattr(L, name)
            fn.restype = res
            fn.argtypes = args
        _lib = L
    return _lib


def check(status, what):
    if status != 0:
        L = lib()
        msg = L.tmq_status_string(status).decode()
        extra = f" (cudaError {L.tmq_last_cuda_error()})" if status == -3 else ""
        raise TmqError(f"{what}: {msg}{extra}")
