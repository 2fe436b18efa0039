"""ctypes binding of ``libnart_b200.so`` -- one Python callable per symbol that
``include/nart_b200.h`` declares.  There is no fallback: if the library is missing, importing
this module raises."""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libnart_b200.so")

OK = 0
ERR_INVALID, ERR_UNSUPPORTED, ERR_CUDA, ERR_NOMEM, ERR_DEVICE_WAIT = -1, -2, -3, -4, -5
ALGO_AUTO, ALGO_DIRECT, ALGO_IGEMM = 0, 1, 2
ACT_U8, ACT_S8 = 0, 1
POOL_MAX, POOL_AVE = 0, 1

i32, u8, f32 = C.c_int32, C.c_uint8, C.c_float
vp, sz = C.c_void_p, C.c_size_t
pi32 = C.POINTER(C.c_int32)


class ConvParams(C.Structure):
    """``b200_conv_params`` (include/nart_b200.h)."""

    _fields_ = [
        ("c", i32), ("h", i32), ("w", i32), ("k", i32), ("r", i32), ("s", i32),
        ("pad_h", i32), ("pad_w", i32), ("stride_h", i32), ("stride_w", i32), ("group", i32),
        ("ialpha", f32), ("izp", u8), ("wzp", u8), ("ozp", u8), ("obits", u8), ("oalpha", f32),
        ("walpha", C.POINTER(f32)), ("n_walpha", i32), ("relu", i32), ("algo", i32),
        ("act_type", i32), ("s8_wrap", i32),
    ]


# name -> (restype, argtypes); every exported symbol of the C-ABI
SIGNATURES = {
    "b200_strerror": (C.c_char_p, [C.c_int]),
    "b200_last_error": (C.c_char_p, []),
    "b200_version": (C.c_int, []),
    "b200_device_count": (C.c_int, [C.POINTER(C.c_int)]),
    "b200_set_device": (C.c_int, [C.c_int]),
    "b200_get_device": (C.c_int, [C.POINTER(C.c_int)]),
    "b200_malloc": (C.c_int, [C.POINTER(vp), sz]),
    "b200_free": (C.c_int, [vp]),
    "b200_malloc_host": (C.c_int, [C.POINTER(vp), sz]),
    "b200_free_host": (C.c_int, [vp]),
    "b200_memset": (C.c_int, [vp, C.c_int, sz, vp]),
    "b200_memcpy_h2d": (C.c_int, [vp, vp, sz, vp]),
    "b200_memcpy_d2h": (C.c_int, [vp, vp, sz, vp]),
    "b200_memcpy_d2d": (C.c_int, [vp, vp, sz, vp]),
    "b200_stream_create": (C.c_int, [C.POINTER(vp)]),
    "b200_stream_destroy": (C.c_int, [vp]),
    "b200_stream_synchronize": (C.c_int, [vp]),
    "b200_device_status": (C.c_int, [vp, C.POINTER(C.c_int)]),
    "b200_selftest_wait_expiry": (C.c_int, [C.c_uint64, vp]),
    "b200_measure_mma_i8_peak": (C.c_int, [i32, C.POINTER(f32), C.POINTER(C.c_double), vp]),
    "b200_get_quant_scale": (None, [f32, C.c_int, C.POINTER(C.c_uint32), C.POINTER(C.c_int8)]),
    "b200_conv2d_create": (C.c_int, [C.POINTER(ConvParams), vp, vp, C.POINTER(vp)]),
    "b200_conv2d_out_dims": (C.c_int, [vp, pi32, pi32]),
    "b200_conv2d_algo": (C.c_int, [vp]),
    "b200_conv2d_describe": (C.c_int, [vp, C.c_char_p, sz]),
    "b200_conv2d_run": (C.c_int, [vp, vp, i32, vp, vp]),
    "b200_conv2d_run_acc": (C.c_int, [vp, vp, i32, vp, vp, vp]),
    "b200_conv2d_reserve": (C.c_int, [vp, i32]),
    "b200_conv2d_destroy": (C.c_int, [vp]),
    "b200_conv2d_run_static_scratch": (C.c_int, [vp, vp, i32, vp, vp]),
    "b200_static_scratch_status": (C.c_int, [vp, C.POINTER(C.c_int)]),
    "b200_conv2d_fuse_residual_add": (C.c_int, [vp, i32, C.POINTER(f32), C.POINTER(u8), C.POINTER(f32), f32, u8, u8,
                                               i32]),
    "b200_conv2d_run_residual": (C.c_int, [vp, vp, i32, vp, vp, vp]),
    "b200_ip_create": (C.c_int, [i32, i32, i32, i32, f32, u8, C.POINTER(f32), i32, u8, f32, u8, u8,
                                 vp, vp, C.POINTER(vp)]),
    "b200_ip_create_s8": (C.c_int, [i32, i32, i32, i32, f32, C.POINTER(f32), i32, f32, u8, i32, vp, vp, C.POINTER(vp)]),
    "b200_quantize_s8": (C.c_int, [vp, vp, i32, i32, i32, i32, f32, u8, i32, vp]),
    "b200_dequantize_s8": (C.c_int, [vp, vp, i32, i32, i32, i32, f32, i32, vp]),
    "b200_quantize_u8": (C.c_int, [vp, vp, i32, i32, i32, i32, f32, u8, u8, i32, vp]),
    "b200_dequantize_u8": (C.c_int, [vp, vp, i32, i32, i32, i32, f32, u8, i32, vp]),
    "b200_nchw_to_nhwc_u8": (C.c_int, [vp, vp, i32, i32, i32, i32, i32, u8, vp]),
    "b200_nhwc_to_nchw_u8": (C.c_int, [vp, vp, i32, i32, i32, i32, i32, vp]),
    "b200_eltwise_sum_u8": (C.c_int, [C.POINTER(vp), i32, sz, C.POINTER(f32), C.POINTER(u8),
                                      C.POINTER(f32), f32, u8, u8, i32, vp, vp]),
    "b200_relu_u8": (C.c_int, [vp, sz, f32, u8, f32, u8, u8, vp, vp]),
    "b200_pool_out_dims": (C.c_int, [i32] * 9 + [pi32, pi32]),
    "b200_pool_u8": (C.c_int, [vp, i32, i32, i32, i32, i32, i32, i32, i32, i32, i32, i32, i32, f32,
                               u8, f32, u8, u8, vp, vp]),
    "b200_case_create": (C.c_int, [C.POINTER(vp)]),
    "b200_case_destroy": (C.c_int, [vp]),
    "b200_case_input_u8": (C.c_int, [vp, i32, i32, i32, pi32]),
    "b200_case_input_f32": (C.c_int, [vp, i32, i32, i32, f32, u8, u8, pi32]),
    "b200_case_conv2d": (C.c_int, [vp, i32, C.POINTER(ConvParams), vp, vp, pi32]),
    "b200_case_ip": (C.c_int, [vp, i32, i32, f32, u8, C.POINTER(f32), i32, u8, f32, u8, u8, vp, vp,
                               pi32]),
    "b200_case_eltwise_sum": (C.c_int, [vp, pi32, i32, C.POINTER(f32), C.POINTER(u8),
                                        C.POINTER(f32), f32, u8, u8, i32, pi32]),
    "b200_case_relu": (C.c_int, [vp, i32, f32, u8, f32, u8, u8, pi32]),
    "b200_case_pool": (C.c_int, [vp, i32, i32, i32, i32, i32, i32, i32, i32, i32, f32, u8, f32, u8,
                                 u8, pi32]),
    "b200_case_output_u8": (C.c_int, [vp, i32]),
    "b200_case_output_f32": (C.c_int, [vp, i32, f32, u8]),
    "b200_case_prepare": (C.c_int, [vp, i32]),
    "b200_case_tensor_dims": (C.c_int, [vp, i32, pi32, pi32, pi32]),
    "b200_case_io_bytes": (C.c_int, [vp, i32, i32, C.POINTER(sz)]),
    "b200_case_io_device_ptr": (C.c_int, [vp, i32, i32, C.POINTER(vp)]),
    "b200_case_tensor_device_ptr": (C.c_int, [vp, i32, C.POINTER(vp)]),
    "b200_case_run_device": (C.c_int, [vp, i32, vp]),
    "b200_case_run_host": (C.c_int, [vp, i32, C.POINTER(vp), C.POINTER(vp), vp]),
    "b200_case_submit_host": (C.c_int, [vp, i32, C.POINTER(vp), C.POINTER(vp)]),
    "b200_case_wait": (C.c_int, [vp]),
    "b200_case_launch_count": (C.c_int, [vp, pi32]),
    "b200_case_use_graph": (C.c_int, [vp, i32]),
    "b200_case_set_fusion": (C.c_int, [vp, i32]),
    "b200_case_set_profiling": (C.c_int, [vp, i32]),
    "b200_case_profile": (C.c_int, [vp, C.POINTER(f32), pi32, i32, pi32]),
}


class B200Error(RuntimeError):
    def __init__(self, status: int, detail: str):
        super().__init__("nart_b200 status %d: %s" % (status, detail))
        self.status = status
        self.detail = detail


def _load() -> C.CDLL:
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            "%s is missing: run `python -m nart_b200.build` (there is no CPU fallback)" % LIB_PATH)
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # raises AttributeError if the symbol is not exported
        fn.restype = res
        fn.argtypes = args
    return lib


lib = _load()


def check(status: int) -> None:
    if status != OK:
        raise B200Error(status, lib.b200_last_error().decode())
