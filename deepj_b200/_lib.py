"""ctypes binding of libdeepj_cuda_jni.so (the C ABI declared in include/deepj_cuda.h).

There is no CPU fallback: if the shared library is missing or a call fails, an
exception is raised.
"""
from __future__ import annotations

import ctypes
import os

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "libdeepj_cuda_jni.so")

_i32p = ctypes.POINTER(ctypes.c_int32)
_f32p = ctypes.POINTER(ctypes.c_float)
_i8p = ctypes.POINTER(ctypes.c_int8)
_i64p = ctypes.POINTER(ctypes.c_int64)

# name → (restype, argtypes); every symbol include/deepj_cuda.h declares
SIGNATURES = {
    "deepj_cuda_alloc_buffers": (ctypes.c_int, [_i32p, _i32p, ctypes.c_int32]),
    "deepj_cuda_upload_buffer": (ctypes.c_int, [ctypes.c_int32, ctypes.c_void_p, ctypes.c_int32]),
    "deepj_cuda_download_buffer": (ctypes.c_int, [ctypes.c_int32, ctypes.c_void_p, ctypes.c_int32]),
    "deepj_cuda_release_buffers": (ctypes.c_int, [_i32p, ctypes.c_int32]),
    "deepj_cuda_flush_ops": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_int32]),
    "deepj_cuda_last_error": (ctypes.c_char_p, []),
    "deepj_cuda_init": (ctypes.c_int, [ctypes.c_int32]),
    "deepj_cuda_shutdown": (ctypes.c_int, []),
    "deepj_cuda_flush_ops_async": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_int32]),
    "deepj_cuda_synchronize": (ctypes.c_int, []),
    "deepj_cuda_pinned_alloc": (ctypes.c_int, [ctypes.POINTER(ctypes.c_void_p), ctypes.c_int64]),
    "deepj_cuda_pinned_free": (ctypes.c_int, [ctypes.c_void_p]),
    "deepj_cuda_timer_begin": (ctypes.c_int, []),
    "deepj_cuda_timer_end": (ctypes.c_int, [_f32p]),
    "deepj_cuda_profile_ops": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_int32, ctypes.c_void_p, ctypes.c_int32, _i32p]),
    "deepj_cuda_trace_read": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_int32, _i32p]),
    "deepj_cuda_stats": (ctypes.c_int, [_i64p, ctypes.c_int32]),
    "deepj_cuda_q8_alloc": (ctypes.c_int, [ctypes.c_int32, ctypes.c_int32, ctypes.c_int32]),
    "deepj_cuda_q8_quantize_into": (ctypes.c_int, [ctypes.c_int32] * 7),
    "deepj_cuda_q8_upload": (ctypes.c_int, [ctypes.c_int32, ctypes.c_void_p, ctypes.c_void_p]),
    "deepj_cuda_q8_download": (ctypes.c_int, [ctypes.c_int32, ctypes.c_void_p, ctypes.c_void_p]),
    "deepj_cuda_synth_fill": (ctypes.c_int, [ctypes.c_int32, ctypes.c_uint64, ctypes.c_uint64, ctypes.c_float, ctypes.c_int64, ctypes.c_int64]),
    "deepj_cuda_kv_alloc": (ctypes.c_int, [ctypes.c_int32] * 6),
    "deepj_cuda_kv_alloc_f16": (ctypes.c_int, [ctypes.c_int32] * 6),
    "deepj_cuda_tp_create": (ctypes.c_int, [ctypes.c_int32, ctypes.c_int32, ctypes.c_int64, ctypes.c_void_p]),
    "deepj_cuda_decode_plan": (ctypes.c_int, [ctypes.c_int32, ctypes.c_void_p, ctypes.c_int32]),
    "deepj_cuda_tp_configure": (ctypes.c_int, [ctypes.c_int64]),
    "deepj_cuda_tc_configure": (ctypes.c_int, [ctypes.c_int32]),
    "deepj_cuda_tp_connect": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_int32]),
    "deepj_cuda_clear_device_error": (ctypes.c_int, []),
    "deepj_cuda_tp_destroy": (ctypes.c_int, []),
    "deepj_cuda_attn_decode_static": (ctypes.c_int, [ctypes.c_int32] * 16),
}

_lib = None


class DeepJCudaError(RuntimeError):
    """Raised when a libdeepj_cuda_jni call reports failure (the JNI shim raises
    java.lang.RuntimeException in the same place)."""


def load() -> ctypes.CDLL:
    """Load the shared library and bind every declared symbol.  Does not touch a GPU."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise DeepJCudaError(
            f"{LIB_PATH} is missing: build it with `python -m deepj_b200.build` (there is no CPU fallback)")
    lib = ctypes.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def check(status: int) -> None:
    if status != 0:
        msg = load().deepj_cuda_last_error()
        raise DeepJCudaError(msg.decode("utf-8", "replace") if msg else "unknown error")
