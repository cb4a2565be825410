"""ctypes binding of libsharplight_cuda.so: one Python function per exported symbol of include/sharplight_cuda.h.

This is the Python counterpart of the [LibraryImport] class the managed provider would carry
(cf. src/Sharplight.Audio/Native/NativeMethods.cs:6-20 of the Sharplight tree): it loads the library, checks the ABI
version, and turns negative result codes into exceptions. There is no fallback: when the library is missing or its
ABI differs, loading raises.
"""
from __future__ import annotations

import ctypes as C
import os

PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("SHARPLIGHT_CUDA_LIBRARY", os.path.join(PKG, "libsharplight_cuda.so"))
ABI_VERSION = 1

OK = 0
ERR_INVALID_ARGUMENT, ERR_OUT_OF_MEMORY, ERR_NO_DEVICE, ERR_UNSUPPORTED = -1, -2, -3, -4
ERR_CUDA, ERR_INVALID_STATE, ERR_TIMEOUT, ERR_BUFFER_TOO_SMALL = -5, -6, -7, -8

FMT_Q4_0, FMT_Q8_0, FMT_Q4_K, FMT_Q6_K = 2, 8, 12, 14
FMT_Q5_0, FMT_IQ4_NL = 6, 20   # rewritten at upload as Q8_0 device records (exactly)
FMT_Q5_K = 13                  # split at upload into two Q4_K weights (exactly)
F32, BF16 = 0, 1
MATMUL_DEFAULT, MATMUL_ROW_INVARIANT, MATMUL_F32_ACTIVATIONS = 0, 1, 2
KERNEL_AUTO, KERNEL_MMVQ, KERNEL_SKINNY, KERNEL_MMQ, KERNEL_TILE, KERNEL_F32 = 0, 1, 2, 3, 4, 5
TP_MAX_RANKS, TP_MAX_ROWS, TP_HANDLE_BYTES, TP_COMM_ID_BYTES = 8, 64, 64, 128

BLOCK = {FMT_Q4_0: (32, 18), FMT_Q8_0: (32, 34), FMT_Q4_K: (256, 144), FMT_Q6_K: (256, 210), FMT_Q5_0: (32, 22), FMT_IQ4_NL: (32, 18),
         FMT_Q5_K: (256, 176)}


class DeviceInfoStruct(C.Structure):
    _fields_ = [("name", C.c_char * 256), ("driver", C.c_char * 64), ("uuid", C.c_uint8 * 16),
                ("total_memory", C.c_int64), ("free_memory", C.c_int64), ("sm_count", C.c_int32),
                ("cc_major", C.c_int32), ("cc_minor", C.c_int32), ("max_shared_per_block", C.c_int32),
                ("l2_bytes", C.c_int32), ("concurrent_workgroups", C.c_int32), ("supported", C.c_int32),
                ("reserved", C.c_int32)]


class NativeError(RuntimeError):
    """A negative slc_result. ``code`` is the result, the text carries slc_last_error_message()."""

    def __init__(self, code: int, message: str):
        super().__init__(f"libsharplight_cuda: {message} (code {code})")
        self.code = code


# every exported symbol with its ctypes signature; tests check the library exports exactly these
_vp, _i32, _i64, _u32 = C.c_void_p, C.c_int32, C.c_int64, C.c_uint32
_P = C.POINTER
SIGNATURES = {
    "slc_abi_version": (_i32, []),
    "slc_version_string": (C.c_char_p, []),
    "slc_error_string": (C.c_char_p, [_i32]),
    "slc_last_error_message": (C.c_char_p, []),
    "slc_device_count": (_i32, [_P(_i32)]),
    "slc_device_info_get": (_i32, [_i32, _P(DeviceInfoStruct)]),
    "slc_device_open": (_i32, [_i32, _P(_vp)]),
    "slc_device_close": (None, [_vp]),
    "slc_device_memory": (_i32, [_vp, _P(_i64), _P(_i64)]),
    "slc_device_sync": (_i32, [_vp]),
    "slc_device_stream": (_vp, [_vp]),
    "slc_last_status": (_i32, [_vp, _P(_i32)]),
    "slc_buffer_alloc": (_i32, [_vp, _i64, _P(_vp)]),
    "slc_buffer_free": (None, [_vp, _vp]),
    "slc_buffer_upload": (_i32, [_vp, _vp, _vp, _i64]),
    "slc_buffer_download": (_i32, [_vp, _vp, _vp, _i64]),
    "slc_host_alloc": (_i32, [_i64, _P(_vp)]),
    "slc_host_free": (None, [_vp]),
    "slc_buffer_copy_async": (_i32, [_vp, _vp, _vp, _i64, _i32, _vp]),
    "slc_stream_create": (_i32, [_vp, _P(_vp)]),
    "slc_stream_destroy": (None, [_vp, _vp]),
    "slc_stream_wait": (_i32, [_vp, _vp, _vp]),
    "slc_graph_begin": (_i32, [_vp, _vp]),
    "slc_graph_end": (_i32, [_vp, _vp, _P(_vp)]),
    "slc_graph_launch": (_i32, [_vp, _vp]),
    "slc_graph_destroy": (None, [_vp]),
    "slc_graph_last_error": (C.c_char_p, []),
    "slc_weight_upload": (_i32, [_vp, _i32, _i64, _i64, _vp, _i64, _P(_vp)]),
    "slc_weight_upload_kslice": (_i32, [_vp, _i32, _i64, _i64, _vp, _i64, _i64, _i64, _P(_vp)]),
    "slc_weight_download": (_i32, [_vp, _vp, _i64]),
    "slc_weight_shape": (_i32, [_vp, _P(_i32), _P(_i64), _P(_i64), _P(_i64)]),
    "slc_gguf_open": (_i32, [C.c_char_p, _P(_vp)]),
    "slc_gguf_close": (None, [_vp]),
    "slc_gguf_tensor_count": (_i32, [_vp, _P(_i64)]),
    "slc_gguf_tensor_info": (_i32, [_vp, _i64, C.c_char_p, _i32, _P(_i32), _P(_i32), _P(_i64), _P(_i64), _P(_i64)]),
    "slc_gguf_find": (_i32, [_vp, C.c_char_p, _P(_i64)]),
    "slc_weight_upload_gguf": (_i32, [_vp, _vp, _i64, _P(_vp)]),
    "slc_gguf_last_error": (C.c_char_p, []),
    "slc_weight_layout_bytes": (_i32, [_vp, _P(_i64)]),
    "slc_weight_export_layout": (_i32, [_vp, _vp, _i64]),
    "slc_weight_import_layout": (_i32, [_vp, _vp, _i64, _P(_vp)]),
    "slc_weight_free": (None, [_vp]),
    "slc_matmul_create": (_i32, [_vp, _vp, _i64, _u32, _P(_vp)]),
    "slc_matmul_create_dual": (_i32, [_vp, _vp, _vp, _i64, _u32, _P(_vp)]),
    "slc_matmul_destroy": (None, [_vp]),
    "slc_matmul_run": (_i32, [_vp, _vp, _i32, _i64, _i64, _i32, _vp, _i64, _i32, _vp]),
    "slc_matmul_set_kernel": (_i32, [_vp, _i32]),
    "slc_matmul_last_kernel": (_i32, [_vp, _P(_i32), _P(_i32)]),
    "slc_activation_create": (_i32, [_vp, _i64, _i64, _P(_vp)]),
    "slc_activation_destroy": (None, [_vp]),
    "slc_activation_quantize": (_i32, [_vp, _vp, _i32, _i64, _i64, _vp]),
    "slc_activation_set_rows": (_i32, [_vp, _vp, _i32, _i64, _i64, _vp]),
    "slc_activation_quantize_rmsnorm": (_i32, [_vp, _vp, _i32, _i64, _i64, _vp, C.c_float, _vp, _i64, _vp]),
    "slc_activation_quantize_silu_mul": (_i32, [_vp, _vp, _i64, _vp, _i64, _i64, _vp, _i64, _vp]),
    "slc_buffer_densify": (_i32, [_vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _i64, _i32, _vp]),
    "slc_argmax_rows": (_i32, [_vp, _vp, _i64, _i64, _i64, _vp, _vp]),
    "slc_matmul_run_quantized": (_i32, [_vp, _vp, _vp, _i64, _vp]),
    "slc_tp_exchange_create": (_i32, [_vp, _i32, _i32, _i64, _i64, _P(_vp), _vp]),
    "slc_tp_exchange_connect": (_i32, [_vp, _vp]),
    "slc_tp_exchange_destroy": (None, [_vp]),
    "slc_tp_exchange_set_wait_ms": (_i32, [_vp, _i32]),
    "slc_tp_comm_unique_id": (_i32, [_vp]),
    "slc_tp_comm_create": (_i32, [_vp, _i32, _i32, _vp, _P(_vp)]),
    "slc_tp_comm_destroy": (None, [_vp]),
    "slc_tp_comm_set_chunking": (_i32, [_vp, _i32]),
    "slc_tp_exchange_set_comm": (_i32, [_vp, _vp, _i32]),
    "slc_matmul_run_allreduce": (_i32, [_vp, _vp, _vp, _i32, _i64, _i64, _vp, _i64, _vp]),
    "slc_matmul_run_quantized_allreduce": (_i32, [_vp, _vp, _vp, _vp, _i64, _vp]),
    "slc_matmul_run_quantized_epilogue": (_i32, [_vp, _vp, _vp, _vp, _vp, _i64, _vp, _i64, _vp]),
    "slc_matmul_run_static": (_i32, [_vp, _vp, _i32, _i64, _i64, _vp, _i64, _vp]),
    "slc_matmul_id_run": (_i32, [_vp, _i32, _vp, _i32, _i64, _vp, _i64, _i64, _i32, _vp, _i64, _vp]),
    "slc_static_last_error": (C.c_char_p, []),
    "slc_debug_quantize": (_i32, [_vp, _vp, _i32, _i64, _i64, _vp, _vp, _vp]),
    "slc_debug_block_dots": (_i32, [_vp, _vp, _i32, _i64, _vp]),
}

_lib = None


def load() -> C.CDLL:
    """Loads the library once. Raises when it is missing (no silent fallback) or its ABI version differs."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise FileNotFoundError(
            f"{LIB_PATH} is missing: build it with `python -m sharplight_b200.build` "
            "(the CUDA provider has no CPU fallback)")
    lib = C.CDLL(LIB_PATH)
    for name, (restype, argtypes) in SIGNATURES.items():
        fn = getattr(lib, name)   # AttributeError names the missing export
        fn.restype = restype
        fn.argtypes = argtypes
    got = lib.slc_abi_version()
    if got != ABI_VERSION:
        raise RuntimeError(f"libsharplight_cuda ABI version {got}, this binding needs {ABI_VERSION}")
    _lib = lib
    return lib


def check(code: int) -> None:
    if code < 0:
        lib = load()
        detail = lib.slc_last_error_message().decode() or lib.slc_error_string(code).decode()
        raise NativeError(code, detail)
