"""ctypes binding of the C ABI in include/sm120_c_interface.h.

This is the Python-side equivalent of ``tf.load_op_library("_sm120_ops.so")``
(python/sm120_ops.py:28-38 in the reference): it loads the same artefact name
from the package directory.  There is no fallback implementation: when the
library is missing, or a launch fails, the caller gets an exception.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import (POINTER, Structure, c_bool, c_char_p, c_float, c_int, c_int32, c_int64, c_uint, c_uint32,
                    c_uint64, c_void_p)

LIBRARY_NAME = "_sm120_ops.so"
LIBRARY_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), LIBRARY_NAME)

# SM120DataType
DTYPE_FLOAT32, DTYPE_FLOAT16, DTYPE_BFLOAT16, DTYPE_FP8_E4M3 = 0, 1, 2, 3
# SM120ActivationType
ACT_NONE, ACT_RELU, ACT_LEAKY_RELU, ACT_ELU, ACT_SELU, ACT_GELU_TANH = -1, 0, 1, 2, 3, 4
ACT_SWISH, ACT_MISH, ACT_TANH, ACT_SIGMOID, ACT_GELU_ERF = 5, 6, 7, 8, 9
# SM120KernelPath
PATH_AUTO, PATH_TENSOR_CORE, PATH_SIMT = 0, 1, 2

CUDA_SUCCESS = 0
CUDA_ERROR_INVALID_VALUE = 1
QUANTIZE_FP8_STATIC_MAX_ELEMENTS = 268435456      # SM120_QUANTIZE_FP8_STATIC_MAX_ELEMENTS

# SM120_TUNE_* bits of SM120GemmDesc.tuning (per-call overrides for tests and tuning runs)
TUNE_CTA_GROUP_1, TUNE_CTA_GROUP_2, TUNE_EPI_WARPS_8, TUNE_EPI_WARPS_16 = 0x1, 0x2, 0x4, 0x8
TUNE_NO_SPLIT_TAIL, TUNE_TRACE, TUNE_NO_SPLIT_K = 0x10, 0x20, 0x40
TRACE_WORDS_PER_CTA, TRACE_MAX_CTAS = 40, 160
TRACE_BYTES = TRACE_MAX_CTAS * TRACE_WORDS_PER_CTA * 8


def tune_group_m(g: int) -> int:
    return (int(g) & 0xFF) << 8


def tune_stall_kblock(kb: int) -> int:
    return ((int(kb) + 1) & 0xFF) << 16


class SM120GemmDesc(Structure):
    """Field-for-field image of ``struct SM120GemmDesc``."""
    _fields_ = [
        ("struct_size", c_uint32),
        ("in_dtype", c_int32),
        ("out_dtype", c_int32),
        ("bias_dtype", c_int32),
        ("A", c_void_p),
        ("B", c_void_p),
        ("C", c_void_p),
        ("bias", c_void_p),
        ("M", c_int64), ("N", c_int64), ("K", c_int64),
        ("lda", c_int64), ("ldb", c_int64), ("ldc", c_int64),
        ("batch", c_int64),
        ("stride_a", c_int64), ("stride_b", c_int64), ("stride_c", c_int64),
        ("transpose_a", c_int32), ("transpose_b", c_int32),
        ("alpha", c_float), ("beta", c_float),
        ("scale_a", c_float), ("scale_b", c_float),
        ("scale_a_dev", c_void_p),
        ("scale_b_dev", c_void_p),
        ("activation", c_int32),
        ("path", c_int32),
        ("optimization_level", c_int32),
        ("tuning", c_int32),
        ("stream", c_void_p),
        ("workspace", c_void_p),
        ("workspace_bytes", c_uint64),
    ]


# name -> (restype, argtypes): every symbol the public header declares
EXPORTS = {
    "sm120_launch_matmul": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_float, c_int, c_void_p]),
    "launch_sm120_matmul": (None, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]),
    "sm120_gemm_desc_init": (None, [POINTER(SM120GemmDesc)]),
    "sm120_launch_matmul_ex": (c_int, [POINTER(SM120GemmDesc)]),
    "sm120_matmul_workspace_bytes": (ctypes.c_size_t, [POINTER(SM120GemmDesc)]),
    "sm120_launch_matmul_gather": (c_int, [POINTER(SM120GemmDesc), POINTER(c_void_p), c_int]),
    "sm120_enable_peer_access": (c_int, [c_int]),
    "sm120_ipc_export": (c_int, [c_void_p, c_void_p, POINTER(c_uint64)]),
    "sm120_ipc_import": (c_int, [c_void_p, POINTER(c_void_p)]),
    "sm120_ipc_close": (c_int, [c_void_p]),
    "sm120_launch_matmul_grad_a": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_int, c_void_p]),
    "sm120_launch_matmul_grad_b": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_int, c_void_p]),
    "sm120_quantize_fp8_scratch_bytes": (ctypes.c_size_t, [c_int64]),
    "sm120_launch_quantize_fp8": (c_int, [c_void_p, c_int, c_int64, c_void_p, c_void_p, c_void_p, ctypes.c_size_t, c_void_p]),
    "sm120_launch_quantize_fp8_static": (c_int, [c_void_p, c_int, c_int64, c_void_p, c_void_p, c_void_p]),
    "sm120_launch_cast_fp8": (c_int, [c_void_p, c_int, c_int64, c_void_p, c_void_p, c_void_p]),
    "sm120_launch_activation": (c_int, [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]),
    "sm120_launch_bias_activation": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_int64, c_int64, c_int, c_int, c_void_p]),
    "sm120_launch_softmax": (c_int, [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p]),
    "sm120_launch_softmax_ex": (c_int, [c_void_p, c_void_p, c_int64, c_int64, c_int, c_int, c_float, c_void_p, c_int64, c_float,
                                        c_int, c_int64, c_void_p]),
    "sm120_launch_attention": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_int, c_void_p]),
    "sm120_launch_attention_ex": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64,
                                          c_float, c_int, c_int, c_void_p]),
    "sm120_launch_bias_grad": (c_int, [c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int, c_int, c_void_p]),
    "sm120_is_supported": (c_bool, [c_int]),
    "sm120_get_error_string": (c_char_p, [c_int]),
    "sm120_get_kernel_status": (c_int, [c_int, POINTER(c_uint), c_int]),
    "sm120_get_kernel_clock": (c_int, [c_int, POINTER(ctypes.c_ulonglong), POINTER(ctypes.c_ulonglong)]),
    "sm120_get_tensor_map_stats": (None, [POINTER(c_uint64), POINTER(c_uint64)]),
    "sm120_set_wait_limit_ms": (None, [c_uint]),
    "sm120_get_launch_count": (c_uint64, []),
    "sm120_get_last_kernel_name": (c_char_p, []),
    "sm120_get_last_split_k": (c_int, []),
}

_lib = None
_load_error: Exception | None = None


def load_library() -> ctypes.CDLL:
    """Load ``_sm120_ops.so`` once and type its entry points.  Raises OSError
    when the library has not been built (run ``make`` in csrc/ or
    ``__graft_entry__.build()``)."""
    global _lib, _load_error
    if _lib is not None:
        return _lib
    if _load_error is not None:
        raise _load_error
    try:
        if not os.path.exists(LIBRARY_PATH):
            raise OSError(f"{LIBRARY_PATH} not found: build it with `make -C {os.path.dirname(LIBRARY_PATH)}/csrc`")
        lib = ctypes.CDLL(LIBRARY_PATH)
        for name, (restype, argtypes) in EXPORTS.items():
            fn = getattr(lib, name)   # AttributeError if the symbol is not exported
            fn.restype = restype
            fn.argtypes = argtypes
    except Exception as e:  # remember and re-raise on every later call
        _load_error = e
        raise
    _lib = lib
    return lib


def library_loaded() -> bool:
    try:
        load_library()
        return True
    except Exception:
        return False


def new_desc() -> SM120GemmDesc:
    d = SM120GemmDesc()
    load_library().sm120_gemm_desc_init(ctypes.byref(d))
    return d


def error_string(code: int) -> str:
    s = load_library().sm120_get_error_string(int(code))
    return s.decode() if s else f"cuda error {code}"


def last_kernel_name() -> str:
    s = load_library().sm120_get_last_kernel_name()
    return s.decode() if s else ""


def last_split_k() -> int:
    """K ranges of this thread's last matmul launch (1 = not split)."""
    return int(load_library().sm120_get_last_split_k())


def launch_count() -> int:
    return int(load_library().sm120_get_launch_count())


def kernel_clock_mhz(device_index: int):
    """SM clock (MHz) seen from inside the last tensor-core launch on the device, or None."""
    cyc, ns = ctypes.c_ulonglong(0), ctypes.c_ulonglong(0)
    rc = load_library().sm120_get_kernel_clock(int(device_index), ctypes.byref(cyc), ctypes.byref(ns))
    if rc != CUDA_SUCCESS or ns.value == 0:
        return None
    return 1e3 * cyc.value / ns.value


def tensor_map_stats():
    """(maps encoded through the driver, launches' maps taken from a thread's cache) since load."""
    enc, hit = c_uint64(0), c_uint64(0)
    load_library().sm120_get_tensor_map_stats(ctypes.byref(enc), ctypes.byref(hit))
    return int(enc.value), int(hit.value)
