"""CPU tests of the C-ABI library: it loads, exports every function that
include/sm120_c_interface.h declares, its descriptor has the layout the ctypes
image assumes, and it rejects bad arguments before touching any device."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "sm120_c_interface.h")
INVALID = 1   # cudaErrorInvalidValue


def declared_functions():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    body = text[text.index('extern "C" {'):]
    names = re.findall(r"\b([a-z_0-9]+)\s*\(", body)
    return sorted({n for n in names if n.startswith("sm120_") or n.startswith("launch_sm120")})


def test_header_declares_expected_entry_points():
    names = declared_functions()
    for must in ("sm120_launch_matmul", "launch_sm120_matmul", "sm120_launch_matmul_ex", "sm120_is_supported",
                 "sm120_get_error_string", "sm120_launch_matmul_grad_a", "sm120_launch_matmul_grad_b"):
        assert must in names


def test_library_exports_every_declared_symbol(binding):
    lib = binding.load_library()
    for name in declared_functions():
        assert hasattr(lib, name), f"{name} is declared in the header but not exported"
        assert name in binding.EXPORTS, f"{name} has no ctypes signature in _binding.EXPORTS"
    assert os.path.basename(binding.LIBRARY_PATH) == "_sm120_ops.so"    # python/sm120_ops.py:30


def test_enum_values_keep_the_reference_numbering(binding):
    text = open(HEADER).read()
    for name, value in (("SM120_DTYPE_FLOAT32", 0), ("SM120_DTYPE_FLOAT16", 1), ("SM120_DTYPE_BFLOAT16", 2),
                        ("SM120_DTYPE_FP8_E4M3", 3), ("SM120_ACTIVATION_RELU", 0), ("SM120_ACTIVATION_GELU", 4),
                        ("SM120_ACTIVATION_SIGMOID", 8), ("SM120_ACTIVATION_GELU_ERF", 9), ("SM120_ACTIVATION_NONE", -1)):
        assert re.search(rf"\b{name}\s*=\s*{value}\b", text), name
    assert (binding.DTYPE_FLOAT32, binding.DTYPE_FLOAT16, binding.DTYPE_BFLOAT16, binding.DTYPE_FP8_E4M3) == (0, 1, 2, 3)


def test_descriptor_layout_and_defaults(binding):
    d = binding.new_desc()
    assert d.struct_size == ctypes.sizeof(binding.SM120GemmDesc)
    assert (d.batch, d.alpha, d.beta, d.scale_a, d.scale_b) == (1, 1.0, 0.0, 1.0, 1.0)
    assert (d.activation, d.path, d.optimization_level) == (-1, 0, 1)
    assert d.A is None and d.stream is None and d.M == 0


def _good_desc(binding):
    d = binding.new_desc()
    d.A, d.B, d.C = 0x1000, 0x2000, 0x3000     # never dereferenced: every case below is rejected first
    d.M, d.N, d.K = 64, 64, 64
    d.in_dtype = d.out_dtype = binding.DTYPE_FLOAT32
    return d


@pytest.mark.parametrize("mutate", [
    lambda d: setattr(d, "struct_size", 8),
    lambda d: setattr(d, "in_dtype", 7),
    lambda d: setattr(d, "out_dtype", 3),          # FP8 output
    lambda d: setattr(d, "out_dtype", -1),
    lambda d: setattr(d, "M", -1),
    lambda d: setattr(d, "batch", 0),
    lambda d: setattr(d, "activation", 10),
    lambda d: setattr(d, "activation", -2),
    lambda d: setattr(d, "path", 3),
    lambda d: setattr(d, "optimization_level", 3),
    lambda d: setattr(d, "lda", 8),                # pitch shorter than a row
    lambda d: setattr(d, "ldc", 63),
    lambda d: setattr(d, "C", None),
    lambda d: setattr(d, "A", None),
    lambda d: setattr(d, "scale_a", -1.0),
    lambda d: (setattr(d, "batch", 2), setattr(d, "stride_c", 10)),       # overlapping outputs
    lambda d: (setattr(d, "bias", 0x4000), setattr(d, "bias_dtype", 3)),  # FP8 bias
    lambda d: setattr(d, "tuning", 0x80),          # an undefined tuning bit
    lambda d: setattr(d, "tuning", 0x3),           # both CTA-group overrides at once
    lambda d: setattr(d, "tuning", 0xC),           # both epilogue-warp overrides at once
    lambda d: setattr(d, "tuning", 0x20),          # a trace without a buffer for it
])
def test_bad_descriptors_are_rejected_without_a_device(binding, mutate):
    lib = binding.load_library()
    d = _good_desc(binding)
    mutate(d)
    assert lib.sm120_launch_matmul_ex(ctypes.byref(d)) == INVALID


def test_null_descriptor_and_bad_dtype_enum(binding):
    lib = binding.load_library()
    assert lib.sm120_launch_matmul_ex(None) == INVALID
    # unknown dtype -> cudaErrorInvalidValue, as src/cuda_kernels/sm120_c_interface.cu:55-57
    assert lib.sm120_launch_matmul(0x1000, 0x2000, 0x3000, 4, 4, 4, 1.0, 0.0, 9, None) == INVALID
    assert lib.sm120_launch_matmul(0x1000, 0x2000, 0x3000, 4, 4, 4, 1.0, 0.0, 3, None) == INVALID
    assert lib.sm120_launch_matmul_grad_a(0x1000, 0x2000, 0x3000, 4, 4, 4, 1.0, 5, None) == INVALID
    assert lib.sm120_launch_matmul(0x1000, 0x2000, 0x3000, -4, 4, 4, 1.0, 0.0, 0, None) == INVALID


def test_empty_output_is_a_successful_no_op(binding):
    lib = binding.load_library()
    assert lib.sm120_launch_matmul(None, None, None, 0, 16, 16, 1.0, 0.0, 0, None) == 0
    assert lib.sm120_launch_matmul(None, None, None, 16, 0, 16, 1.0, 0.0, 1, None) == 0


def test_error_string_and_counters(binding):
    assert "invalid" in binding.error_string(1).lower()
    assert binding.error_string(0)
    assert isinstance(binding.launch_count(), int)
    assert isinstance(binding.last_kernel_name(), str)
