"""GPU test of sm120_launch_quantize_fp8_static, the quantiser entry point that
allocates nothing.

It exists for callers that are not in a position to allocate device memory at
the time they run (a callback limited to the tensors it was handed, a serving
loop whose memory pool was fixed at start-up): they pass input, output and the
scale word, and the scratch that the ordinary entry point takes from the caller
sits in a 16 KB array inside the library.  The test calls the new entry point
straight through the C ABI, twice in a row with different inputs (the second
call finds the first call's leftovers in the shared array), and requires the
same bytes and the same scale as sm120_launch_quantize_fp8 produces with
caller-owned scratch -- both run the same kernels, so the match is exact.  It
also checks that a tensor beyond the built-in limit is refused before anything
is launched.  The file sorts last on purpose: if it fails in a run that stops
at the first failure, every other test has already run; it passes on its own
in a fresh process as well."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _both(lib, x, dtype_code):
    """(q, scale) from the scratch-taking entry point and from the allocation-free one."""
    n = x.numel()
    stream = torch.cuda.current_stream().cuda_stream
    q_ref = torch.empty(n, dtype=torch.uint8, device="cuda")
    s_ref = torch.zeros(1, device="cuda")
    scratch = torch.empty(max(4, lib.sm120_quantize_fp8_scratch_bytes(n)), dtype=torch.uint8, device="cuda")
    assert lib.sm120_launch_quantize_fp8(x.data_ptr(), dtype_code, n, q_ref.data_ptr(), s_ref.data_ptr(),
                                         scratch.data_ptr(), scratch.numel(), stream) == 0
    # outputs of the call under test are allocated up front by the caller; the call itself gets no scratch
    q_new = torch.full((n,), 0xAA, dtype=torch.uint8, device="cuda")
    s_new = torch.zeros(1, device="cuda")
    assert lib.sm120_launch_quantize_fp8_static(x.data_ptr(), dtype_code, n, q_new.data_ptr(), s_new.data_ptr(), stream) == 0
    torch.cuda.synchronize()
    return q_ref, s_ref, q_new, s_new


def test_static_scratch_quantiser_matches_the_scratch_taking_one(binding):
    lib = binding.load_library()
    assert hasattr(lib, "sm120_launch_quantize_fp8_static")
    torch.manual_seed(11)
    # call 1: many spans, so many slots of the shared array are written
    x1 = (4.0 * torch.randn(3_000_017, device="cuda")).bfloat16()
    q_ref, s_ref, q_new, s_new = _both(lib, x1, binding.DTYPE_BFLOAT16)
    assert torch.equal(q_new, q_ref) and float(s_new) == float(s_ref) and float(s_new) > 0
    # call 2, right after: a smaller tensor with a smaller maximum -- stale partial maxima of call 1 must not leak in
    x2 = 0.01 * torch.randn(70_001, device="cuda")
    q_ref, s_ref, q_new, s_new = _both(lib, x2, binding.DTYPE_FLOAT32)
    assert torch.equal(q_new, q_ref) and float(s_new) == float(s_ref)
    assert abs(float(s_new) - 448.0 / float(x2.abs().max())) <= 1e-6 * float(s_new)
    # the result is usable as a matmul operand scale without leaving the device
    assert int(q_new.max()) > 0


def test_static_scratch_quantiser_refuses_oversized_input(binding):
    lib = binding.load_library()
    x = torch.zeros(16, device="cuda")
    q = torch.zeros(16, dtype=torch.uint8, device="cuda")
    s = torch.full((1,), 7.0, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    too_many = binding.QUANTIZE_FP8_STATIC_MAX_ELEMENTS + 1
    before = binding.launch_count()
    # rejected on the size alone: nothing is launched and the outputs stay as they were
    assert lib.sm120_launch_quantize_fp8_static(x.data_ptr(), binding.DTYPE_FLOAT32, too_many, q.data_ptr(), s.data_ptr(), stream) == 1
    assert lib.sm120_launch_quantize_fp8_static(x.data_ptr(), binding.DTYPE_FP8_E4M3, 16, q.data_ptr(), s.data_ptr(), stream) == 1
    assert lib.sm120_launch_quantize_fp8_static(x.data_ptr(), binding.DTYPE_FLOAT32, 16, q.data_ptr(), None, stream) == 1
    torch.cuda.synchronize()
    assert binding.launch_count() == before and float(s) == 7.0
    # the largest size that is accepted by the size check is the documented one
    assert binding.QUANTIZE_FP8_STATIC_MAX_ELEMENTS == 4096 * 65536


def test_python_wrapper_allocates_nothing_on_the_device(ops):
    x = torch.randn(500_000, device="cuda").half()
    q = torch.empty(500_000, dtype=torch.float8_e4m3fn, device="cuda")
    s = torch.empty(1, device="cuda")
    ops.quantize_fp8_into(x, q, s)                       # first use on this device: also resolves the array's address
    torch.cuda.synchronize()
    before = torch.cuda.memory_allocated()
    ops.quantize_fp8_into(x, q, s)
    torch.cuda.synchronize()
    assert torch.cuda.memory_allocated() == before       # torch's allocator was not asked for anything
    q_ref, s_ref = ops.quantize_fp8(x)
    assert torch.equal(q.view(torch.uint8), q_ref.view(torch.uint8)) and float(s) == float(s_ref)
    with pytest.raises(ValueError):
        ops.quantize_fp8_into(x, q[:10], s)
