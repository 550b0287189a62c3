"""GPU parity against code the reference itself holds: its activation kernel
(src/cuda_kernels/sm120_pure_kernels.cu:128-176), compiled unmodified for B200
into oracle/_ref/ by oracle/Makefile and launched as the reference launcher does
(src/cuda_kernels/sm120_c_interface.cu:139-164).  It pins the activation table
shared by the standalone launcher, the fused GEMM epilogue and the numpy oracle
to the reference's own formulas and constants.  (The reference's matmul
launchers do not build; oracle/Makefile quotes the compiler.)"""
import ctypes
import os

import numpy as np
import pytest
import torch

from oracle import reference as ref
from tests import _util as U

pytestmark = pytest.mark.gpu

REF_SO = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle", "_ref", "libsm120_reference_kernels.so")


@pytest.fixture(scope="module")
def reflib():
    if not os.path.exists(REF_SO):
        pytest.skip("oracle/_ref/libsm120_reference_kernels.so is not built (needs the reference tree at build time)")
    lib = ctypes.CDLL(REF_SO)
    lib.sm120_reference_activation.restype = ctypes.c_int
    lib.sm120_reference_activation.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int]
    return lib


def _inputs(n, seed):
    rng = np.random.default_rng(seed)
    x = 3.0 * rng.standard_normal(n, dtype=np.float32)
    x[:9] = [0.0, -0.0, 1.0, -1.0, 1e-6, -1e-6, 8.0, -8.0, 0.5]
    return x


@pytest.mark.parametrize("code", list(range(0, 9)))
def test_standalone_activation_matches_reference_kernel(reflib, binding, code):
    lib = binding.load_library()
    n = 70_001
    for is_half in (0, 1):
        x = _inputs(n, 40 + code)
        tx = torch.from_numpy(x).cuda()
        if is_half:
            tx = tx.half()
        want = torch.empty_like(tx)
        got = torch.empty_like(tx)
        torch.cuda.synchronize()
        assert reflib.sm120_reference_activation(tx.data_ptr(), want.data_ptr(), n, code, is_half) == 0
        assert lib.sm120_launch_activation(tx.data_ptr(), got.data_ptr(), n, code, is_half, torch.cuda.current_stream().cuda_stream) == 0
        torch.cuda.synchronize()
        # the same fp32 formulas compiled twice: identical up to the compiler's contraction choices
        g, w = got.float().cpu().numpy(), want.float().cpu().numpy()
        assert np.all(np.isfinite(g))
        assert np.max(np.abs(g - w) / (1.0 + np.abs(w))) <= (1e-3 if is_half else 2e-6), (code, is_half)
        if code in (0, 1) or (code == 7 and not is_half):    # relu, leaky relu, fp32 tanh: nothing to contract differently
            assert np.array_equal(g, w)                      # (16-bit tensors use exponential forms, exact after rounding but for rare ties)
        # and the numpy oracle's table agrees with the reference kernel
        o = ref.activation(tx.float().cpu().numpy().astype(np.float64), code)
        assert np.max(np.abs(o - w) / (1.0 + np.abs(o))) <= (1e-3 if is_half else 2e-6), (code, is_half)


@pytest.mark.parametrize("code", list(range(0, 9)))
def test_fused_epilogue_matches_reference_kernel(reflib, ops, code):
    # act(x . w + b) in one launch (fp32 out) == the reference's activation kernel applied to the unfused x . w + b
    torch.manual_seed(50 + code)
    x = torch.randn(264, 136, device="cuda").bfloat16()
    w = (0.2 * torch.randn(136, 392, device="cuda")).bfloat16()
    b = torch.randn(392, device="cuda")
    fused = ops.fused_matmul(x, w, bias=b, activation=code, out_dtype=torch.float32)
    pre = ops.fused_matmul(x, w, bias=b, out_dtype=torch.float32).contiguous()
    want = torch.empty_like(pre)
    torch.cuda.synchronize()
    assert reflib.sm120_reference_activation(pre.data_ptr(), want.data_ptr(), pre.numel(), code, 0) == 0
    assert float(((fused - want).abs() / (1.0 + want.abs())).max()) <= 2e-6, code
