"""GPU parity tests of the FP8 quantiser (sm120_launch_quantize_fp8, through the
C ABI) against the oracle's quantiser: scale = 448 / amax, saturating
round-to-nearest-even e4m3 (src/cuda_kernels/sm120_datatype_support.h:168-171)."""
import ctypes

import numpy as np
import pytest
import torch

from oracle import reference as ref
from tests import _util as U

pytestmark = pytest.mark.gpu


def _oracle(x32: np.ndarray):
    s = np.float32(ref.fp8_scale(x32))
    return ref.quantize(x32.astype(np.float32) * s, "fp8_e4m3"), float(s)


@pytest.mark.parametrize("dtype", ["float32", "float16", "bfloat16"])
@pytest.mark.parametrize("n", [1, 7, 4096, 65535, 65536, 65537, 1_000_003])
def test_quantizer_matches_oracle(ops, dtype, n):
    rng = np.random.default_rng(n)
    x = ref.quantize(3.0 * rng.standard_normal(n, dtype=np.float32), dtype)
    q, s = ops.quantize_fp8(U.to_cuda(x))
    torch.cuda.synchronize()
    want_q, want_s = _oracle(x.astype(np.float32))
    got_s = float(s.item())
    assert abs(got_s - want_s) <= 1.2e-7 * want_s            # fp32 division vs float64 division rounded to fp32
    got_q = U.to_numpy(q)
    assert got_q.shape == x.shape and got_q.dtype == want_q.dtype
    if got_s == want_s:
        assert np.array_equal(got_q.view(np.uint8), want_q.view(np.uint8))
    else:
        assert np.mean(got_q.view(np.uint8) == want_q.view(np.uint8)) > 0.999
    assert float(np.max(np.abs(got_q.astype(np.float32)))) == 448.0      # amax maps to 448 (the FP8 workload)


def test_quantizer_edge_cases(ops, binding):
    lib = binding.load_library()
    # an all-zero tensor keeps scale 1 and stays zero
    q, s = ops.quantize_fp8(torch.zeros(1000, device="cuda"))
    assert float(s.item()) == 1.0 and int(q.view(torch.uint8).max()) == 0
    # operands that are not 16-byte aligned take the element-wise path
    rng = np.random.default_rng(3)
    base = torch.from_numpy(rng.standard_normal(200_001, dtype=np.float32)).cuda().bfloat16()
    x = base[1:]
    assert x.data_ptr() % 16 != 0
    q, s = ops.quantize_fp8(x)
    want_q, want_s = _oracle(U.to_numpy(x).astype(np.float32))
    assert abs(float(s.item()) - want_s) <= 1.2e-7 * want_s
    assert np.mean(U.to_numpy(q).view(np.uint8) == want_q.view(np.uint8)) > 0.999
    # 2-D input keeps its shape; the scale feeds the matmul as a device scalar
    a32 = torch.randn(256, 512, device="cuda")
    b32 = torch.randn(384, 512, device="cuda")
    qa, sa = ops.quantize_fp8(a32)
    qb, sb = ops.quantize_fp8(b32)
    c = ops.fused_matmul(qa, qb, transpose_b=True, scale_a=sa, scale_b=sb)
    exact = (a32.double() @ b32.double().T).cpu().numpy()
    assert ref.rel_frobenius(U.to_numpy(c), exact) <= ref.TOLERANCE["fp8_e4m3"]
    # argument checks of the C entry point: too little scratch, bad dtype, null scale
    n = 100_000
    need = lib.sm120_quantize_fp8_scratch_bytes(n)
    assert need == 8 and lib.sm120_quantize_fp8_scratch_bytes(0) == 0 and lib.sm120_quantize_fp8_scratch_bytes(65536) == 4
    x = torch.randn(n, device="cuda")
    out = torch.empty(n, dtype=torch.uint8, device="cuda")
    sc = torch.empty(1, device="cuda")
    scratch = torch.empty(16, dtype=torch.uint8, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    assert lib.sm120_launch_quantize_fp8(x.data_ptr(), 0, n, out.data_ptr(), sc.data_ptr(), scratch.data_ptr(), 4, stream) == 1
    assert lib.sm120_launch_quantize_fp8(x.data_ptr(), 3, n, out.data_ptr(), sc.data_ptr(), scratch.data_ptr(), 16, stream) == 1
    assert lib.sm120_launch_quantize_fp8(x.data_ptr(), 0, n, out.data_ptr(), None, scratch.data_ptr(), 16, stream) == 1
    assert lib.sm120_launch_quantize_fp8(x.data_ptr(), 0, n, out.data_ptr(), sc.data_ptr(), scratch.data_ptr(), 16, stream) == 0
    torch.cuda.synchronize()


def test_quantizer_full_size_slab(ops):
    # one rank's A slab of the M-sharded FP8 workload: 8192 x 8192 fp32 -> e4m3; idempotence and round trip as size-independent checks
    torch.manual_seed(0)
    x = torch.randn(8192, 8192, device="cuda")
    q, s = ops.quantize_fp8(x)
    deq = q.float() / s
    # e4m3 keeps 3 mantissa bits: relative error of a normal value is at most 2^-4
    big = x.abs() > (2.0 ** -6) / s
    assert float(((deq - x).abs() / x.abs())[big].max()) <= 2.0 ** -4 + 1e-6
    q2, s2 = ops.quantize_fp8(deq)                      # quantising the dequantised tensor changes nothing
    assert torch.equal(q2.view(torch.uint8), q.view(torch.uint8)) and abs(float(s2) - float(s)) <= 1e-6 * float(s)
