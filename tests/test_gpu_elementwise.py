"""GPU parity tests of the HBM-bound companions of the matmul op, called through
the C ABI: the standalone activation launcher (sm120_launch_activation, the
reference signature of src/cuda_kernels/sm120_c_interface.h:95-100), its bias
form, the bias gradient (column sums), the FP8 cast with a given scale, and a
trainable Dense step against float64 autograd on the CPU."""
import ctypes

import numpy as np
import pytest
import torch

from oracle import reference as ref
from tests import _util as U

pytestmark = pytest.mark.gpu

DT = {"float32": 0, "float16": 1, "bfloat16": 2}
# fp32 math, one rounding to the output type: half an ulp of the type plus the error of the device's math functions
TOL_ABS = {"float32": 2e-6, "float16": 1e-3, "bfloat16": 8e-3}


def _act_oracle(x, code, dtype, bias=None):
    v = x.astype(np.float64)
    if bias is not None:
        v = v + bias.astype(np.float64)
    return ref.activation(v, code)


@pytest.mark.parametrize("dtype", ["float32", "float16", "bfloat16"])
@pytest.mark.parametrize("code", list(range(0, 10)))
def test_activation_reference_signature(binding, dtype, code):
    lib = binding.load_library()
    rng = np.random.default_rng(10 * code + DT[dtype])
    for n in (1, 7, 4096, 100_003, 1_048_576 + 24):
        x = ref.quantize(2.5 * rng.standard_normal(n, dtype=np.float32), dtype)
        tx = U.to_cuda(x)
        out = torch.empty_like(tx)
        rc = lib.sm120_launch_activation(tx.data_ptr(), out.data_ptr(), n, code, DT[dtype], torch.cuda.current_stream().cuda_stream)
        assert rc == 0
        torch.cuda.synchronize()
        assert binding.last_kernel_name() == "activation_vec16"
        want = _act_oracle(x, code, dtype)
        got = U.to_numpy(out).astype(np.float64)
        assert np.max(np.abs(got - want) / (1.0 + np.abs(want))) <= TOL_ABS[dtype], (dtype, code, n)


def test_activation_edges(binding, ops):
    lib = binding.load_library()
    stream = torch.cuda.current_stream().cuda_stream
    x = torch.randn(1000, device="cuda")
    out = torch.empty_like(x)
    # unknown codes leave the values unchanged (src/cuda_kernels/sm120_pure_kernels.cu:167-169); so does NONE
    for code in (-1, 10, 99):
        assert lib.sm120_launch_activation(x.data_ptr(), out.data_ptr(), 1000, code, 0, stream) == 0
        assert torch.equal(out, x)
    # a dtype the launcher does not know is rejected (src/cuda_kernels/sm120_c_interface.cu:160-162)
    assert lib.sm120_launch_activation(x.data_ptr(), out.data_ptr(), 1000, 0, 3, stream) == 1
    assert lib.sm120_launch_activation(x.data_ptr(), out.data_ptr(), -1, 0, 0, stream) == 1
    assert lib.sm120_launch_activation(None, out.data_ptr(), 10, 0, 0, stream) == 1
    assert lib.sm120_launch_activation(None, None, 0, 0, 0, stream) == 0
    # in place, and on a view that is not 16-byte aligned (element-wise path)
    y = x.clone()
    assert lib.sm120_launch_activation(y.data_ptr(), y.data_ptr(), 1000, 0, 0, stream) == 0
    assert torch.equal(y, torch.relu(x))
    base = torch.randn(5001, device="cuda").half()
    v = base[1:]
    assert v.data_ptr() % 16 != 0
    got = ops.fused_activation(v, "sigmoid")
    want = _act_oracle(U.to_numpy(v), 8, "float16")
    assert np.max(np.abs(U.to_numpy(got).astype(np.float64) - want)) <= 1e-3
    torch.cuda.synchronize()


@pytest.mark.parametrize("dtype,bias_dtype", [("bfloat16", "bfloat16"), ("float16", "float32"), ("float32", "float32"),
                                              ("bfloat16", "float32")])
def test_bias_activation(ops, binding, dtype, bias_dtype):
    rng = np.random.default_rng(5)
    for (rows, cols), act in (((64, 264), "gelu"), ((33, 1000), "relu"), ((7, 13), "tanh"), ((1024, 2048), "swish")):
        x = ref.quantize(rng.standard_normal((rows, cols), dtype=np.float32), dtype)
        bias = ref.quantize(rng.standard_normal(cols, dtype=np.float32), bias_dtype)
        got = ops.fused_activation(U.to_cuda(x), act, bias=U.to_cuda(bias))
        torch.cuda.synchronize()
        assert binding.last_kernel_name() == "bias_activation_vec16"
        want = _act_oracle(x, ops.activation_code(act), dtype, bias=bias)
        err = np.max(np.abs(U.to_numpy(got).astype(np.float64) - want) / (1.0 + np.abs(want)))
        assert err <= TOL_ABS[dtype], (rows, cols, act, err)
    # a rank-3 tensor: the bias runs along the last dimension
    x = torch.randn(4, 50, 264, device="cuda").bfloat16()
    b = torch.randn(264, device="cuda").bfloat16()
    got = ops.fused_activation(x, None, bias=b)
    want = (x.float() + b.float()).bfloat16()
    assert torch.equal(got, want)


def test_dense_unfused_equals_fused(ops):
    # matmul without epilogue, then the standalone bias + activation pass == the fused launch, on fp32 output
    torch.manual_seed(3)
    x = torch.randn(520, 264, device="cuda").bfloat16()
    w = torch.randn(264, 392, device="cuda").bfloat16()
    b = torch.randn(392, device="cuda")
    for act in ("gelu", "relu", "mish", "sigmoid"):
        fused = ops.fused_matmul(x, w, bias=b, activation=act, out_dtype=torch.float32)
        two = ops.fused_activation(ops.fused_matmul(x, w, out_dtype=torch.float32), act, bias=b)
        assert float((fused - two).abs().max()) <= 2e-5 * (1.0 + float(fused.abs().max())), act


@pytest.mark.parametrize("dtype", ["float32", "float16", "bfloat16"])
def test_bias_grad(ops, binding, dtype):
    rng = np.random.default_rng(8)
    # the last two shapes have enough columns for the 256- and the 512-byte strip rows (ragged last strip)
    for (M, N) in ((1, 1), (5, 7), (300, 264), (4096, 1000), (1000, 64), (8192, 1032), (1024, 4100), (2048, 8200)):
        g = ref.quantize(rng.standard_normal((M, N), dtype=np.float32), dtype)
        tg = U.to_cuda(g)
        got32 = ops.bias_grad(tg, out_dtype=torch.float32)
        torch.cuda.synchronize()
        assert binding.last_kernel_name() == "bias_grad_colsum"
        want = g.astype(np.float64).sum(axis=0)
        scale = np.sqrt(M) + 1.0
        assert np.max(np.abs(got32.cpu().numpy() - want)) <= 2e-6 * M * scale / np.sqrt(M), (M, N)
        got = ops.bias_grad(tg)
        assert got.dtype == tg.dtype
        assert ref.rel_frobenius(U.to_numpy(got), want) <= ref.TOLERANCE[dtype] if dtype != "float32" else True
        assert torch.equal(ops.bias_grad(tg, out_dtype=torch.float32), got32)          # fixed summation order
    # a pitched view (row pitch > N) and leading dimensions
    big = torch.randn(6, 40, 300, device="cuda")
    view = big[:, :, :264]
    got = ops.bias_grad(view)
    assert torch.allclose(got, view.reshape(-1, 264).double().sum(0).float(), rtol=1e-5, atol=1e-4)
    lib = binding.load_library()
    out = torch.empty(8, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    assert lib.sm120_launch_bias_grad(big.data_ptr(), out.data_ptr(), 4, 8, 4, 0, 0, stream) == 1       # pitch < N
    assert lib.sm120_launch_bias_grad(big.data_ptr(), out.data_ptr(), 4, 8, 8, 0, 1, stream) == 1       # fp16 out of fp32 in
    assert lib.sm120_launch_bias_grad(None, out.data_ptr(), 0, 8, 8, 0, 0, stream) == 0                 # no rows: zeros
    torch.cuda.synchronize()
    assert float(out.abs().max()) == 0.0


def test_dense_training_step_matches_autograd(ops):
    """Forward and backward of a Dense layer through this library (fused GEMM forward; GradA, GradB and the
    bias column sum backward) against float64 autograd on the CPU: the training use of
    tests/integration/test_comprehensive_validation.py:346-434."""
    torch.manual_seed(12)
    M, K, N = 392, 264, 136
    for act in (None, "relu"):
        x = torch.randn(M, K, device="cuda", requires_grad=True)
        w = (0.1 * torch.randn(K, N, device="cuda")).requires_grad_()
        b = torch.randn(N, device="cuda", requires_grad=True)
        y = ops.dense_trainable(x, w, b, activation=act)
        loss = (y * y).sum()
        loss.backward()
        xd, wd, bd = (t.detach().double().cpu().requires_grad_() for t in (x, w, b))
        yd = xd @ wd + bd
        if act == "relu":
            yd = torch.relu(yd)
        (yd * yd).sum().backward()
        for got, want, name in ((x.grad, xd.grad, "dx"), (w.grad, wd.grad, "dw"), (b.grad, bd.grad, "db")):
            assert ref.rel_frobenius(got.cpu().numpy(), want.numpy()) <= 1e-5, (act, name)


def test_cast_fp8_with_given_scale_and_non_finite_input(ops, binding):
    rng = np.random.default_rng(2)
    x32 = 3.0 * rng.standard_normal((512, 1000), dtype=np.float32)
    # two shards of one tensor quantised with the scale of the whole: same bytes as quantising the whole
    whole_q, whole_s = ops.quantize_fp8(torch.from_numpy(x32).cuda())
    top, _ = ops.quantize_fp8(torch.from_numpy(x32[:200]).cuda(), scale=whole_s)
    bottom, s2 = ops.quantize_fp8(torch.from_numpy(x32[200:]).cuda(), scale=whole_s)
    assert s2 is whole_s and binding.last_kernel_name() == "quant_e4m3_scale_cast"
    assert torch.equal(torch.cat([top, bottom]).view(torch.uint8), whole_q.view(torch.uint8))
    want = ref.quantize(x32 * np.float32(float(whole_s)), "fp8_e4m3")
    assert np.array_equal(U.to_numpy(whole_q).view(np.uint8), want.view(np.uint8))
    # an infinity does not zero the scale: it saturates, finite values go to zero, the scale stays usable
    y = torch.tensor([1.0, -2.0, float("inf"), 0.5, float("-inf")], device="cuda")
    q, s = ops.quantize_fp8(y)
    assert float(s) > 0.0 and np.isfinite(float(s))
    assert q.float().tolist() == [0.0, -0.0, 448.0, 0.0, -448.0] or q.float().abs().tolist() == [0.0, 0.0, 448.0, 0.0, 448.0]
    # a NaN is ignored by the maximum and stays a NaN
    z = torch.tensor([1.0, float("nan"), -4.0], device="cuda")
    q, s = ops.quantize_fp8(z)
    assert float(s) == 112.0
    qf = q.float()
    assert float(qf[0]) == 112.0 and float(qf[2]) == -448.0 and bool(torch.isnan(qf[1]))


_SWEEP_ROWS = [1, 3, 17, 64, 129, 500, 1024, 3000]
_SWEEP_COLS = [1, 2, 7, 8, 33, 64, 200, 264, 1000, 1032, 4100]


@pytest.mark.parametrize("seed", range(40))
def test_companion_kernels_seeded_sweep(ops, binding, seed):
    """One of the HBM-bound companions (activation with and without bias, bias gradient, softmax along a random axis,
    FP8 quantiser) on a shape, type and argument set drawn from a seeded stream, against the float64 oracle."""
    rng = np.random.default_rng(8000 + seed)
    pick = lambda xs: xs[int(rng.integers(len(xs)))]
    op = pick(["activation", "bias_activation", "bias_grad", "softmax", "quantize"])
    dtype = pick(["float32", "float16", "bfloat16"])
    rows, cols = pick(_SWEEP_ROWS), pick(_SWEEP_COLS)
    x = ref.quantize(2.0 * rng.standard_normal((rows, cols), dtype=np.float32), dtype)
    tx = U.to_cuda(x)
    what = (op, dtype, rows, cols)
    if op in ("activation", "bias_activation"):
        code = int(rng.integers(0, 10))
        bias = None
        if op == "bias_activation":
            bias = ref.quantize(rng.standard_normal(cols, dtype=np.float32), pick([dtype, "float32"]))
        got = ops.fused_activation(tx, code, bias=None if bias is None else U.to_cuda(bias))
        want = _act_oracle(x, code, dtype, bias=bias)
        err = np.max(np.abs(U.to_numpy(got).astype(np.float64) - want) / (1.0 + np.abs(want)))
        assert got.shape == tx.shape and err <= TOL_ABS[dtype], what + (code, err)
    elif op == "bias_grad":
        got = ops.bias_grad(tx, out_dtype=torch.float32)
        want = x.astype(np.float64).sum(axis=0)
        assert np.max(np.abs(got.cpu().numpy() - want)) <= 4e-6 * (rows + np.sqrt(rows)), what
    elif op == "softmax":
        t3 = tx.reshape(rows, cols, 1).expand(rows, cols, 3).contiguous() if cols <= 264 else tx
        axis = int(rng.integers(0, t3.dim()))
        got = ops.softmax(t3, axis=axis)
        want = ref.softmax_oracle(U.to_numpy(t3), axis=axis)
        tol = {"float32": 2e-6, "float16": 6e-4, "bfloat16": 5e-3}[dtype]
        assert np.max(np.abs(U.to_numpy(got).astype(np.float64) - want)) <= tol, what + (axis,)
    else:
        q, s = ops.quantize_fp8(tx)
        x32 = x.astype(np.float32)
        want_s = np.float32(ref.fp8_scale(x32))
        assert abs(float(s) - float(want_s)) <= 1.2e-7 * float(want_s), what
        want_q = ref.quantize(x32 * np.float32(float(s)), "fp8_e4m3")          # the device's own scale: bytes must match
        assert np.array_equal(U.to_numpy(q).view(np.uint8), want_q.view(np.uint8)), what
    torch.cuda.synchronize()
