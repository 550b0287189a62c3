"""GPU parity tests: the CUDA path, called through the C ABI (ctypes, via the
package's host code), against the CPU oracle on identical seeded inputs.

Shapes, dtypes and tolerances of the first groups restate the reference's own
tests (tests/test_sm120_operations.py:47-214,
tests/integration/test_comprehensive_validation.py:145-193); the "workload" groups
use the op's five benchmark workloads (fp32 1024^3; fp16 4096^3 with B stored
[N,K]; the bf16 Dense 8192x4096 . 4096x11008 + bias + GELU; the bf16 batch of 64
attention-score products 2048x128 . 128x2048; the FP8 65536x8192x8192 product)
with relative-Frobenius gates of 1e-5 fp32, 1e-2 fp16/bf16 and 5e-2 fp8."""
import threading

import ctypes

import numpy as np
import pytest
import torch

from oracle import reference as ref
from tests import _util as U

pytestmark = pytest.mark.gpu

TOL = ref.TOLERANCE


def run(ops, a, b, *, ta=False, tb=False, bias=None, act=-1, alpha=1.0, beta=0.0, c_in=None, out_dtype=None,
        sa=None, sb=None, use_tensor_cores=None, optimization_level=None):
    """numpy operands -> CUDA -> fused_matmul -> numpy result (+ kernel name)."""
    ta_, tb_ = U.to_cuda(a), U.to_cuda(b)
    out = U.to_cuda(c_in) if c_in is not None else None
    r = ops.fused_matmul(ta_, tb_, transpose_a=ta, transpose_b=tb, bias=None if bias is None else U.to_cuda(bias),
                         activation=act, alpha=alpha, beta=beta, out=out,
                         out_dtype=None if out_dtype is None else U.torch_dtype(out_dtype), scale_a=sa, scale_b=sb,
                         use_tensor_cores=use_tensor_cores, optimization_level=optimization_level)
    torch.cuda.synchronize()
    return U.to_numpy(r)


def check(got, want, dtype_name, what=""):
    err = ref.rel_frobenius(got, want)
    assert np.isfinite(np.asarray(got).astype(np.float32)).all(), f"{what}: non-finite output"
    assert err <= TOL[dtype_name], f"{what}: rel Frobenius {err:.3e} > {TOL[dtype_name]:.0e}"
    return err


def test_device_is_supported(ops, binding):
    assert ops.is_sm120_available()
    assert binding.load_library().sm120_is_supported(0)
    info = ops.get_sm120_device_info()
    assert info["available"] and info["devices"][0]["compute_capability"][0] == 10


def test_known_answer_2x2(ops):
    # scripts/validate-installation.py:381-388
    a = np.array([[1.0, 2.0], [3.0, 4.0]], dtype=np.float32)
    b = np.array([[2.0, 0.0], [0.0, 2.0]], dtype=np.float32)
    assert run(ops, a, b).tolist() == [[2.0, 4.0], [6.0, 8.0]]


def test_golden_vectors(ops, binding):
    for name, g in U.load_golden().items():
        got = run(ops, g["a"], g["b"], ta=g["ta"], tb=g["tb"], bias=g["bias"], act=g["act"], alpha=g["alpha"],
                  beta=g["beta"], c_in=g["c_in"], out_dtype=g["out_dtype"],
                  sa=g["sa"] if g["in_dtype"] == "fp8_e4m3" else None, sb=g["sb"] if g["in_dtype"] == "fp8_e4m3" else None)
        assert got.dtype == g["c"].dtype and got.shape == g["c"].shape, name
        tol_name = g["in_dtype"] if g["in_dtype"] != "fp8_e4m3" else "bfloat16"   # vs the dequantised product: 1e-2
        check(got, g["c"], tol_name, name)
        if g["in_dtype"] != "float32":
            assert binding.last_kernel_name().startswith("tc_"), (name, binding.last_kernel_name())


# ----- the reference's own test shapes (tests/test_sm120_operations.py:47,71-72) -----
@pytest.mark.parametrize("dtype", ["float32", "float16", "bfloat16"])
@pytest.mark.parametrize("M,K", [(32, 64), (64, 32), (128, 256)])
def test_reference_shapes(ops, dtype, M, K):
    rng = np.random.default_rng(M * 131 + K)
    a = ref.quantize(0.1 * rng.standard_normal((M, K), dtype=np.float32), dtype)
    b = ref.quantize(0.1 * rng.standard_normal((K, K), dtype=np.float32), dtype)
    got = run(ops, a, b)
    want = ref.matmul_oracle(a, b, out_dtype=dtype)
    check(got, want, dtype, f"{dtype} {M}x{K}")
    # and the reference's own criterion: max|d| <= atol + rtol*max|ref| with 1e-3 (1e-2 for fp16)
    t = 1e-2 if dtype != "float32" else 1e-3
    assert ref.max_abs_tolerance_ok(got, want, rtol=t, atol=t)


@pytest.mark.parametrize("dtype", ["float32", "float16", "bfloat16"])
@pytest.mark.parametrize("ta,tb", [(False, False), (False, True), (True, False), (True, True)])
def test_transposes(ops, dtype, ta, tb):
    # tests/test_sm120_operations.py:124-145, with shapes that are valid for every combination
    M, N, K = 128, 256, 192
    rng = np.random.default_rng(11 + 2 * ta + tb)
    a, b, _, _ = U.random_operands(rng, M, N, K, 1, ta, tb, dtype, scale=0.1)
    got = run(ops, a, b, ta=ta, tb=tb)
    check(got, ref.matmul_oracle(a, b, transpose_a=ta, transpose_b=tb, out_dtype=dtype), dtype, f"{dtype} ta={ta} tb={tb}")


@pytest.mark.parametrize("level", [0, 1, 2])
def test_optimization_levels_and_tensor_core_switch(ops, binding, level):
    # tests/test_sm120_operations.py:147-173
    rng = np.random.default_rng(5)
    a, b, _, _ = U.random_operands(rng, 256, 384, 128, 1, False, False, "float16", scale=0.1)
    want = ref.matmul_oracle(a, b, out_dtype="float16")
    check(run(ops, a, b, optimization_level=level), want, "float16", f"level {level}")
    assert binding.last_kernel_name().startswith("tc_f16")
    check(run(ops, a, b, optimization_level=level, use_tensor_cores=False), want, "float16", f"level {level} simt")
    assert binding.last_kernel_name().startswith("simt_f16")


@pytest.mark.parametrize("dtype,size", [("float32", 512), ("float16", 512), ("bfloat16", 2048), ("float16", 2048)])
def test_square_sizes(ops, dtype, size):
    # tests/test_sm120_operations.py:175-198 (2048^2) and :479-516 (512..4096)
    rng = np.random.default_rng(size)
    a, b, _, _ = U.random_operands(rng, size, size, size, 1, False, False, dtype, scale=0.1)
    check(run(ops, a, b), ref.matmul_oracle(a, b, out_dtype=dtype), dtype, f"{dtype} {size}^2")


def test_batch_flattened_projection(ops):
    # tests/integration/test_comprehensive_validation.py:145-184: A[batch,512,768] . B[768,256], f32 and f16
    for dtype in ("float32", "float16"):
        rng = np.random.default_rng(9)
        a = ref.quantize(0.1 * rng.standard_normal((4, 512, 768), dtype=np.float32), dtype)
        b = ref.quantize(0.1 * rng.standard_normal((768, 256), dtype=np.float32), dtype)
        want = ref.matmul_oracle(a, b, out_dtype=dtype)
        got3 = run(ops, a, b)                                   # rank-3 A, B broadcast over the batch
        got2 = run(ops, a.reshape(-1, 768), b).reshape(4, 512, 256)
        check(got3, want, dtype, f"{dtype} batched-broadcast")
        check(got2, want, dtype, f"{dtype} flattened")
        assert np.array_equal(got3.view(np.uint8), got2.view(np.uint8))


# ----- edge shapes: every extent off the tile grid, operands TMA cannot describe -----
EDGE = [1, 7, 16, 17, 127, 129, 255]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16", "float16"])
def test_edge_shapes(ops, binding, dtype):
    rng = np.random.default_rng(21)
    seen = set()
    for M in EDGE:
        for N, K in ((1, 129), (7, 16), (16, 7), (17, 255), (127, 1), (129, 17), (255, 127), (264, 72), (136, 4104)):
            for ta, tb in ((False, False), (False, True), (True, False)):
                a, b, _, _ = U.random_operands(rng, M, N, K, 1, ta, tb, dtype, scale=0.25)
                got = run(ops, a, b, ta=ta, tb=tb)
                check(got, ref.matmul_oracle(a, b, transpose_a=ta, transpose_b=tb, out_dtype=dtype), dtype,
                      f"{dtype} M={M} N={N} K={K} ta={ta} tb={tb}")
                seen.add(binding.last_kernel_name().split("_")[0])
    if dtype != "float32":
        assert seen == {"tc", "simt"}     # aligned shapes ran on tensor cores, the rest on the SIMT kernel


def test_ragged_tensor_core_tiles(ops, binding):
    # extents that are multiples of 8 (so TMA applies) but of no tile size: M, N, K tails are zero-filled by TMA
    rng = np.random.default_rng(33)
    for (M, N, K) in ((136, 264, 72), (8, 8, 8), (120, 1000, 40), (392, 136, 520), (1, 512, 64)):
        for tb in (False, True):
            a, b, _, _ = U.random_operands(rng, M, N, K, 1, False, tb, "bfloat16", scale=0.25)
            got = run(ops, a, b, tb=tb)
            assert binding.last_kernel_name().startswith("tc_bf16"), binding.last_kernel_name()
            check(got, ref.matmul_oracle(a, b, transpose_b=tb, out_dtype="bfloat16"), "bfloat16", f"{M}x{N}x{K} tb={tb}")


def test_guard_bands_are_untouched(ops):
    # C with a pitch wider than N and spare rows: everything outside [M, N] must keep its sentinel
    rng = np.random.default_rng(4)
    for dtype, (M, N, K) in (("bfloat16", (200, 328, 136)), ("float32", (77, 90, 33))):
        a, b, _, _ = U.random_operands(rng, M, N, K, 1, False, False, dtype)
        ta_, tb_ = U.to_cuda(a), U.to_cuda(b)
        pitch, rows = N + 24, M + 5
        big = torch.full((rows, pitch), 512.0, dtype=U.torch_dtype(dtype), device="cuda")
        view = big[:M, :N]
        ops.fused_matmul(ta_, tb_, out=view)
        torch.cuda.synchronize()
        host = U.to_numpy(big).astype(np.float32)
        check(host[:M, :N], ref.matmul_oracle(a, b, out_dtype=dtype), dtype, f"{dtype} guarded")
        assert (host[M:, :] == 512.0).all() and (host[:, N:] == 512.0).all()


# ----- epilogue -----
@pytest.mark.parametrize("act", list(range(-1, 10)))
def test_activations_fused(ops, act):
    rng = np.random.default_rng(100 + act)
    M, N, K = 160, 192, 64
    a, b, _, _ = U.random_operands(rng, M, N, K, 1, False, False, "bfloat16", scale=0.3)
    bias = rng.standard_normal((N,), dtype=np.float32)
    want = ref.matmul_oracle(a, b, bias=bias, act=act, out_dtype="float32")
    got_tc = run(ops, a, b, bias=bias, act=act, out_dtype="float32")
    got_simt = run(ops, a, b, bias=bias, act=act, out_dtype="float32", use_tensor_cores=False)
    assert ref.rel_frobenius(got_tc, want) <= 2e-5, act      # fp32 out of exact bf16 products: only fp32 rounding
    assert ref.rel_frobenius(got_simt, want) <= 2e-5, act
    assert ref.max_abs_tolerance_ok(got_tc, want, rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("bias_dtype", ["float32", "float16", "bfloat16"])
@pytest.mark.parametrize("out_dtype", ["float32", "float16", "bfloat16"])
def test_bias_and_output_dtypes(ops, bias_dtype, out_dtype):
    rng = np.random.default_rng(17)
    M, N, K = 130, 200, 96
    a, b, _, _ = U.random_operands(rng, M, N, K, 1, False, True, "float16", scale=0.2)
    bias = ref.quantize(rng.standard_normal((N,), dtype=np.float32), bias_dtype)
    got = run(ops, a, b, tb=True, bias=bias, act=0, out_dtype=out_dtype)
    want = ref.matmul_oracle(a, b, transpose_b=True, bias=bias, act=0, out_dtype=out_dtype)
    check(got, want, "float16" if out_dtype == "float32" else out_dtype, f"bias {bias_dtype} out {out_dtype}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_alpha_beta(ops, dtype):
    # src/cuda_kernels/sm120_pure_kernels.cu:58-63
    rng = np.random.default_rng(8)
    M, N, K = 96, 136, 64
    a, b, _, _ = U.random_operands(rng, M, N, K, 1, False, False, dtype, scale=0.3)
    c0 = ref.quantize(rng.standard_normal((M, N), dtype=np.float32), dtype)
    got = run(ops, a, b, alpha=0.5, beta=2.0, c_in=c0)
    check(got, ref.matmul_oracle(a, b, alpha=0.5, beta=2.0, c_in=c0, out_dtype=dtype), dtype, f"{dtype} alpha/beta")
    # beta == 0 never reads C: a NaN-filled output buffer is simply overwritten
    nan_c = np.full((M, N), np.nan, dtype=np.float32).astype(ref.NP_DTYPES[dtype])
    got = run(ops, a, b, alpha=1.0, beta=0.0, c_in=nan_c)
    check(got, ref.matmul_oracle(a, b, out_dtype=dtype), dtype, f"{dtype} beta=0")


# ----- strided batch (src/cuda_kernels/sm120_dynamic_shapes.cu:107-183) -----
@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
def test_strided_batch(ops, dtype):
    rng = np.random.default_rng(12)
    batch, M, N, K = 5, 136, 264, 128
    for ta, tb in ((False, False), (False, True), (True, False)):
        a, b, _, _ = U.random_operands(rng, M, N, K, batch, ta, tb, dtype, scale=0.3)
        got = run(ops, a, b, ta=ta, tb=tb)
        check(got, ref.matmul_oracle(a, b, transpose_a=ta, transpose_b=tb, out_dtype=dtype), dtype, f"{dtype} batch ta={ta} tb={tb}")
    # padded batch stride and pitch on A; B broadcast (stride 0)
    a_full = torch.zeros(batch, M + 8, K + 16, dtype=U.torch_dtype(dtype), device="cuda")
    a_np, b_np, _, _ = U.random_operands(rng, M, N, K, batch, False, False, dtype, scale=0.3)
    a_full[:, :M, :K] = U.to_cuda(a_np)
    got = U.to_numpy(ops.fused_matmul(a_full[:, :M, :K], U.to_cuda(b_np[0])))
    check(got, ref.matmul_oracle(a_np, b_np[0], out_dtype=dtype), dtype, f"{dtype} strided A, broadcast B")


# ----- FP8 -----
def test_fp8_scaled(ops, binding):
    rng = np.random.default_rng(40)
    M, N, K = 256, 384, 512
    a32 = rng.standard_normal((M, K), dtype=np.float32)
    b32 = rng.standard_normal((N, K), dtype=np.float32)
    sa, sb = float(np.float32(ref.fp8_scale(a32))), float(np.float32(ref.fp8_scale(b32)))
    a, b = ref.quantize(a32 * np.float32(sa), "fp8_e4m3"), ref.quantize(b32 * np.float32(sb), "fp8_e4m3")
    want_deq = ref.matmul_oracle(a, b, transpose_b=True, scale_a=sa, scale_b=sb, out_dtype="bfloat16")
    want_true = ref.matmul_oracle(a32, b32, transpose_b=True, round_output=False)
    got = run(ops, a, b, tb=True, sa=sa, sb=sb)
    assert binding.last_kernel_name().startswith("tc_e4m3")
    assert got.dtype == ref.NP_DTYPES["bfloat16"]
    assert ref.rel_frobenius(got, want_deq) <= 1e-2          # kernel error alone
    assert ref.rel_frobenius(got, want_true) <= TOL["fp8_e4m3"]   # the FP8 gate: against the unquantised product
    # scales supplied as device scalars give the same bits
    r2 = ops.fused_matmul(U.to_cuda(a), U.to_cuda(b), transpose_b=True,
                          scale_a=torch.tensor([sa], device="cuda"), scale_b=torch.tensor([sb], device="cuda"))
    assert ref.rel_frobenius(U.to_numpy(r2), got) <= 1e-2
    # the helper quantiser agrees with the oracle's
    q, s = ops.quantize_fp8(torch.from_numpy(a32).cuda())
    assert abs(float(s) - sa) / sa < 1e-6
    assert np.mean(U.to_numpy(q).view(np.uint8) == a.view(np.uint8)) > 0.999
    # SIMT path on the same FP8 operands
    got_simt = run(ops, a, b, tb=True, sa=sa, sb=sb, use_tensor_cores=False)
    assert ref.rel_frobenius(got_simt, want_deq) <= 1e-2


@pytest.mark.parametrize("ta,tb", [(False, False), (False, True), (True, False), (True, True)])
def test_fp8_all_operand_layouts(ops, binding, ta, tb):
    # an FP8 operand whose M or N is contiguous (A stored [K,M], B stored [K,N]) is loaded in 128-byte
    # boxes of M/N and multiplied through the MN-major descriptor mode: every pairing against float64
    rng = np.random.default_rng(300 + 2 * ta + tb)
    for (M, N, K) in ((256, 384, 512), (144, 272, 400)):          # on the tile grid, and ragged in M, N and K
        a, b, sa, sb = U.random_operands(rng, M, N, K, 1, ta, tb, "fp8_e4m3")
        want = ref.matmul_oracle(a, b, transpose_a=ta, transpose_b=tb, scale_a=sa, scale_b=sb, out_dtype="bfloat16")
        got = run(ops, a, b, ta=ta, tb=tb, sa=sa, sb=sb)
        assert binding.last_kernel_name().startswith("tc_e4m3"), binding.last_kernel_name()
        assert ref.rel_frobenius(got, want) <= 1e-2, (M, N, K, ta, tb)
        simt = run(ops, a, b, ta=ta, tb=tb, sa=sa, sb=sb, use_tensor_cores=False)
        assert ref.rel_frobenius(simt, want) <= 1e-2
        assert ref.rel_frobenius(got, simt) <= 1e-2


@pytest.mark.parametrize("ta,tb", [(False, False), (True, False), (True, True)])
def test_fp8_mn_major_on_pair_tiles_with_split_tail(ops, binding, ta, tb):
    # the CTA-pair kernel on FP8 operands stored with M / N contiguous: K > 1024 keeps the 8-warp variant, whose
    # short last wave is cut into half-width tiles (each CTA then multiplies 64 of the 128 N-bytes of a swizzle atom)
    torch.manual_seed(31)
    M, N, K = 2304, 2560 + 128, 1152                  # 9 x 11 = 99 pair tiles on 74 clusters: 25 tiles in the last wave
    a32 = torch.randn((K, M) if ta else (M, K), device="cuda")
    b32 = torch.randn((N, K) if tb else (K, N), device="cuda")
    qa, sa = ops.quantize_fp8(a32)
    qb, sb = ops.quantize_fp8(b32)
    kw = dict(transpose_a=ta, transpose_b=tb, scale_a=sa, scale_b=sb)
    got = ops.fused_matmul(qa, qb, tuning=binding.TUNE_CTA_GROUP_2 | binding.TUNE_EPI_WARPS_8, **kw)
    assert binding.last_kernel_name() == "tc_e4m3_2cta_256x256x128_s6"
    whole = ops.fused_matmul(qa, qb, tuning=binding.TUNE_CTA_GROUP_2 | binding.TUNE_EPI_WARPS_8 | binding.TUNE_NO_SPLIT_TAIL, **kw)
    assert torch.equal(got, whole)                    # half-width tiles change the schedule, not the sums
    simt = ops.fused_matmul(qa, qb, use_tensor_cores=False, **kw)
    assert binding.last_kernel_name().startswith("simt_e4m3")
    diff = (got.float() - simt.float()).abs().max().item()
    assert diff <= 2.0 ** -6 * simt.float().abs().max().item(), diff       # whole matrix: at most a couple of bf16 ulps
    rows = torch.randint(0, M, (24,), device="cuda")
    A = (qa.float().double().T if ta else qa.float().double())[rows].cpu().numpy()
    B = qb.float().double().cpu().numpy()
    want = (A @ (B.T if tb else B)) / (float(sa) * float(sb))
    assert ref.rel_frobenius(got[rows].float().cpu().numpy(), want) <= 1e-2


# ----- the benchmark workloads at oracle-friendly size -----
@pytest.mark.parametrize("idx,shrink", [(1, 1), (2, 4), (3, 8), (4, 4), (5, 16)])
def test_baseline_configs_reduced(ops, idx, shrink):
    cfg = ref.make_config(idx, shrink)
    fp8 = cfg["in_dtype"] == "fp8_e4m3"
    got = run(ops, cfg["a"], cfg["b"], ta=cfg["transpose_a"], tb=cfg["transpose_b"], bias=cfg["bias"], act=cfg["act"],
              out_dtype=cfg["out_dtype"], sa=cfg["scale_a"] if fp8 else None, sb=cfg["scale_b"] if fp8 else None)
    want = ref.oracle_for_config(cfg)
    if fp8:
        assert ref.rel_frobenius(got, want) <= 1e-2
        exact = ref.matmul_oracle(cfg["a_unquantized"], cfg["b_unquantized"], transpose_b=True, round_output=False)
        check(got, exact, "fp8_e4m3", cfg["name"])
    else:
        check(got, want, cfg["in_dtype"], cfg["name"])


def _sampled_rows_check(ops, a_t, b_t, got_t, rows, *, tb, bias_t=None, act=-1, inv_scale=1.0, tol=1e-2):
    """Full-size parity without a full-size CPU product: the oracle recomputes a sample of rows."""
    a_rows = U.to_numpy(a_t[rows]).astype(np.float64)
    b_np = U.to_numpy(b_t).astype(np.float64)
    acc = a_rows @ (b_np.T if tb else b_np)
    v = acc * inv_scale
    if bias_t is not None:
        v = v + U.to_numpy(bias_t).astype(np.float64)
    v = ref.activation(v, act)
    return ref.rel_frobenius(U.to_numpy(got_t[rows]), v) <= tol


def _whole_matrix_vs_simt(ops, binding, a, b, got, **kw):
    """Every element of a tensor-core result against the SIMT kernel's (itself oracle-tested): a wrong tile
    anywhere would show as a large difference, which row samples and run-to-run equality cannot see."""
    simt = ops.fused_matmul(a, b, use_tensor_cores=False, **kw)
    assert binding.last_kernel_name().startswith("simt_")
    scale = simt.float().abs().max().item()
    diff = (got.float() - simt.float()).abs().max().item()
    assert diff <= 2.0 ** -6 * scale, (diff, scale)           # 16-bit outputs: a couple of ulps of the largest value
    return diff


def test_baseline_config2_full_size(ops, binding):
    torch.manual_seed(1)
    n = 4096
    a = (torch.randn(n, n, device="cuda") / 64).half()
    b = (torch.randn(n, n, device="cuda") / 64).half()          # stored [N, K]
    c = ops.advanced_matmul(a, b, transpose_b=True)
    assert binding.last_kernel_name().startswith("tc_f16")
    rows = torch.randint(0, n, (48,), device="cuda")
    assert _sampled_rows_check(ops, a, b, c, rows, tb=True)
    # linearity in A: (2A) B == 2 (A B) bit for bit when the fp32 accumulator is written out unrounded
    c32 = ops.fused_matmul(a, b, transpose_b=True, out_dtype=torch.float32)
    c32x2 = ops.fused_matmul(a * 2, b, transpose_b=True, out_dtype=torch.float32)
    assert torch.equal(c32x2, c32 * 2)
    assert torch.equal(c32.half(), c)
    # run-to-run determinism (DEPLOYMENT_GUIDE.md:498-519)
    assert torch.equal(ops.advanced_matmul(a, b, transpose_b=True), c)
    _whole_matrix_vs_simt(ops, binding, a, b, c, transpose_b=True)
    # same shape in bf16 (the headline size)
    cb = ops.advanced_matmul(a.bfloat16(), b.bfloat16(), transpose_b=True)
    assert _sampled_rows_check(ops, a.bfloat16(), b.bfloat16(), cb, rows, tb=True)


def test_baseline_config3_full_size(ops, binding):
    torch.manual_seed(2)
    x = torch.randn(8192, 4096, device="cuda").bfloat16()
    w = (0.02 * torch.randn(4096, 11008, device="cuda")).bfloat16()
    bias = (0.02 * torch.randn(11008, device="cuda")).bfloat16()
    y = ops.fused_matmul(x, w, bias=bias, activation="gelu")
    assert binding.last_kernel_name().startswith("tc_bf16") and tuple(y.shape) == (8192, 11008)
    rows = torch.randint(0, 8192, (32,), device="cuda")
    assert _sampled_rows_check(ops, x, w, y, rows, tb=False, bias_t=bias, act=9)
    assert torch.equal(ops.fused_matmul(x, w, bias=bias, activation="gelu"), y)
    _whole_matrix_vs_simt(ops, binding, x, w, y, bias=bias, activation="gelu")


def test_baseline_config4_full_size(ops, binding):
    torch.manual_seed(3)
    q = torch.randn(64, 2048, 128, device="cuda").bfloat16()
    k = torch.randn(64, 128, 2048, device="cuda").bfloat16()
    s = ops.batched_matmul(q, k)
    assert tuple(s.shape) == (64, 2048, 2048)
    for bz in (0, 31, 63):
        rows = torch.randint(0, 2048, (16,), device="cuda")
        assert _sampled_rows_check(ops, q[bz], k[bz], s[bz], rows, tb=False)
    assert torch.equal(ops.batched_matmul(q, k), s)
    _whole_matrix_vs_simt(ops, binding, q, k, s)


def test_baseline_config5_slab(ops, binding):
    # one rank's slab of the 8-way M-sharded FP8 config: 8192 x 8192 x 8192
    torch.manual_seed(4)
    a32 = torch.randn(8192, 8192, device="cuda")
    b32 = torch.randn(8192, 8192, device="cuda")
    qa, sa = ops.quantize_fp8(a32)
    qb, sb = ops.quantize_fp8(b32)
    c = ops.fused_matmul(qa, qb, transpose_b=True, scale_a=sa, scale_b=sb)
    assert binding.last_kernel_name().startswith("tc_e4m3") and c.dtype == torch.bfloat16
    rows = torch.randint(0, 8192, (32,), device="cuda")
    inv = 1.0 / (float(sa) * float(sb))
    assert _sampled_rows_check(ops, qa, qb, c, rows, tb=True, inv_scale=inv, tol=1e-2)
    # the FP8 gate against the unquantised product on the sampled rows
    exact = a32[rows].double() @ b32.double().T
    assert ref.rel_frobenius(U.to_numpy(c[rows]), exact.cpu().numpy()) <= TOL["fp8_e4m3"]


def test_baseline_config5_full_size_one_gpu(ops, binding):
    # the whole FP8 workload, M = 65536, N = K = 8192, on one GPU (1.7 GB): 256 x 32 pair tiles, more row tiles
    # and raster groups than any slab has
    torch.manual_seed(4)
    M, N, K, G = 65536, 8192, 8192, 8
    b32 = torch.randn(N, K, device="cuda")
    qb, sb = ops.quantize_fp8(b32)
    qa = torch.empty(M, K, dtype=torch.float8_e4m3fn, device="cuda")
    # one scale for the whole A, from its global amax, as every rank of the sharded run would use
    amax = torch.zeros((), device="cuda")
    slabs = []
    gen = torch.Generator(device="cuda")
    for r in range(G):
        gen.manual_seed(1000 + r)
        a32 = torch.randn(M // G, K, device="cuda", generator=gen)
        amax = torch.maximum(amax, a32.abs().max())
    sa = (448.0 / amax).reshape(1).float()
    for r in range(G):
        gen.manual_seed(1000 + r)
        a32 = torch.randn(M // G, K, device="cuda", generator=gen)
        qa[r * (M // G):(r + 1) * (M // G)] = (a32 * sa).clamp_(-448, 448).to(torch.float8_e4m3fn)
        if r in (0, G - 1):
            slabs.append((r, a32))
    c = ops.fused_matmul(qa, qb, transpose_b=True, scale_a=sa, scale_b=sb)
    assert binding.last_kernel_name().startswith("tc_e4m3_2cta") and tuple(c.shape) == (M, N) and c.dtype == torch.bfloat16
    # float64 oracle on one row of every 128-row tile
    rows = torch.arange(0, M, 128, device="cuda") + torch.randint(0, 128, (M // 128,), device="cuda")
    inv = 1.0 / (float(sa) * float(sb))
    assert _sampled_rows_check(ops, qa, qb, c, rows, tb=True, inv_scale=inv, tol=1e-2)
    # the gate against the unquantised product, on the rows of the first and the last slab
    for r, a32 in slabs:
        rr = torch.randint(0, M // G, (16,), device="cuda")
        exact = a32[rr].double() @ b32.double().T
        assert ref.rel_frobenius(U.to_numpy(c[r * (M // G) + rr]), exact.cpu().numpy()) <= TOL["fp8_e4m3"]
    # the eight slab launches of the M-sharded run produce the same bits
    for r in range(G):
        lo, hi = r * (M // G), (r + 1) * (M // G)
        assert torch.equal(ops.fused_matmul(qa[lo:hi], qb, transpose_b=True, scale_a=sa, scale_b=sb), c[lo:hi]), r
    assert torch.equal(ops.fused_matmul(qa, qb, transpose_b=True, scale_a=sa, scale_b=sb), c)


@pytest.mark.parametrize("dtype", ["float16", "bfloat16"])
@pytest.mark.parametrize("ta,tb", [(False, False), (False, True), (True, False), (True, True)])
def test_split_k_matches_oracle(ops, binding, dtype, ta, tb):
    """Few output tiles and a long K: the launcher cuts K into parts that run as one launch into fp32 workspace and
    a second kernel adds them in a fixed order (with alpha, beta, bias, activation).  Every operand layout, a ragged
    M and N, skinny M; the result against the oracle, against the unsplit launch, and run to run."""
    rng = np.random.default_rng(70 + 2 * ta + tb)
    for (M, N, K) in ((296, 520, 4096), (128, 1024, 2048), (1000, 264, 8192)):
        a = ref.quantize(rng.standard_normal((K, M) if ta else (M, K), dtype=np.float32), dtype)
        b = ref.quantize(0.05 * rng.standard_normal((N, K) if tb else (K, N), dtype=np.float32), dtype)
        bias = rng.standard_normal(N).astype(np.float32)
        c_in = ref.quantize(rng.standard_normal((M, N), dtype=np.float32), dtype)
        kw = dict(ta=ta, tb=tb, bias=bias, act=0, alpha=0.5, beta=0.25)          # 0 = relu
        got = run(ops, a, b, c_in=c_in.copy(), **kw)
        assert binding.last_split_k() >= 2, (M, N, K, binding.last_kernel_name())
        want = ref.matmul_oracle(a, b, transpose_a=ta, transpose_b=tb, alpha=0.5, beta=0.25, c_in=c_in, bias=bias, act=kw["act"],
                                 out_dtype=dtype)
        check(got, want, dtype, f"split-K {M}x{N}x{K}")
        again = run(ops, a, b, c_in=c_in.copy(), **kw)
        assert np.array_equal(got.view(np.uint16), again.view(np.uint16))
        # the unsplit launch of the same product (switched off per call) agrees within the output rounding
        r = ops.fused_matmul(U.to_cuda(a), U.to_cuda(b), transpose_a=ta, transpose_b=tb, bias=U.to_cuda(bias), activation=kw["act"],
                             alpha=0.5, beta=0.25, out=U.to_cuda(c_in.copy()), tuning=binding.TUNE_NO_SPLIT_K)
        torch.cuda.synchronize()
        assert binding.last_split_k() == 1
        assert ref.rel_frobenius(U.to_numpy(r), got) <= TOL[dtype]


def test_split_k_fp8_and_when_it_is_not_used(ops, binding):
    rng = np.random.default_rng(80)
    M, N, K = 256, 512, 8192
    a32 = rng.standard_normal((M, K), dtype=np.float32)
    b32 = rng.standard_normal((N, K), dtype=np.float32)
    sa, sb = float(np.float32(ref.fp8_scale(a32))), float(np.float32(ref.fp8_scale(b32)))
    a, b = ref.quantize(a32 * np.float32(sa), "fp8_e4m3"), ref.quantize(b32 * np.float32(sb), "fp8_e4m3")
    want = ref.matmul_oracle(a, b, transpose_b=True, scale_a=sa, scale_b=sb, out_dtype="bfloat16")
    got = run(ops, a, b, tb=True, sa=sa, sb=sb)
    assert binding.last_split_k() >= 2 and binding.last_kernel_name().startswith("tc_e4m3")
    assert ref.rel_frobenius(got, want) <= 1e-2
    r2 = ops.fused_matmul(U.to_cuda(a), U.to_cuda(b), transpose_b=True,
                          scale_a=torch.tensor([sa], device="cuda"), scale_b=torch.tensor([sb], device="cuda"))
    torch.cuda.synchronize()
    assert binding.last_split_k() >= 2 and ref.rel_frobenius(U.to_numpy(r2), want) <= 1e-2
    # a width that neither TMA stores nor 16-byte loads can use (N % 4 != 0): the general epilogue writes the partial sums,
    # the element-wise form of the second kernel adds them; fp32 output
    a16 = ref.quantize(rng.standard_normal((200, 4096), dtype=np.float32), "float16")
    b16 = ref.quantize(0.05 * rng.standard_normal((262, 4096), dtype=np.float32), "float16")
    got32 = run(ops, a16, b16, tb=True, out_dtype="float32")
    assert binding.last_split_k() >= 2
    assert ref.rel_frobenius(got32, ref.matmul_oracle(a16, b16, transpose_b=True, round_output=False)) <= 1e-3
    # enough tiles, a short K, or a batch: one launch as before
    for shape in ((4096, 4096, 4096), (256, 512, 512)):
        x = torch.randn(shape[0], shape[2], device="cuda", dtype=torch.bfloat16)
        w = torch.randn(shape[2], shape[1], device="cuda", dtype=torch.bfloat16)
        ops.fused_matmul(x, w)
        assert binding.last_split_k() == 1, shape
    xb = torch.randn(2, 256, 4096, device="cuda", dtype=torch.bfloat16)
    wb = torch.randn(2, 4096, 256, device="cuda", dtype=torch.bfloat16)
    ops.fused_matmul(xb, wb)
    assert binding.last_split_k() == 1
    # through the C ABI without workspace (the reference-signature entry point carries none): unsplit
    lib = binding.load_library()
    x = torch.randn(256, 8192, device="cuda", dtype=torch.float16)
    w = torch.randn(8192, 512, device="cuda", dtype=torch.float16)
    c = torch.empty(256, 512, device="cuda", dtype=torch.float16)
    assert lib.sm120_launch_matmul(x.data_ptr(), w.data_ptr(), c.data_ptr(), 256, 512, 8192, 1.0, 0.0, 1,
                                   torch.cuda.current_stream().cuda_stream) == 0
    torch.cuda.synchronize()
    assert binding.last_split_k() == 1
    assert ref.rel_frobenius(c.float().cpu().numpy(), (x.float() @ w.float()).cpu().numpy()) <= 1e-2


def test_determinism_small_and_ragged(ops):
    rng = np.random.default_rng(77)
    for dtype, shape in (("bfloat16", (392, 520, 264)), ("float32", (300, 200, 100))):
        a, b, _, _ = U.random_operands(rng, *shape, 1, False, False, dtype)
        r1, r2 = run(ops, a, b), run(ops, a, b)
        assert np.array_equal(r1.view(np.uint8), r2.view(np.uint8))


# ----- the C entry points with the reference's own signatures -----
def test_reference_signature_entry_points(binding):
    lib = binding.load_library()
    rng = np.random.default_rng(55)
    M, N, K = 96, 72, 40
    stream = torch.cuda.current_stream().cuda_stream
    for dtype, code in (("float32", 0), ("float16", 1), ("bfloat16", 2)):
        a, b, _, _ = U.random_operands(rng, M, N, K, 1, False, False, dtype, scale=0.3)
        c0 = ref.quantize(rng.standard_normal((M, N), dtype=np.float32), dtype)
        ta_, tb_, tc_ = U.to_cuda(a), U.to_cuda(b), U.to_cuda(c0)
        rc = lib.sm120_launch_matmul(ta_.data_ptr(), tb_.data_ptr(), tc_.data_ptr(), M, N, K, 1.5, 0.5, code, stream)
        assert rc == 0
        torch.cuda.synchronize()
        check(U.to_numpy(tc_), ref.matmul_oracle(a, b, alpha=1.5, beta=0.5, c_in=c0, out_dtype=dtype), dtype, f"launch_matmul {dtype}")
    # launch_sm120_matmul: fp32, void return (src/cuda_kernels/sm120_optimized_kernels_fixed.cu:788-798)
    a, b, _, _ = U.random_operands(rng, M, N, K, 1, False, False, "float32")
    ta_, tb_ = U.to_cuda(a), U.to_cuda(b)
    out = torch.empty(M, N, device="cuda")
    lib.launch_sm120_matmul(ta_.data_ptr(), tb_.data_ptr(), out.data_ptr(), M, N, K, stream)
    torch.cuda.synchronize()
    check(U.to_numpy(out), ref.matmul_oracle(a, b), "float32", "launch_sm120_matmul")


@pytest.mark.parametrize("dtype,code", [("float32", 0), ("bfloat16", 2)])
def test_gradient_entry_points(binding, ops, dtype, code):
    # dA = dC . B^T, dB = A^T . dC (src/tensorflow_ops/sm120_gradients.cc:22-55)
    lib = binding.load_library()
    rng = np.random.default_rng(66)
    M, N, K = 136, 264, 72
    a, b, _, _ = U.random_operands(rng, M, N, K, 1, False, False, dtype, scale=0.3)
    g = ref.quantize(0.3 * rng.standard_normal((M, N), dtype=np.float32), dtype)
    ta_, tb_, tg_ = U.to_cuda(a), U.to_cuda(b), U.to_cuda(g)
    da = torch.empty(M, K, dtype=ta_.dtype, device="cuda")
    db = torch.empty(K, N, dtype=ta_.dtype, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    assert lib.sm120_launch_matmul_grad_a(tg_.data_ptr(), tb_.data_ptr(), da.data_ptr(), M, N, K, 1.0, code, stream) == 0
    assert lib.sm120_launch_matmul_grad_b(ta_.data_ptr(), tg_.data_ptr(), db.data_ptr(), M, N, K, 1.0, code, stream) == 0
    torch.cuda.synchronize()
    check(U.to_numpy(da), ref.matmul_oracle(g, b, transpose_b=True, out_dtype=dtype), dtype, "grad_a")
    check(U.to_numpy(db), ref.matmul_oracle(a, g, transpose_a=True, out_dtype=dtype), dtype, "grad_b")
    ga, gb = ops.matmul_grad(tg_, ta_, tb_)
    assert torch.equal(ga, da) and torch.equal(gb, db)


# ----- the layer and the host-array path -----
def test_dense_layer_forward(pkg):
    layers, ops = pkg.sm120_keras_layers, pkg.sm120_ops
    for act in (None, "relu", "gelu", "tanh"):
        layer = layers.SM120Dense(264, activation=act, dtype="bfloat16")
        x = torch.randn(4, 50, 136, device="cuda").bfloat16()      # rank-3 input is flattened and restored
        layer.build(tuple(x.shape), seed=1)
        layer.set_weights([layer.kernel, (0.1 * torch.randn(264, device="cuda")).bfloat16()])
        y = layer(x)
        assert tuple(y.shape) == (4, 50, 264) and y.dtype == torch.bfloat16
        want = ref.matmul_oracle(U.to_numpy(x).reshape(-1, 136), U.to_numpy(layer.kernel), bias=U.to_numpy(layer.bias),
                                 act=ops.activation_code(act), out_dtype="bfloat16").reshape(4, 50, 264)
        check(U.to_numpy(y), want, "bfloat16", f"SM120Dense {act}")
    # a callable activation is applied after the fused matmul + bias
    layer = layers.SM120Dense(64, activation=torch.sigmoid, dtype="float32")
    x = torch.randn(32, 48, device="cuda")
    y = layer(x)
    want = ref.matmul_oracle(U.to_numpy(x), U.to_numpy(layer.kernel), bias=U.to_numpy(layer.bias), act=8)
    check(U.to_numpy(y), want, "float32", "SM120Dense callable")
    out = ops.optimized_dense(torch.randn(8, 16, 32, device="cuda"), 24, activation="relu")
    assert tuple(out.shape) == (8, 16, 24) and float(out.min()) >= 0.0


def test_host_arrays_round_trip(ops):
    rng = np.random.default_rng(91)
    for dtype in ("float32", "bfloat16"):
        a, b, _, _ = U.random_operands(rng, 200, 136, 72, 1, False, False, dtype, scale=0.3)
        got = ops.advanced_matmul(a, b)                       # numpy in -> numpy out
        assert isinstance(got, np.ndarray) and got.dtype == a.dtype
        check(got, ref.matmul_oracle(a, b, out_dtype=dtype), dtype, f"host {dtype}")
    a = torch.randn(64, 32)
    got = ops.advanced_matmul(a, torch.randn(32, 16))         # CPU tensors in -> CPU tensor out
    assert isinstance(got, torch.Tensor) and not got.is_cuda


def test_host_operands_pipelined_chunks(ops, binding):
    """Host operands large enough for the chunked pipeline (copies in, products and copies out overlap chunk by
    chunk), with a ragged row count, a bias and an activation, pinned and pageable buffers, against the oracle."""
    rng = np.random.default_rng(92)
    for (M, N, K, tb, dtype) in ((1300, 520, 264, True, "bfloat16"), (2048 + 77, 392, 136, False, "float16"), (600, 264, 72, False, "float32")):
        a, b, _, _ = U.random_operands(rng, M, N, K, 1, False, tb, dtype, scale=0.3)
        bias = ref.quantize(rng.standard_normal((N,), dtype=np.float32), "float32")
        want = ref.matmul_oracle(a, b, transpose_b=tb, bias=bias, act=0, out_dtype=dtype)
        assert len(ops._HostPipeline.chunk_rows(M)) >= 2
        got = ops.fused_matmul(a, b, transpose_b=tb, bias=bias, activation="relu")            # numpy in, numpy out
        assert isinstance(got, np.ndarray) and got.shape == (M, N)
        check(got, want, dtype, f"host pipeline {dtype} M={M}")
        # pinned torch buffers in, pinned result buffer out; the same bits as the one-shot device product
        ta = torch.empty(a.shape, dtype=U.torch_dtype(dtype), pin_memory=True).copy_(U.to_cuda(a).cpu())
        tb_ = torch.empty(b.shape, dtype=U.torch_dtype(dtype), pin_memory=True).copy_(U.to_cuda(b).cpu())
        out = torch.empty((M, N), dtype=U.torch_dtype(dtype), pin_memory=True)
        res = ops.fused_matmul(ta, tb_, transpose_b=tb, bias=torch.from_numpy(bias), activation="relu", out=out)
        assert res is out
        dev = ops.fused_matmul(U.to_cuda(a), U.to_cuda(b), transpose_b=tb, bias=torch.from_numpy(bias).cuda(), activation="relu")
        if dtype != "float32":          # (fp32 rows may take the tensor-core or the FFMA kernel depending on the chunk's size)
            assert torch.equal(out, dev.cpu())
        check(U.to_numpy(out), want, dtype, f"host pipeline pinned {dtype}")


def test_kernel_status_is_clean(binding):
    status = ctypes.c_uint(123)
    assert binding.load_library().sm120_get_kernel_status(0, ctypes.byref(status), 0) == 0
    assert status.value == 0


# ----- FP32 on the tensor cores (3xTF32 split with run-wise promotion) -----
def test_fp32_tensor_core_path(ops, binding):
    rng = np.random.default_rng(123)
    for (M, N, K, batch, ta, tb) in ((1024, 1024, 1024, 1, False, False), (520, 776, 1000, 1, True, False),
                                     (1000, 520, 333, 1, False, True), (513, 257, 1031, 1, True, True),
                                     (256, 384, 200, 8, False, False)):
        a, b, _, _ = U.random_operands(rng, M, N, K, batch, ta, tb, "float32")
        bias = rng.standard_normal((N,), dtype=np.float32)
        want = ref.matmul_oracle(a, b, transpose_a=ta, transpose_b=tb, bias=bias, act=0)
        # large products take the tensor cores by default and stay inside the 1e-5 gate
        got = run(ops, a, b, ta=ta, tb=tb, bias=bias, act=0)
        assert binding.last_kernel_name().startswith("tc_tf32x3"), binding.last_kernel_name()
        check(got, want, "float32", "3xTF32")
        # the exact FFMA kernel on request
        exact = run(ops, a, b, ta=ta, tb=tb, bias=bias, act=0, use_tensor_cores=False)
        assert binding.last_kernel_name().startswith("simt_f32")
        assert ref.rel_frobenius(exact, want) <= 2e-6
    # small products stay on the FFMA kernel
    a, b, _, _ = U.random_operands(rng, 100, 90, 80, 1, False, False, "float32")
    run(ops, a, b)
    assert binding.last_kernel_name().startswith("simt_f32")
    # forcing the tensor-core path without workspace is rejected, not silently rerouted
    lib = binding.load_library()
    d = binding.new_desc()
    x = torch.zeros(256, 256, device="cuda")
    d.A = d.B = d.C = x.data_ptr()
    d.M = d.N = d.K = 256
    d.path = binding.PATH_TENSOR_CORE
    assert lib.sm120_matmul_workspace_bytes(ctypes.byref(d)) == 2 * 256 * 2 * 256 * 4      # both operands as [hi | lo] rows
    assert lib.sm120_launch_matmul_ex(ctypes.byref(d)) == 1
    # AUTO without workspace: the FFMA kernel (the reference-signature entry point carries none)
    d.path = binding.PATH_AUTO
    assert lib.sm120_launch_matmul_ex(ctypes.byref(d)) == 0
    assert binding.last_kernel_name().startswith("simt_f32")
    torch.cuda.synchronize()


@pytest.mark.parametrize("K", [1024, 4096, 8192])
@pytest.mark.parametrize("dist", ["uniform_pm1", "uniform_01", "normal"])
def test_fp32_tensor_core_accuracy_gate(ops, binding, K, dist):
    """rel-Frobenius <= 1e-5 against float64 for long inner dimensions; same-sign data (U[0,1]) is the worst case
    for the tensor cores' truncating accumulation, which the run-wise promotion bounds."""
    rng = np.random.default_rng(K)
    M, N = 384, 512
    draw = {"uniform_pm1": lambda s: rng.uniform(-1, 1, s), "uniform_01": lambda s: rng.uniform(0, 1, s),
            "normal": lambda s: rng.standard_normal(s)}[dist]
    a = draw((M, K)).astype(np.float32)
    b = draw((K, N)).astype(np.float32)
    want = a.astype(np.float64) @ b.astype(np.float64)
    got = run(ops, a, b)
    assert binding.last_kernel_name().startswith("tc_tf32x3"), binding.last_kernel_name()
    err = ref.rel_frobenius(got, want)
    assert err <= ref.TOLERANCE["float32"], (K, dist, err)
    assert np.array_equal(got, run(ops, a, b))                      # and reproducible bit for bit


def test_empty_and_zero_inner_dimension(ops, binding):
    # no rows / no columns: nothing is launched, the (empty) result has the right shape
    for (M, N, K) in ((0, 8, 16), (8, 0, 16), (0, 0, 0)):
        out = ops.advanced_matmul(torch.zeros(M, K, device="cuda"), torch.zeros(K, N, device="cuda"))
        assert tuple(out.shape) == (M, N)
    # K == 0: the product is the zero matrix; the epilogue still applies (bias, activation)
    bias = torch.arange(7, dtype=torch.float32, device="cuda") - 3
    out = ops.fused_matmul(torch.zeros(5, 0, device="cuda"), torch.zeros(0, 7, device="cuda"), bias=bias, activation="relu")
    torch.cuda.synchronize()
    assert binding.last_kernel_name().startswith("simt_f32")
    assert torch.equal(out, torch.relu(bias).expand(5, 7))
    out = ops.advanced_matmul(torch.zeros(5, 0, device="cuda").bfloat16(), torch.zeros(0, 7, device="cuda").bfloat16())
    assert tuple(out.shape) == (5, 7) and float(out.abs().max()) == 0.0


# ----- short-K problems: the 16-warp epilogue of the pair tile against the 8-warp one and the oracle -----
@pytest.mark.parametrize("case", ["bf16", "bf16_bias_gelu_f32out", "fp8", "f16_relu_batched_ragged_tail"])
def test_short_k_epilogue_variants_agree(ops, binding, case):
    lib = binding.load_library()
    torch.manual_seed(21)
    kw = {}
    if case == "bf16":
        a = torch.randn(2560, 192, device="cuda").bfloat16(); b = torch.randn(192, 2304, device="cuda").bfloat16()
    elif case == "bf16_bias_gelu_f32out":
        a = torch.randn(2048, 256, device="cuda").bfloat16(); b = torch.randn(256, 3072, device="cuda").bfloat16()
        kw = dict(bias=torch.randn(3072, device="cuda").bfloat16(), activation="gelu", out_dtype=torch.float32)
    elif case == "fp8":
        a, sa = ops.quantize_fp8(torch.randn(2048, 512, device="cuda")); b, sb = ops.quantize_fp8(torch.randn(2560, 512, device="cuda"))
        kw = dict(transpose_b=True, scale_a=sa, scale_b=sb)
    else:   # 5 x 20 x 8 = 800 pair tiles: the last wave is short; M is not a multiple of the tile
        a = torch.randn(5, 2500, 128, device="cuda").half(); b = torch.randn(5, 128, 2048, device="cuda").half()
        kw = dict(activation="relu")
    outs, names = [], []
    for bit in (binding.TUNE_EPI_WARPS_8, binding.TUNE_EPI_WARPS_16):
        outs.append(ops.fused_matmul(a, b, tuning=bit, **kw))
        torch.cuda.synchronize()
        names.append(binding.last_kernel_name())
    assert "2cta" in names[0] and not names[0].endswith("_e16") and names[1].endswith("_e16"), names
    assert torch.equal(outs[0], outs[1]), case
    assert torch.equal(ops.fused_matmul(a, b, **kw), outs[1])     # the launcher's own choice for short K
    assert binding.last_kernel_name().endswith("_e16")
    # and against the float64 oracle on sampled rows (operands as stored; fp8 through its scales)
    rows = torch.randint(0, a.shape[-2], (24,), device="cuda")
    a2, b2 = (a[0], b[0]) if a.dim() == 3 else (a, b)
    o2 = outs[1][0] if a.dim() == 3 else outs[1]
    A = a2[rows].float().double().cpu().numpy()
    B = b2.float().double().cpu().numpy()
    want = A @ (B.T if kw.get("transpose_b") else B)
    if case == "fp8":
        want = want / (float(kw["scale_a"]) * float(kw["scale_b"]))
    if "bias" in kw:
        want = ref.activation(want + kw["bias"].float().double().cpu().numpy(), ref.ACT_CODES["gelu"])
    if kw.get("activation") == "relu":
        want = np.maximum(want, 0.0)
    assert ref.rel_frobenius(o2[rows].float().cpu().numpy(), want) <= TOL["bfloat16"]


# ----- re-entrancy: the launchers carry no per-call state outside the descriptor -----
def test_concurrent_host_threads(ops, binding):
    """Four host threads, each with its own stream, shape, dtype and tuning bits, launch at the same
    time; every result must match the oracle."""
    rng = np.random.default_rng(404)
    jobs = [
        dict(M=520, N=264, K=136, dtype="bfloat16", tb=False, tuning=binding.TUNE_CTA_GROUP_1, act=0),
        dict(M=1024, N=768, K=512, dtype="float16", tb=True, tuning=binding.TUNE_CTA_GROUP_2, act=-1),
        dict(M=300, N=200, K=100, dtype="float32", tb=False, tuning=0, act=9),
        dict(M=384, N=640, K=256, dtype="fp8_e4m3", tb=True, tuning=binding.TUNE_CTA_GROUP_2 | binding.TUNE_EPI_WARPS_8, act=-1),
    ]
    for j in jobs:
        j["a"], j["b"], j["sa"], j["sb"] = U.random_operands(rng, j["M"], j["N"], j["K"], 1, False, j["tb"], j["dtype"], scale=0.5)
        fp8 = j["dtype"] == "fp8_e4m3"
        j["want"] = ref.matmul_oracle(j["a"], j["b"], transpose_b=j["tb"], act=j["act"],
                                      scale_a=j["sa"] if fp8 else 1.0, scale_b=j["sb"] if fp8 else 1.0,
                                      out_dtype="bfloat16" if fp8 else j["dtype"])
        j["ta_"], j["tb_"] = U.to_cuda(j["a"]), U.to_cuda(j["b"])
    torch.cuda.synchronize()
    start = threading.Barrier(len(jobs))
    errors = []

    def work(j):
        try:
            torch.cuda.set_device(0)
            stream = torch.cuda.Stream()
            fp8 = j["dtype"] == "fp8_e4m3"
            start.wait()
            with torch.cuda.stream(stream):
                outs = [ops.fused_matmul(j["ta_"], j["tb_"], transpose_b=j["tb"], activation=j["act"], tuning=j["tuning"],
                                         scale_a=j["sa"] if fp8 else None, scale_b=j["sb"] if fp8 else None)
                        for _ in range(25)]
            stream.synchronize()
            j["got"] = [U.to_numpy(o) for o in (outs[0], outs[-1])]
        except Exception as e:      # surfaced by the main thread
            errors.append(e)

    threads = [threading.Thread(target=work, args=(j,)) for j in jobs]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not errors, errors
    for j in jobs:
        tol = "bfloat16" if j["dtype"] == "fp8_e4m3" else j["dtype"]
        for got in j["got"]:
            check(got, j["want"], tol, f"thread {j['dtype']}")
        assert np.array_equal(j["got"][0].view(np.uint8), j["got"][1].view(np.uint8))


def test_tensor_map_cache_is_reused(ops, binding):
    a = torch.randn(512, 256, device="cuda").bfloat16()
    b = torch.randn(256, 384, device="cuda").bfloat16()
    out = torch.empty(512, 384, device="cuda", dtype=torch.bfloat16)
    ops.fused_matmul(a, b, out=out)
    enc0, hit0 = binding.tensor_map_stats()
    for _ in range(10):
        ops.fused_matmul(a, b, out=out)
    enc1, hit1 = binding.tensor_map_stats()
    assert enc1 == enc0 and hit1 - hit0 == 30          # three maps per launch, all from the cache
    torch.cuda.synchronize()


def test_launch_trace(ops, binding):
    """The optional timeline (SM120_TUNE_TRACE) of a CTA-pair launch: every CTA reports its tiles in order."""
    torch.manual_seed(9)
    a = torch.randn(2048, 1024, device="cuda").bfloat16()
    b = torch.randn(2048, 1024, device="cuda").bfloat16()
    trace = torch.zeros(binding.TRACE_BYTES // 8, dtype=torch.int64, device="cuda")
    c = ops.fused_matmul(a, b, transpose_b=True, tuning=binding.TUNE_CTA_GROUP_2, trace=trace)
    assert torch.equal(c, ops.fused_matmul(a, b, transpose_b=True, tuning=binding.TUNE_CTA_GROUP_2))
    t = trace.cpu().numpy().reshape(binding.TRACE_MAX_CTAS, binding.TRACE_WORDS_PER_CTA)
    ctas = 2 * 64                                       # 8 x 8 pair tiles, one per cluster
    assert (t[:ctas, 6] == 1).all() and (t[ctas:, :] == 0).all()
    assert (t[:ctas, 0] <= t[:ctas, 2]).all() and (t[:ctas, 2] < t[:ctas, 4]).all()       # entry <= set-up done < exit (ns)
    lead = t[0:ctas:2]
    assert (lead[:, 8] > lead[:, 3]).all() and (lead[:, 9] > lead[:, 8]).all()            # first k-block, last MMA issued
    assert (t[:ctas, 10] > t[:ctas, 3]).all() and (t[:ctas, 11] > t[:ctas, 10]).all()     # accumulator ready, last store
    assert (t[:ctas, 5] >= t[:ctas, 11]).all()


# ----- seeded sweep over random shapes and argument combinations -----
_SWEEP_DIMS = [1, 2, 7, 8, 16, 24, 33, 64, 72, 100, 128, 136, 200, 256, 264, 384, 520, 640]
_SWEEP_DIMS_LARGE = [64, 128, 520, 776, 1024, 1160, 2048, 2312]          # pair tiles, ragged edges, few-tile shapes
_SWEEP_K_LARGE = [264, 1024, 2048, 4096, 8192]                           # long enough for split-K and the fp32 split


def _sweep_case(seed, large=False):
    rng = np.random.default_rng((9500 if large else 9000) + seed)
    pick = lambda xs: xs[int(rng.integers(len(xs)))]
    din = pick(["float32", "float16", "bfloat16", "bfloat16", "fp8_e4m3"])
    dims = _SWEEP_DIMS_LARGE if large else _SWEEP_DIMS
    M, N, K = pick(dims), pick(dims), pick(_SWEEP_K_LARGE if large else dims)
    if din == "fp8_e4m3":
        K = max(16, K - K % 16)                  # FP8 operands: K a multiple of 16 (the ABI's rule)
    case = dict(din=din, M=M, N=N, K=K, batch=pick([1, 1, 1, 2] if large else [1, 1, 1, 3]), ta=bool(rng.integers(2)), tb=bool(rng.integers(2)),
                act=int(rng.integers(-1, 10)), alpha=pick([1.0, 1.0, 0.5, -1.25]), beta=pick([0.0, 0.0, 0.75]),
                bias=pick([None, None, "float32", "float16", "bfloat16"]),
                dout=pick(["float32", "float16", "bfloat16"]) if din == "fp8_e4m3" or rng.integers(3) == 0 else din,
                tc=pick([None, None, None, False]))
    return rng, case


@pytest.mark.parametrize("large,seed", [(False, s) for s in range(48)] + [(True, s) for s in range(20)])
def test_seeded_sweep_matches_oracle(ops, large, seed):
    """Shapes from 1 to 640 with ragged and unaligned sizes (and, in the large class, up to 2312 x 2312 x 8192), every
    operand layout, bias, activation, alpha / beta and output type drawn together from one seeded stream, each against
    the float64 oracle at the looser of the input and output types' gates."""
    rng, c = _sweep_case(seed, large)
    a, b, sa, sb = U.random_operands(rng, c["M"], c["N"], c["K"], c["batch"], c["ta"], c["tb"], c["din"], scale=0.3)
    lead = (c["batch"],) if c["batch"] > 1 else ()
    bias = None if c["bias"] is None else ref.quantize(rng.standard_normal((c["N"],), dtype=np.float32), c["bias"])
    c_in = None
    if c["beta"] != 0.0:
        c_in = ref.quantize(rng.standard_normal(lead + (c["M"], c["N"]), dtype=np.float32), c["dout"])
    fp8 = c["din"] == "fp8_e4m3"
    got = run(ops, a, b, ta=c["ta"], tb=c["tb"], bias=bias, act=c["act"], alpha=c["alpha"], beta=c["beta"], c_in=c_in,
              out_dtype=c["dout"], sa=sa if fp8 else None, sb=sb if fp8 else None, use_tensor_cores=c["tc"])
    want = ref.matmul_oracle(a, b, transpose_a=c["ta"], transpose_b=c["tb"], alpha=c["alpha"], beta=c["beta"], c_in=c_in,
                             bias=bias, act=c["act"], out_dtype=c["dout"], scale_a=sa, scale_b=sb)
    assert got.shape == want.shape, c
    gate = "float16" if (c["din"] == "float32") != (c["dout"] == "float32") and not fp8 else c["din"]
    if np.linalg.norm(np.asarray(want).astype(np.float64)) == 0.0:
        assert not np.asarray(got).astype(np.float32).any(), c
    else:
        check(got, want, gate, str(c))
