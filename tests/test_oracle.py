"""CPU tests of the oracle itself: the reference's one literal known answer,
agreement of the numpy (float64) and plain-C (fp32, sequential k) restatements,
quantisers, activation constants, and the committed golden vectors."""
import math

import ml_dtypes
import numpy as np
import pytest

from oracle import reference as ref
from tests import _util as U


def test_known_answer_2x2():
    # scripts/validate-installation.py:381-388: [[1,2],[3,4]] @ [[2,0],[0,2]] == [[2,4],[6,8]]
    a = np.array([[1.0, 2.0], [3.0, 4.0]], dtype=np.float32)
    b = np.array([[2.0, 0.0], [0.0, 2.0]], dtype=np.float32)
    expected = [[2.0, 4.0], [6.0, 8.0]]
    assert ref.matmul_oracle(a, b).tolist() == expected
    assert U.c_oracle_matmul(a, b, 2, 2, 2).tolist() == expected


@pytest.mark.parametrize("M,N,K,batch,ta,tb", [
    (32, 64, 64, 1, False, False), (64, 32, 32, 1, False, True), (128, 256, 256, 1, True, False),
    (17, 7, 129, 1, True, True), (1, 1, 1, 1, False, False), (16, 24, 40, 3, False, False),
    (5, 9, 0, 1, False, False),
])
def test_numpy_and_c_oracles_agree(M, N, K, batch, ta, tb):
    rng = np.random.default_rng(7)
    a, b, _, _ = U.random_operands(rng, M, N, K, batch, ta, tb, "float32", scale=0.1)
    c64 = ref.matmul_oracle(a, b, transpose_a=ta, transpose_b=tb, round_output=False)
    c32 = U.c_oracle_matmul(a, b, M, N, K, batch, ta, tb)
    assert c32.shape == c64.shape
    # fp32 sequential accumulation vs float64: the reference tests' own tolerance for f32
    assert ref.max_abs_tolerance_ok(c32, c64, rtol=1e-5, atol=1e-5)
    assert ref.rel_frobenius(c32, c64) <= 1e-5 or K == 0


def test_alpha_beta_semantics():
    # src/cuda_kernels/sm120_pure_kernels.cu:58-63: result = alpha*acc (+ beta*C only when beta != 0)
    rng = np.random.default_rng(3)
    a = rng.standard_normal((8, 5)).astype(np.float32)
    b = rng.standard_normal((5, 6)).astype(np.float32)
    c0 = rng.standard_normal((8, 6)).astype(np.float32)
    want = 0.5 * (a.astype(np.float64) @ b.astype(np.float64)) + 2.0 * c0
    got = ref.matmul_oracle(a, b, alpha=0.5, beta=2.0, c_in=c0, round_output=False)
    assert np.allclose(got, want, rtol=0, atol=1e-12)
    got_c = U.c_oracle_matmul(a, b, 8, 6, 5, alpha=0.5, beta=2.0, c_in=c0)
    assert ref.rel_frobenius(got_c, want) < 1e-6
    # beta == 0 must not read C: NaNs in c_in do not propagate
    nan_c = np.full((8, 6), np.nan, dtype=np.float32)
    assert np.isfinite(U.c_oracle_matmul(a, b, 8, 6, 5, alpha=1.0, beta=0.0, c_in=nan_c)).all()


def test_quantizers():
    x = np.array([0.0, 1.0, -1.0, 447.0, 448.0, 500.0, -1e9, 1e-9, 0.3], dtype=np.float32)
    q = ref.quantize(x, "fp8_e4m3").astype(np.float32)
    assert q.max() == 448.0 and q.min() == -448.0 and np.isfinite(q).all()   # saturating-finite
    assert q[1] == 1.0 and q[2] == -1.0 and q[3] == 448.0
    # round trip is exact for representable values
    for name in ("float16", "bfloat16", "fp8_e4m3"):
        once = ref.quantize(x, name)
        twice = ref.quantize(once.astype(np.float32), name)
        assert np.array_equal(once.view(np.uint8), twice.view(np.uint8))
    # bf16 rounding is to nearest even: 1 + 2^-8 is a tie between 1 and 1 + 2^-7
    assert float(ref.quantize(np.float32(1.0 + 2.0 ** -8), "bfloat16")) == 1.0
    assert float(ref.quantize(np.float32(1.0 + 3 * 2.0 ** -8), "bfloat16")) == 1.0 + 2.0 ** -6
    s = ref.fp8_scale(np.array([-3.5, 2.0], dtype=np.float32))
    assert s == 448.0 / 3.5


def test_activation_constants():
    x = np.linspace(-6, 6, 1001)
    gelu_tanh = ref.activation(x, 4)
    gelu_erf = ref.activation(x, 9)
    # the reference's tanh-GELU constants (src/cuda_kernels/sm120_pure_kernels.cu:154-156)
    want = 0.5 * x * (1 + np.tanh(0.7978845608 * (x + 0.044715 * x ** 3)))
    assert np.allclose(gelu_tanh, want, rtol=1e-14, atol=0)
    assert abs(0.7978845608 - math.sqrt(2 / math.pi)) < 1e-9
    assert 1e-4 < np.max(np.abs(gelu_tanh - gelu_erf)) < 1e-3     # the two GELUs differ, slightly
    assert np.array_equal(ref.activation(x, 0), np.maximum(0, x))
    assert np.allclose(ref.activation(np.array([-1.0]), 1), [-0.01])
    assert np.allclose(ref.activation(np.array([-1.0]), 3), [1.0507 * 1.67326 * (math.exp(-1) - 1)])
    assert np.allclose(ref.activation(np.array([0.0]), 8), [0.5])
    assert np.array_equal(ref.activation(x, -1), x)
    with pytest.raises(ValueError):
        ref.activation(x, 42)


def test_golden_vectors_match_oracle():
    cases = U.load_golden()
    assert len(cases) >= 7
    for name, g in cases.items():
        c = ref.matmul_oracle(g["a"], g["b"], transpose_a=g["ta"], transpose_b=g["tb"], alpha=g["alpha"], beta=g["beta"],
                              c_in=g["c_in"], bias=g["bias"], act=g["act"], out_dtype=g["out_dtype"], scale_a=g["sa"],
                              scale_b=g["sb"])
        assert c.dtype == g["c"].dtype, name
        assert np.array_equal(c.view(np.uint8), g["c"].view(np.uint8)), name
        # and the fp32 C oracle lands within the dtype's tolerance of the golden output
        if g["act"] == -1 and g["bias"] is None:
            c32 = U.c_oracle_matmul(g["a"], g["b"], g["M"], g["N"], g["K"], g["batch"], g["ta"], g["tb"],
                                    alpha=g["alpha"] / (g["sa"] * g["sb"]), beta=g["beta"], c_in=g["c_in"])
            assert ref.rel_frobenius(c32, g["c"]) <= ref.TOLERANCE[g["out_dtype"]], name


def test_baseline_config_generators():
    for idx in range(1, 6):
        cfg = ref.make_config(idx, shrink=32 if idx != 4 else 16)
        a, b = cfg["a"], cfg["b"]
        assert a.dtype == ref.NP_DTYPES[cfg["in_dtype"]] and b.dtype == a.dtype
        c = ref.oracle_for_config(cfg)
        lead = (cfg["batch"],) if cfg["batch"] > 1 else ()
        assert c.shape == lead + (cfg["M"], cfg["N"])
        assert c.dtype == ref.NP_DTYPES[cfg["out_dtype"]]
        assert np.isfinite(c.astype(np.float32)).all()
    # full-size shapes and FLOP counts of the five benchmark configurations
    assert ref.config_flops(2) == 2 * 4096 ** 3
    assert ref.config_shapes(3) == dict(M=8192, N=11008, K=4096, batch=1)
    assert ref.config_shapes(4) == dict(M=2048, N=2048, K=128, batch=64)
    assert ref.config_shapes(5) == dict(M=65536, N=8192, K=8192, batch=1)
    # config 5: amax maps to 448 and the quantised product stays within 5e-2 of the unquantised one
    cfg = ref.make_config(5, shrink=64)
    assert float(np.max(np.abs(cfg["a"].astype(np.float32)))) == 448.0
    exact = ref.matmul_oracle(cfg["a_unquantized"], cfg["b_unquantized"], transpose_b=True, round_output=False)
    assert ref.rel_frobenius(ref.oracle_for_config(cfg), exact) <= ref.TOLERANCE["fp8_e4m3"]


def test_cpu_baseline_matches_oracle():
    cfg = ref.make_config(3, shrink=32)
    out, secs, threads = ref.cpu_baseline_fp32(cfg["a"], cfg["b"], bias=cfg["bias"], act=cfg["act"], repeats=1)
    assert secs > 0 and threads >= 1
    assert ref.rel_frobenius(out, ref.oracle_for_config(cfg, round_output=False)) < 1e-5


def test_softmax_and_attention_oracle():
    rng = np.random.default_rng(0)
    x = rng.standard_normal((4, 9))
    w = ref.softmax_oracle(x)
    assert np.allclose(w.sum(-1), 1.0) and np.all(w > 0)
    assert np.allclose(ref.softmax_oracle(x + 100.0), w)                     # shift invariance
    assert np.array_equal(ref.softmax_oracle(np.full((2, 3), -np.inf)), np.zeros((2, 3)))
    q, k, v = rng.standard_normal((2, 5, 8)), rng.standard_normal((2, 7, 8)), rng.standard_normal((2, 7, 8))
    out, wts = ref.attention_oracle(q, k, v, return_weights=True)
    assert out.shape == (2, 5, 8) and np.allclose(wts.sum(-1), 1.0)
    # one key only: the output is that key's value
    assert np.allclose(ref.attention_oracle(q, k[:, :1], v[:, :1]), np.repeat(v[:, :1], 5, axis=1))
    # causal, aligned to the end: query i of 5 sees keys 0 .. i + 2 of 7
    _, wc = ref.attention_oracle(q, k, v, causal=True, return_weights=True)
    assert np.all(wc[:, 0, 3:] == 0) and np.all(wc[:, 0, :3] > 0) and np.all(wc[:, 4] > 0)
    # a mask entry excludes its position
    mask = np.zeros((5, 7)); mask[:, 2] = 1
    _, wm = ref.attention_oracle(q, k, v, mask=mask, return_weights=True)
    assert np.all(wm[..., 2] < 1e-300)
