"""CPU oracle for the SM120 matmul op.  TEST INFRASTRUCTURE ONLY.

Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline legs may import
this module; the product (the package's csrc/ and its Python host code) never
does.

PARITY UNPINNED.  The reference's CPU path is ``tf.linalg.matmul`` followed by
``tf.nn.bias_add`` and a Keras activation (python/sm120_ops.py:210-213,
python/sm120_keras_layers.py:159-174).  TensorFlow (pinned only as
``tensorflow>=2.10.0``, setup.py:562-565) is a third-party dependency that is
not part of the reference tree and is not installed here, and the reference's
own GPU kernel is numerically wrong for K >= 4
(src/cuda_kernels/sm120_pure_kernels.cu:41-47), so neither can be run to pin
this file.  The reference holds no golden vectors for the path; its tests
compare against ``tf.matmul`` by tolerance on unseeded inputs
(tests/test_sm120_operations.py:80-122).  The only literal known answer in the
reference is the 2x2 product at scripts/validate-installation.py:381-388; it is
checked in tests/test_oracle.py.  What this file restates is therefore the
published definition of the op, not TensorFlow's code:

    C[b,i,j] = act( alpha * inv_scale * sum_k op(A)[b,i,k] * op(B)[b,k,j]
                    + beta * C_in[b,i,j] + bias[j] )

with the sum carried in float64 (the gate oracle), rounded once to the output
dtype (round-to-nearest-even).  alpha/beta follow
src/cuda_kernels/sm120_pure_kernels.cu:58-63, the transposed/batched indexing
follows src/cuda_kernels/sm120_dynamic_shapes.cu:121-182, the activation
formulas follow src/cuda_kernels/sm120_pure_kernels.cu:141-171 (code 9 is the
exact erf GELU of Keras), FP8 quantisation is the saturating-finite e4m3
conversion of src/cuda_kernels/sm120_datatype_support.h:168-171.
"""
from __future__ import annotations

import math
import os
import time

import ml_dtypes
import numpy as np

# SM120DataType / SM120ActivationType codes of include/sm120_c_interface.h
DTYPE_CODES = {"float32": 0, "float16": 1, "bfloat16": 2, "fp8_e4m3": 3}
NP_DTYPES = {
    "float32": np.dtype(np.float32),
    "float16": np.dtype(np.float16),
    "bfloat16": np.dtype(ml_dtypes.bfloat16),
    "fp8_e4m3": np.dtype(ml_dtypes.float8_e4m3fn),
}
ACT_CODES = {
    None: -1, "linear": -1, "none": -1,
    "relu": 0, "leaky_relu": 1, "elu": 2, "selu": 3, "gelu_tanh": 4, "swish": 5,
    "mish": 6, "tanh": 7, "sigmoid": 8, "gelu": 9, "gelu_erf": 9,
}
E4M3_MAX = 448.0

# parity tolerances per input type (relative Frobenius error against this oracle)
TOLERANCE = {"float32": 1e-5, "float16": 1e-2, "bfloat16": 1e-2, "fp8_e4m3": 5e-2}


def quantize(x: np.ndarray, dtype: str) -> np.ndarray:
    """Round float values to `dtype` (round-to-nearest-even).  FP8 saturates at
    +-448 instead of producing NaN (saturating-finite conversion,
    src/cuda_kernels/sm120_datatype_support.h:168-171)."""
    if dtype == "fp8_e4m3":
        x = np.clip(np.asarray(x, dtype=np.float32), -E4M3_MAX, E4M3_MAX)
    with np.errstate(over="ignore"):
        return np.asarray(x).astype(NP_DTYPES[dtype])


def fp8_scale(x: np.ndarray) -> float:
    """Per-tensor scale that maps amax(x) to 448 (the FP8 workload)."""
    amax = float(np.max(np.abs(x)))
    return E4M3_MAX / amax if amax > 0 else 1.0


_erf = np.vectorize(math.erf, otypes=[np.float64])


def erf64(x: np.ndarray) -> np.ndarray:
    try:
        from scipy.special import erf  # vectorised; same function
        return erf(x)
    except Exception:  # pragma: no cover
        return _erf(x)


def activation(x: np.ndarray, code: int) -> np.ndarray:
    """float64 restatement of the activation table
    (src/cuda_kernels/sm120_pure_kernels.cu:141-171) plus code 9 = erf GELU."""
    x = np.asarray(x, dtype=np.float64)
    if code == -1:
        return x
    if code == 0:
        return np.maximum(0.0, x)
    if code == 1:
        return np.where(x > 0, x, 0.01 * x)
    if code == 2:
        return np.where(x > 0, x, np.expm1(np.minimum(x, 0)))
    if code == 3:
        return np.where(x > 0, 1.0507 * x, 1.0507 * 1.67326 * np.expm1(np.minimum(x, 0)))
    if code == 4:
        return 0.5 * x * (1.0 + np.tanh(0.7978845608 * (x + 0.044715 * x * x * x)))
    if code == 5:
        return x / (1.0 + np.exp(-x))
    if code == 6:
        return x * np.tanh(np.log1p(np.exp(x)))
    if code == 7:
        return np.tanh(x)
    if code == 8:
        return 1.0 / (1.0 + np.exp(-x))
    if code == 9:
        return 0.5 * x * (1.0 + erf64(x / math.sqrt(2.0)))
    raise ValueError(f"unknown activation code {code}")


def _op(x: np.ndarray, transpose: bool) -> np.ndarray:
    return np.swapaxes(x, -1, -2) if transpose else x


def matmul_oracle(a, b, *, transpose_a=False, transpose_b=False, alpha=1.0, beta=0.0, c_in=None, bias=None,
                  act=-1, out_dtype="float32", scale_a=1.0, scale_b=1.0, round_output=True):
    """The gate oracle: float64 product of the values `a` and `b` hold (whatever
    their dtype), epilogue in float64, one rounding to `out_dtype`.

    a: [..., M, K] (or [..., K, M] with transpose_a); b likewise; leading batch
    dimensions broadcast as in a strided-batch GEMM with stride 0."""
    a64 = _op(np.asarray(a).astype(np.float64), transpose_a)
    b64 = _op(np.asarray(b).astype(np.float64), transpose_b)
    acc = np.matmul(a64, b64)
    v = (float(alpha) / (float(scale_a) * float(scale_b))) * acc
    if beta != 0.0:
        v = v + float(beta) * np.asarray(c_in).astype(np.float64)
    if bias is not None:
        v = v + np.asarray(bias).astype(np.float64)
    v = activation(v, act)
    if not round_output:
        return v
    return quantize(v, out_dtype)


def softmax_oracle(x: np.ndarray, axis: int = -1) -> np.ndarray:
    """float64 softmax with the maximum subtracted (src/cuda_kernels/sm120_pure_kernels.cu:489-549)."""
    x = np.asarray(x).astype(np.float64)
    m = np.max(x, axis=axis, keepdims=True)
    m = np.where(np.isfinite(m), m, 0.0)
    e = np.exp(x - m)
    s = np.sum(e, axis=axis, keepdims=True)
    return np.divide(e, s, out=np.zeros_like(e), where=s > 0)


def attention_oracle(q, k, v, scale=None, mask=None, causal=False, return_weights=False):
    """softmax(scale * Q K^T + mask * -1e9 [causal]) V in float64 over the last two dimensions: the layer's
    standard attention (python/sm120_keras_layers.py:810-826; causal as python/sm120_ops.py:388-398, aligned
    to the end of the keys).  `mask` marks excluded positions with non-zero entries."""
    q, k, v = (np.asarray(t).astype(np.float64) for t in (q, k, v))
    d = q.shape[-1]
    scale = 1.0 / math.sqrt(d) if scale is None else scale
    s = np.matmul(q, np.swapaxes(k, -1, -2)) * scale
    if mask is not None:
        s = s + np.asarray(mask).astype(np.float64) * -1e9
    if causal:
        sq, sk = s.shape[-2], s.shape[-1]
        keep = np.arange(sk)[None, :] <= (np.arange(sq)[:, None] + sk - sq)
        s = np.where(keep, s, -np.inf)
    w = softmax_oracle(s, axis=-1)
    out = np.matmul(w, v)
    return (out, w) if return_weights else out


def rel_frobenius(x, ref) -> float:
    """||x - ref||_F / ||ref||_F in float64 (the parity metric)."""
    x = np.asarray(x).astype(np.float64)
    ref = np.asarray(ref).astype(np.float64)
    den = float(np.linalg.norm(ref.ravel()))
    num = float(np.linalg.norm((x - ref).ravel()))
    if den == 0.0:
        return 0.0 if num == 0.0 else float("inf")
    return num / den


def max_abs_tolerance_ok(x, ref, rtol=1e-3, atol=1e-3) -> bool:
    """The reference tests' own criterion: max|x-ref| <= atol + rtol*max|ref|
    (tests/test_sm120_operations.py:80-102)."""
    x = np.asarray(x).astype(np.float64)
    ref = np.asarray(ref).astype(np.float64)
    return float(np.max(np.abs(x - ref))) <= atol + rtol * float(np.max(np.abs(ref)))


# ---------------------------------------------------------------------------
# Seeded inputs for the five benchmark configurations.  `shrink` divides the
# large extents so the same distributions can be checked at oracle-friendly size.
# ---------------------------------------------------------------------------
CONFIG_NAMES = {
    1: "cfg1_fp32_1024",
    2: "cfg2_fp16_4096_tn",
    3: "cfg3_bf16_dense_gelu",
    4: "cfg4_bf16_batched_qk",
    5: "cfg5_fp8_mshard",
}


def config_shapes(idx: int, shrink: int = 1) -> dict:
    s = max(1, int(shrink))
    if idx == 1:
        n = 1024 // s
        return dict(M=n, N=n, K=n, batch=1)
    if idx == 2:
        n = 4096 // s
        return dict(M=n, N=n, K=n, batch=1)
    if idx == 3:
        return dict(M=8192 // s, N=11008 // s, K=4096 // s, batch=1)
    if idx == 4:
        return dict(M=2048 // s, N=2048 // s, K=128, batch=max(1, 64 // s))
    if idx == 5:
        return dict(M=65536 // s, N=8192 // s, K=8192 // s, batch=1)
    raise ValueError(idx)


def config_flops(idx: int, shrink: int = 1) -> float:
    sh = config_shapes(idx, shrink)
    return 2.0 * sh["M"] * sh["N"] * sh["K"] * sh["batch"]


def make_config(idx: int, shrink: int = 1) -> dict:
    """Inputs (already quantised to the config's input dtype), descriptor fields
    and oracle keyword arguments for benchmark configuration `idx` (1..5), drawn from
    numpy.random.default_rng(idx - 1)."""
    sh = config_shapes(idx, shrink)
    M, N, K, batch = sh["M"], sh["N"], sh["K"], sh["batch"]
    rng = np.random.default_rng(idx - 1)
    cfg = dict(idx=idx, name=CONFIG_NAMES[idx], **sh, transpose_a=False, transpose_b=False, bias=None, act=-1,
               scale_a=1.0, scale_b=1.0)
    if idx == 1:
        cfg.update(in_dtype="float32", out_dtype="float32")
        cfg["a"] = rng.uniform(-1, 1, (M, K)).astype(np.float32)
        cfg["b"] = rng.uniform(-1, 1, (K, N)).astype(np.float32)
    elif idx == 2:
        cfg.update(in_dtype="float16", out_dtype="float16", transpose_b=True)
        cfg["a"] = quantize(rng.standard_normal((M, K), dtype=np.float32) / math.sqrt(K), "float16")
        cfg["b"] = quantize(rng.standard_normal((N, K), dtype=np.float32) / math.sqrt(K), "float16")  # stored [N,K]
    elif idx == 3:
        cfg.update(in_dtype="bfloat16", out_dtype="bfloat16", act=ACT_CODES["gelu"])
        cfg["a"] = quantize(rng.standard_normal((M, K), dtype=np.float32), "bfloat16")
        cfg["b"] = quantize(0.02 * rng.standard_normal((K, N), dtype=np.float32), "bfloat16")
        cfg["bias"] = quantize(0.02 * rng.standard_normal((N,), dtype=np.float32), "bfloat16")
    elif idx == 4:
        cfg.update(in_dtype="bfloat16", out_dtype="bfloat16")
        cfg["a"] = quantize(rng.standard_normal((batch, M, K), dtype=np.float32), "bfloat16")
        cfg["b"] = quantize(rng.standard_normal((batch, K, N), dtype=np.float32), "bfloat16")
    elif idx == 5:
        cfg.update(in_dtype="fp8_e4m3", out_dtype="bfloat16", transpose_b=True)
        a32 = rng.standard_normal((M, K), dtype=np.float32)
        b32 = rng.standard_normal((N, K), dtype=np.float32)   # stored [N,K]: K-major
        sa, sb = fp8_scale(a32), fp8_scale(b32)
        cfg["a_unquantized"], cfg["b_unquantized"] = a32, b32
        cfg["a"] = quantize(a32 * np.float32(sa), "fp8_e4m3")
        cfg["b"] = quantize(b32 * np.float32(sb), "fp8_e4m3")
        cfg["scale_a"], cfg["scale_b"] = float(np.float32(sa)), float(np.float32(sb))
    return cfg


def oracle_for_config(cfg: dict, round_output: bool = True):
    return matmul_oracle(cfg["a"], cfg["b"], transpose_a=cfg["transpose_a"], transpose_b=cfg["transpose_b"],
                         bias=cfg["bias"], act=cfg["act"], out_dtype=cfg["out_dtype"], scale_a=cfg["scale_a"],
                         scale_b=cfg["scale_b"], round_output=round_output)


# ---------------------------------------------------------------------------
# Timed CPU baseline: the same computation in fp32 through the host BLAS with
# every core, standing in for TensorFlow's CPU matmul (+ bias_add + activation).
# ---------------------------------------------------------------------------
def cpu_baseline_fp32(a, b, *, transpose_a=False, transpose_b=False, bias=None, act=-1, scale_a=1.0, scale_b=1.0,
                      threads: int | None = None, repeats: int = 3):
    """Returns (result_fp32, best_seconds, threads_used).  Inputs are up-cast from
    their quantised values to fp32 outside the timed region."""
    import torch

    threads = threads or os.cpu_count() or 1
    torch.set_num_threads(threads)
    ta = torch.from_numpy(np.ascontiguousarray(np.asarray(a).astype(np.float32)))
    tb = torch.from_numpy(np.ascontiguousarray(np.asarray(b).astype(np.float32)))
    tbias = None if bias is None else torch.from_numpy(np.asarray(bias).astype(np.float32))
    inv = 1.0 / (float(scale_a) * float(scale_b))
    best = float("inf")
    out = None
    for _ in range(max(1, repeats)):
        t0 = time.perf_counter()
        x = ta.transpose(-1, -2) if transpose_a else ta
        y = tb.transpose(-1, -2) if transpose_b else tb
        r = torch.matmul(x, y)
        if inv != 1.0:
            r = r * inv
        if tbias is not None:
            r = r + tbias
        if act == 0:
            r = torch.relu(r)
        elif act == 9:
            r = torch.nn.functional.gelu(r)
        elif act == 4:
            r = torch.nn.functional.gelu(r, approximate="tanh")
        elif act != -1:
            r = torch.from_numpy(activation(r.numpy(), act).astype(np.float32))
        dt = time.perf_counter() - t0
        best = min(best, dt)
        out = r
    return out.numpy(), best, threads
