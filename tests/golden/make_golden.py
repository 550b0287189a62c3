"""Writes tests/golden/golden_small.npz: seeded inputs and oracle outputs for a
handful of small SM120 matmul cases, so that the GPU parity tests have committed
vectors to compare against (the reference itself ships none for this path, and
its CPU implementation, TensorFlow, cannot be imported here: these vectors pin
the CUDA path to this repository's oracle, not to TensorFlow).

Run from the repository root:  python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import reference as ref  # noqa: E402

CASES = [
    # name, M, N, K, batch, in_dtype, out_dtype, ta, tb, act, bias, alpha, beta
    ("f32_plain", 48, 40, 36, 1, "float32", "float32", False, False, -1, False, 1.0, 0.0),
    ("f32_alpha_beta", 33, 65, 17, 1, "float32", "float32", False, False, -1, False, 0.5, 2.0),
    ("f16_tn", 128, 64, 64, 1, "float16", "float16", False, True, -1, False, 1.0, 0.0),
    ("bf16_dense_gelu", 96, 160, 128, 1, "bfloat16", "bfloat16", False, False, 9, True, 1.0, 0.0),
    ("bf16_batched", 64, 128, 64, 3, "bfloat16", "bfloat16", False, False, -1, False, 1.0, 0.0),
    ("bf16_nt_relu", 72, 48, 80, 1, "bfloat16", "float32", True, True, 0, True, 1.0, 0.0),
    ("fp8_scaled", 128, 128, 256, 1, "fp8_e4m3", "bfloat16", False, True, -1, False, 1.0, 0.0),
]


def build():
    out = {}
    for i, (name, M, N, K, batch, din, dout, ta, tb, act, has_bias, alpha, beta) in enumerate(CASES):
        rng = np.random.default_rng(1000 + i)
        lead = (batch,) if batch > 1 else ()
        a = rng.standard_normal(lead + ((K, M) if ta else (M, K)), dtype=np.float32)
        b = rng.standard_normal(lead + ((N, K) if tb else (K, N)), dtype=np.float32)
        sa = sb = 1.0
        if din == "fp8_e4m3":
            sa, sb = float(np.float32(ref.fp8_scale(a))), float(np.float32(ref.fp8_scale(b)))
            a, b = a * np.float32(sa), b * np.float32(sb)
        a, b = ref.quantize(a, din), ref.quantize(b, din)
        bias = ref.quantize(rng.standard_normal((N,), dtype=np.float32), "float32") if has_bias else None
        c_in = ref.quantize(rng.standard_normal(lead + (M, N), dtype=np.float32), dout) if beta != 0.0 else None
        c = ref.matmul_oracle(a, b, transpose_a=ta, transpose_b=tb, alpha=alpha, beta=beta, c_in=c_in, bias=bias,
                              act=act, out_dtype=dout, scale_a=sa, scale_b=sb)
        # store raw bits for the ml_dtypes types (npz cannot hold them)
        def bits(x):
            return x.view(np.uint16) if x.dtype.itemsize == 2 and x.dtype != np.float16 else (
                x.view(np.uint8) if x.dtype.itemsize == 1 else x)
        out[f"{name}__a"] = bits(a)
        out[f"{name}__b"] = bits(b)
        out[f"{name}__c"] = bits(c)
        if bias is not None:
            out[f"{name}__bias"] = bias
        if c_in is not None:
            out[f"{name}__c_in"] = bits(c_in)
        out[f"{name}__meta"] = np.array([M, N, K, batch, int(ta), int(tb), act, ref.DTYPE_CODES[din], ref.DTYPE_CODES[dout]], dtype=np.int64)
        out[f"{name}__scal"] = np.array([alpha, beta, sa, sb], dtype=np.float64)
    return out


if __name__ == "__main__":
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden_small.npz")
    np.savez_compressed(path, **build())
    print("wrote", path, os.path.getsize(path), "bytes")
