"""Helpers shared by the test files (not collected as tests)."""
import ctypes
import os

import ml_dtypes
import numpy as np

from oracle import reference as ref

GOLDEN_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "golden_small.npz")
CODE_TO_NAME = {v: k for k, v in ref.DTYPE_CODES.items()}


def from_bits(x: np.ndarray, dtype_name: str) -> np.ndarray:
    if dtype_name == "bfloat16":
        return x.view(ml_dtypes.bfloat16)
    if dtype_name == "fp8_e4m3":
        return x.view(ml_dtypes.float8_e4m3fn)
    return x


def load_golden():
    """name -> dict(a, b, c, bias, c_in, M, N, K, batch, ta, tb, act, in_dtype, out_dtype, alpha, beta, sa, sb)."""
    z = np.load(GOLDEN_PATH)
    names = sorted({k.split("__")[0] for k in z.files})
    cases = {}
    for n in names:
        M, N, K, batch, ta, tb, act, din, dout = [int(v) for v in z[f"{n}__meta"]]
        alpha, beta, sa, sb = [float(v) for v in z[f"{n}__scal"]]
        din_n, dout_n = CODE_TO_NAME[din], CODE_TO_NAME[dout]
        cases[n] = dict(
            a=from_bits(z[f"{n}__a"], din_n), b=from_bits(z[f"{n}__b"], din_n), c=from_bits(z[f"{n}__c"], dout_n),
            bias=z[f"{n}__bias"] if f"{n}__bias" in z.files else None,
            c_in=from_bits(z[f"{n}__c_in"], dout_n) if f"{n}__c_in" in z.files else None,
            M=M, N=N, K=K, batch=batch, ta=bool(ta), tb=bool(tb), act=act, in_dtype=din_n, out_dtype=dout_n,
            alpha=alpha, beta=beta, sa=sa, sb=sb)
    return cases


def to_cuda(x: np.ndarray):
    """numpy (incl. ml_dtypes) -> torch CUDA tensor of the matching dtype."""
    import torch
    x = np.ascontiguousarray(x)
    if x.dtype == np.dtype(ml_dtypes.bfloat16):
        return torch.from_numpy(x.view(np.uint16)).cuda().view(torch.bfloat16)
    if x.dtype == np.dtype(ml_dtypes.float8_e4m3fn):
        return torch.from_numpy(x.view(np.uint8)).cuda().view(torch.float8_e4m3fn)
    return torch.from_numpy(x).cuda()


def to_numpy(t):
    import torch
    t = t.detach().cpu().contiguous()
    if t.dtype == torch.bfloat16:
        return t.view(torch.uint16).numpy().view(ml_dtypes.bfloat16)
    if t.dtype == torch.float8_e4m3fn:
        return t.view(torch.uint8).numpy().view(ml_dtypes.float8_e4m3fn)
    return t.numpy()


def torch_dtype(name: str):
    import torch
    return {"float32": torch.float32, "float16": torch.float16, "bfloat16": torch.bfloat16,
            "fp8_e4m3": torch.float8_e4m3fn}[name]


def random_operands(rng, M, N, K, batch, ta, tb, dtype_name, scale=1.0):
    """Quantised operands (+ fp8 scales) drawn from N(0, scale^2)."""
    lead = (batch,) if batch > 1 else ()
    a = scale * rng.standard_normal(lead + ((K, M) if ta else (M, K)), dtype=np.float32)
    b = scale * rng.standard_normal(lead + ((N, K) if tb else (K, N)), dtype=np.float32)
    sa = sb = 1.0
    if dtype_name == "fp8_e4m3":
        sa, sb = float(np.float32(ref.fp8_scale(a))), float(np.float32(ref.fp8_scale(b)))
        a, b = a * np.float32(sa), b * np.float32(sb)
    return ref.quantize(a, dtype_name), ref.quantize(b, dtype_name), sa, sb


_c_oracle = None


def c_oracle():
    """The plain-C oracle (oracle/matmul_ref.c), built on demand with gcc."""
    global _c_oracle
    if _c_oracle is not None:
        return _c_oracle
    import subprocess
    odir = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle")
    so = os.path.join(odir, "libsm120_ref.so")
    if not os.path.exists(so):
        subprocess.check_call(["make", "-C", odir], stdout=subprocess.DEVNULL)
    lib = ctypes.CDLL(so)
    i64, f32p = ctypes.c_int64, ctypes.POINTER(ctypes.c_float)
    lib.sm120_ref_matmul_f32.restype = ctypes.c_int
    lib.sm120_ref_matmul_f32.argtypes = [f32p, f32p, f32p, i64, i64, i64, i64, i64, i64, i64, i64, i64, i64,
                                         ctypes.c_int, ctypes.c_int, ctypes.c_float, ctypes.c_float]
    _c_oracle = lib
    return lib


def c_oracle_matmul(a, b, M, N, K, batch=1, ta=False, tb=False, alpha=1.0, beta=0.0, c_in=None):
    """fp32-accumulate product through the C oracle; operands are up-cast to fp32 first."""
    lib = c_oracle()
    a32 = np.ascontiguousarray(np.asarray(a).astype(np.float32))
    b32 = np.ascontiguousarray(np.asarray(b).astype(np.float32))
    lead = (batch,) if batch > 1 else ()
    c = np.zeros(lead + (M, N), dtype=np.float32) if c_in is None else np.ascontiguousarray(np.asarray(c_in).astype(np.float32)).copy()
    f32p = ctypes.POINTER(ctypes.c_float)
    lda = M if ta else K
    ldb = K if tb else N
    rc = lib.sm120_ref_matmul_f32(a32.ctypes.data_as(f32p), b32.ctypes.data_as(f32p), c.ctypes.data_as(f32p),
                                  M, N, K, lda, ldb, N, batch, M * K if a32.ndim == 3 else 0,
                                  K * N if b32.ndim == 3 else 0, M * N, int(ta), int(tb), alpha, beta)
    assert rc == 0
    return c
