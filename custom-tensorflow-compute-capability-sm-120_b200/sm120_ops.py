"""Python API of the SM120 matmul op, B200 build.

Same public names, arguments and error behaviour as the reference's
``python/sm120_ops.py`` for the matmul path (``advanced_matmul`` :142-217,
``SM120Config`` :108-139, ``is_sm120_available`` :41-63, ``benchmark_operation``
:448-490, ``optimized_dense`` :494-552), with two deliberate differences:

* tensors are ``torch`` CUDA tensors (TensorFlow is not part of this build);
  host arrays (numpy or CPU torch tensors) are also accepted and are copied to
  the device, multiplied there and copied back;
* there is NO fallback to a stock or CPU matmul.  Where the reference warns and
  calls ``tf.linalg.matmul`` (:203-213) this module raises.

The computation itself happens in ``_sm120_ops.so`` through the C ABI
(``sm120_launch_matmul_ex``); this file only validates, allocates the output
with the caller's framework allocator (torch) and passes pointers and the
current CUDA stream, which is what ``SM120MatMulOp<T>::Compute`` does in the
reference (src/tensorflow_ops/sm120_ops_fixed.cc:111-150).
"""
from __future__ import annotations

import ctypes
import time
import warnings
from typing import Any, Callable, Dict, List, Optional, Sequence, Union

import numpy as np
import torch

from . import _binding as _b

try:
    import ml_dtypes as _ml
except Exception:  # pragma: no cover - ml_dtypes ships with the image
    _ml = None


class InvalidArgumentError(ValueError):
    """Stands in for ``tf.errors.InvalidArgumentError`` (incompatible shapes)."""


class UnimplementedError(RuntimeError):
    """Stands in for ``tf.errors.UnimplementedError``
    (python/sm120_ops.py:215-217: SM120 operations not available)."""


class InternalError(RuntimeError):
    """Stands in for ``errors::Internal`` raised by the OpKernel when the launcher
    fails (src/tensorflow_ops/sm120_ops_fixed.cc:145-146)."""


try:
    _b.load_library()
    _SM120_AVAILABLE = True
except Exception as _e:  # same warning site as python/sm120_ops.py:33-38, but nothing falls back later
    warnings.warn(f"SM120 operations library not found: {_e}. SM120 operations will raise.")
    _SM120_AVAILABLE = False


_TORCH_TO_SM120 = {
    torch.float32: _b.DTYPE_FLOAT32,
    torch.float16: _b.DTYPE_FLOAT16,
    torch.bfloat16: _b.DTYPE_BFLOAT16,
    torch.float8_e4m3fn: _b.DTYPE_FP8_E4M3,
}

_ACTIVATIONS = {
    None: _b.ACT_NONE, "linear": _b.ACT_NONE, "none": _b.ACT_NONE,
    "relu": _b.ACT_RELU, "leaky_relu": _b.ACT_LEAKY_RELU, "elu": _b.ACT_ELU, "selu": _b.ACT_SELU,
    "gelu": _b.ACT_GELU_ERF, "gelu_erf": _b.ACT_GELU_ERF, "gelu_tanh": _b.ACT_GELU_TANH,
    "swish": _b.ACT_SWISH, "silu": _b.ACT_SWISH, "mish": _b.ACT_MISH, "tanh": _b.ACT_TANH,
    "sigmoid": _b.ACT_SIGMOID,
}


def activation_code(activation: Union[None, str, int]) -> int:
    """Epilogue code for a Keras-style activation name.  ``"gelu"`` is the exact
    (erf) GELU, as in Keras; ``"gelu_tanh"`` is the reference's C-interface GELU."""
    if isinstance(activation, int):
        if not (-1 <= activation <= 9):
            raise ValueError(f"unknown activation code {activation}")
        return activation
    key = activation.lower() if isinstance(activation, str) else activation
    if key not in _ACTIVATIONS:
        raise ValueError(f"activation {activation!r} is not implemented by the fused epilogue")
    return _ACTIVATIONS[key]


def is_sm120_available() -> bool:
    """True when the library is loaded and a supported GPU is visible.  The
    reference requires compute capability >= (12, 0) (python/sm120_ops.py:56);
    this build requires 10.x (B200)."""
    if not _SM120_AVAILABLE:
        return False
    try:
        if not torch.cuda.is_available():
            return False
        lib = _b.load_library()
        return any(bool(lib.sm120_is_supported(i)) for i in range(torch.cuda.device_count()))
    except Exception:
        return False


def get_sm120_device_info() -> Dict[str, Any]:
    """Same keys as python/sm120_ops.py:66-105."""
    info: Dict[str, Any] = {"available": False, "devices": [], "library_loaded": _SM120_AVAILABLE}
    if not _SM120_AVAILABLE or not torch.cuda.is_available():
        return info
    lib = _b.load_library()
    for i in range(torch.cuda.device_count()):
        try:
            props = torch.cuda.get_device_properties(i)
            cc = (props.major, props.minor)
            ok = bool(lib.sm120_is_supported(i))
            info["devices"].append({
                "index": i, "name": props.name, "compute_capability": cc, "sm120_compatible": ok,
                "details": {"multi_processor_count": props.multi_processor_count, "total_memory": props.total_memory},
            })
            info["available"] = info["available"] or ok
        except Exception as e:  # pragma: no cover
            info["devices"].append({"index": i, "error": str(e)})
    return info


class SM120Config:
    """Configuration class for SM120 operations (python/sm120_ops.py:108-135).

    ``fallback_to_standard`` is kept for source compatibility; this build has no
    standard implementation to fall back to, so the flag has no effect."""

    def __init__(self):
        self.optimization_level = 1  # 0 = conservative tile, 1/2 = tuned tile choice
        self.use_tensor_cores = True
        self.enable_profiling = False
        self.memory_optimization = True
        self.fallback_to_standard = True

    def set_optimization_level(self, level: int) -> None:
        if level not in [0, 1, 2]:
            raise ValueError("Optimization level must be 0, 1, or 2")
        self.optimization_level = level

    def enable_tensor_cores(self, enable: bool = True) -> None:
        self.use_tensor_cores = enable

    def enable_memory_optimization(self, enable: bool = True) -> None:
        self.memory_optimization = enable


_config = SM120Config()


def get_config() -> SM120Config:
    return _config


# ---------------------------------------------------------------------------
# host <-> device plumbing
# ---------------------------------------------------------------------------
def _numpy_to_torch(x: np.ndarray) -> torch.Tensor:
    """Zero-copy view of a numpy array as a CPU torch tensor, including the
    ml_dtypes types torch.from_numpy does not know."""
    x = np.ascontiguousarray(x)
    if _ml is not None and x.dtype == np.dtype(_ml.bfloat16):
        return torch.from_numpy(x.view(np.uint16)).view(torch.bfloat16)
    if _ml is not None and x.dtype == np.dtype(_ml.float8_e4m3fn):
        return torch.from_numpy(x.view(np.uint8)).view(torch.float8_e4m3fn)
    return torch.from_numpy(x)


def _torch_to_numpy(t: torch.Tensor) -> np.ndarray:
    t = t.contiguous()
    if t.dtype == torch.bfloat16:
        return t.view(torch.uint16).numpy().view(_ml.bfloat16)
    if t.dtype == torch.float8_e4m3fn:
        return t.view(torch.uint8).numpy().view(_ml.float8_e4m3fn)
    return t.numpy()


def _require_available() -> None:
    if not _SM120_AVAILABLE:
        raise UnimplementedError("SM120 operations library is not loaded and there is no fallback")
    if not torch.cuda.is_available():
        raise UnimplementedError("SM120 operations need a CUDA device (compute capability 10.x); there is no CPU fallback")


def _row_major_2d(t: torch.Tensor) -> bool:
    return t.stride(-1) == 1 and (t.shape[-2] == 1 or t.stride(-2) >= t.shape[-1])


_WORKSPACES: Dict[Any, torch.Tensor] = {}


_SM_COUNTS: Dict[int, int] = {}


def _few_tiles(device: torch.device, m: int, n: int) -> bool:
    """Could the launcher want to split K?  Only when the output tiles (256 x 256 above 128 rows, else 128 x 128)
    leave at least half of the SMs idle; asking the library for the workspace size is skipped otherwise."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    sms = _SM_COUNTS.get(idx)
    if sms is None:
        sms = _SM_COUNTS[idx] = torch.cuda.get_device_properties(idx).multi_processor_count
    if m > 128:
        return 2 * ((m + 255) // 256) * ((n + 255) // 256) <= sms // 2
    return 2 * ((n + 127) // 128) <= sms


def _workspace(device: torch.device, nbytes: int) -> torch.Tensor:
    """A scratch buffer of at least `nbytes` for the current stream of `device`, reused by
    later calls on that stream (which orders the launches that use it).  Streams do not
    share a buffer, and a buffer that is replaced by a larger one stays reserved until
    the work already queued on its stream has finished."""
    stream = torch.cuda.current_stream(device)
    key = (device.type, device.index, stream.cuda_stream)
    ws = _WORKSPACES.get(key)
    if ws is None or ws.numel() < nbytes:
        if ws is not None:
            ws.record_stream(stream)
        ws = torch.empty(nbytes, dtype=torch.uint8, device=device)
        _WORKSPACES[key] = ws
    return ws


class _HostPipeline:
    """Per-device state of the host-operand path: one stream per copy direction and
    device staging buffers that are kept between calls."""

    MIN_ROWS = 256        # a chunk is a whole number of 256-row tiles
    # Shares of the rows per chunk, largest first.  The link carries both directions at once only at a reduced
    # rate per direction, and every copy has a fixed cost, so few chunks are better than many; what the chunking
    # must keep short is the tail after the last rows of A have arrived (their product and their trip back),
    # hence a small last chunk.  Measured on fp16 4096^3: 1.60 ms with four equal chunks, 1.72 ms with eight.
    SHARES = (0.375, 0.25, 0.1875, 0.125, 0.0625)

    @classmethod
    def chunk_rows(cls, m: int) -> List[int]:
        """Row counts of the chunks of an m-row operand (multiples of MIN_ROWS except the last)."""
        out, left = [], m
        for share in cls.SHARES[:-1]:
            rows = max(cls.MIN_ROWS, int(round(m * share / cls.MIN_ROWS)) * cls.MIN_ROWS)
            if left - rows < cls.MIN_ROWS:
                break
            out.append(rows)
            left -= rows
        out.append(left)
        return out

    def __init__(self, device: torch.device):
        self.device = device
        self.h2d = torch.cuda.Stream(device=device)
        self.d2h = torch.cuda.Stream(device=device)
        self._staging: Dict[str, torch.Tensor] = {}

    def staging(self, role: str, shape, dtype: torch.dtype) -> torch.Tensor:
        """A device tensor of `shape` / `dtype` carved from this role's buffer, which grows on demand."""
        nbytes = 1
        for e in shape:
            nbytes *= int(e)
        nbytes = max(16, nbytes * torch.empty((), dtype=dtype).element_size())
        buf = self._staging.get(role)
        if buf is None or buf.numel() < nbytes:
            buf = torch.empty(nbytes, dtype=torch.uint8, device=self.device)
            self._staging[role] = buf
        return buf[:nbytes].view(dtype).view(*shape)


_HOST_PIPELINES: Dict[int, _HostPipeline] = {}


def _host_pipelined(a: torch.Tensor, b: torch.Tensor, bias, host_out: Optional[torch.Tensor], out_dtype, kwargs) -> torch.Tensor:
    """C = op for HOST operands a [M, K] and b, as a three-stage pipeline over row chunks of A:
    B travels first; then chunk i+1 of A goes to the device on one copy stream while chunk i is
    multiplied on the caller's stream and chunk i-1 of C returns on a second copy stream (PCIe is
    full duplex).  Every copy is one plain asynchronous memcpy.  Returns the host result (pinned)."""
    dev = torch.device("cuda", torch.cuda.current_device())
    pipe = _HOST_PIPELINES.get(dev.index)
    if pipe is None:
        pipe = _HOST_PIPELINES[dev.index] = _HostPipeline(dev)
    M, K = a.shape
    N = b.shape[0] if kwargs.get("transpose_b") else b.shape[1]
    if out_dtype is None:
        out_dtype = torch.bfloat16 if a.dtype == torch.float8_e4m3fn else a.dtype
    if host_out is None:
        host_out = torch.empty((M, N), dtype=out_dtype, pin_memory=True)
    elif tuple(host_out.shape) != (M, N) or host_out.dtype != out_dtype or not host_out.is_contiguous():
        raise ValueError(f"host `out` must be a contiguous {out_dtype} tensor of shape {(M, N)}")
    a = a.contiguous()
    b = b.contiguous()
    a_dev = pipe.staging("a", a.shape, a.dtype)
    b_dev = pipe.staging("b", b.shape, b.dtype)
    c_dev = pipe.staging("c", (M, N), out_dtype)
    main = torch.cuda.current_stream(dev)
    pipe.h2d.wait_stream(main)              # earlier work on the caller's stream may still read the staging buffers
    pipe.d2h.wait_stream(main)
    with torch.cuda.stream(pipe.h2d):
        b_dev.copy_(b, non_blocking=True)
        if isinstance(bias, torch.Tensor) and not bias.is_cuda:
            bias_dev = pipe.staging("bias", bias.shape, bias.dtype)
            bias_dev.copy_(bias, non_blocking=True)
            bias = bias_dev
    r1 = 0
    for rows in _HostPipeline.chunk_rows(M):
        r0, r1 = r1, r1 + rows
        with torch.cuda.stream(pipe.h2d):
            a_dev[r0:r1].copy_(a[r0:r1], non_blocking=True)
            arrived = torch.cuda.Event()
            arrived.record(pipe.h2d)
        main.wait_event(arrived)            # also orders B and the bias, copied earlier on the same stream
        fused_matmul(a_dev[r0:r1], b_dev, bias=bias, out=c_dev[r0:r1], out_dtype=out_dtype, **kwargs)
        computed = torch.cuda.Event()
        computed.record(main)
        with torch.cuda.stream(pipe.d2h):
            pipe.d2h.wait_event(computed)
            host_out[r0:r1].copy_(c_dev[r0:r1], non_blocking=True)
    pipe.d2h.synchronize()                  # the host result is complete when the call returns
    return host_out


def fused_matmul(
    a, b, *,
    transpose_a: bool = False,
    transpose_b: bool = False,
    bias=None,
    activation: Union[None, str, int] = None,
    alpha: float = 1.0,
    beta: float = 0.0,
    out: Optional[torch.Tensor] = None,
    out_dtype: Optional[torch.dtype] = None,
    scale_a: Union[float, torch.Tensor, None] = None,
    scale_b: Union[float, torch.Tensor, None] = None,
    use_tensor_cores: Optional[bool] = None,
    optimization_level: Optional[int] = None,
    fp32_tensor_cores: Optional[bool] = None,
    peer_outs: Optional[Sequence[torch.Tensor]] = None,
    tuning: int = 0,
    trace: Optional[torch.Tensor] = None,
):
    """out = act(alpha / (scale_a * scale_b) * op(a) @ op(b) + beta * out + bias).

    The full form of the op (``sm120_launch_matmul_ex``).  ``a`` and ``b`` are
    rank-2, or rank-3 with a leading batch dimension (a rank-2 operand is
    broadcast over the batch).  FP8 inputs (``torch.float8_e4m3fn``) produce
    bfloat16 unless ``out_dtype`` says otherwise.  ``scale_a`` / ``scale_b`` are the
    per-tensor quantisation scales (floats, or one-element CUDA float32 tensors
    that a producer kernel wrote).

    float32 operands of a large product (at least 2^24 multiply-adds) run on the tensor
    cores by the 3xTF32 split, whose partial sums are promoted to round-to-nearest fp32
    every 192 products so that the result stays inside the op's 1e-5 gate; smaller ones,
    and everything with ``use_tensor_cores=False`` or ``fp32_tensor_cores=False``, run on
    the exact FFMA kernel.  ``fp32_tensor_cores=True`` forces the tensor cores.

    ``peer_outs`` (used by ``mshard``): up to 7 more destinations, tensors or raw device
    addresses (other GPUs' memory opened through CUDA IPC), that receive the same
    result as ``out`` from the same launch (``sm120_launch_matmul_gather``); they use
    ``out``'s shape, dtype and strides.

    ``tuning`` passes ``SM120_TUNE_*`` bits (``_binding.TUNE_*``) to this one launch;
    ``trace`` is a CUDA int64 tensor of at least ``_binding.TRACE_BYTES // 8`` words
    that receives the launch's timeline (``SM120_TUNE_TRACE``).  Both are for tests
    and tuning runs.

    Inputs on the host (numpy arrays or CPU tensors) are copied to the current
    CUDA device, and the result is copied back and returned in the same form;
    `out` may then be a host buffer (ideally pinned) that receives the result.
    """
    host_kind = None
    if isinstance(a, np.ndarray) or isinstance(b, np.ndarray):
        host_kind = "numpy"
        a = _numpy_to_torch(a) if isinstance(a, np.ndarray) else a
        b = _numpy_to_torch(b) if isinstance(b, np.ndarray) else b
        if isinstance(bias, np.ndarray):
            bias = _numpy_to_torch(bias)
    if not isinstance(a, torch.Tensor) or not isinstance(b, torch.Tensor):
        raise TypeError("a and b must be torch tensors or numpy arrays")
    if a.dtype != b.dtype:
        raise ValueError(f"Input tensors must have the same dtype, got {a.dtype} and {b.dtype}")
    if a.dtype not in _TORCH_TO_SM120:
        raise ValueError(f"dtype {a.dtype} is not supported (float32, float16, bfloat16, float8_e4m3fn)")
    if a.dim() not in (2, 3) or b.dim() not in (2, 3):
        raise ValueError("Input tensors must be 2-dimensional (or 3-dimensional with a leading batch dimension)")
    if not a.is_cuda and host_kind is None:
        host_kind = "torch"

    # shapes under the transposes (src/tensorflow_ops/sm120_ops_fixed.cc:121-127)
    M, Ka = (a.shape[-1], a.shape[-2]) if transpose_a else (a.shape[-2], a.shape[-1])
    Kb, N = (b.shape[-1], b.shape[-2]) if transpose_b else (b.shape[-2], b.shape[-1])
    if Ka != Kb:
        raise InvalidArgumentError(f"Matrix dimensions must be compatible: inner dimensions {Ka} and {Kb}")
    K = Ka
    batch = 1
    if a.dim() == 3 or b.dim() == 3:
        ba = a.shape[0] if a.dim() == 3 else None
        bb = b.shape[0] if b.dim() == 3 else None
        if ba is not None and bb is not None and ba != bb:
            raise InvalidArgumentError(f"batch dimensions differ: {ba} and {bb}")
        batch = ba if ba is not None else bb
        if batch < 1:
            raise InvalidArgumentError("empty batch")

    # everything above is pure validation; from here on a device is needed
    _require_available()
    host_out = None
    if host_kind is not None and isinstance(out, np.ndarray):
        out = _numpy_to_torch(out)
    if host_kind is not None and isinstance(out, torch.Tensor) and not out.is_cuda:
        # a host result buffer (pinned for an asynchronous copy): the device result is copied into it
        if beta != 0.0:
            raise ValueError("beta != 0 is not supported with host operands")
        host_out, out = out, None
    if (host_kind is not None and not a.is_cuda and not b.is_cuda and a.dim() == 2 and b.dim() == 2 and not transpose_a
            and out is None and beta == 0.0 and not peer_outs and trace is None
            and not isinstance(scale_a, torch.Tensor) and not isinstance(scale_b, torch.Tensor)
            and M >= 2 * _HostPipeline.MIN_ROWS and N >= 1 and K >= 1):
        # large host operands: copies and products overlap chunk by chunk
        host = _host_pipelined(a, b, bias, host_out, out_dtype,
                               dict(transpose_b=transpose_b, activation=activation, alpha=alpha, scale_a=scale_a, scale_b=scale_b,
                                    use_tensor_cores=use_tensor_cores, optimization_level=optimization_level, tuning=tuning,
                                    fp32_tensor_cores=fp32_tensor_cores))
        return _torch_to_numpy(host) if host_kind == "numpy" else host
    if host_kind is not None:
        dev = torch.device("cuda", torch.cuda.current_device())
        a = a.to(dev, non_blocking=True)
        b = b.to(dev, non_blocking=True)
        if isinstance(bias, torch.Tensor) and not bias.is_cuda:
            bias = bias.to(dev, non_blocking=True)
    if a.device != b.device:
        raise ValueError(f"a and b are on different devices: {a.device} and {b.device}")

    if not _row_major_2d(a):
        a = a.contiguous()
    if not _row_major_2d(b):
        b = b.contiguous()

    in_code = _TORCH_TO_SM120[a.dtype]
    if out_dtype is None:
        out_dtype = out.dtype if out is not None else (torch.bfloat16 if a.dtype == torch.float8_e4m3fn else a.dtype)
    if out_dtype not in _TORCH_TO_SM120 or out_dtype == torch.float8_e4m3fn:
        raise ValueError(f"output dtype {out_dtype} is not supported")
    out_shape = (batch, M, N) if (a.dim() == 3 or b.dim() == 3) else (M, N)
    if out is None:
        if beta != 0.0:
            raise ValueError("beta != 0 needs `out` to hold the matrix to accumulate into")
        out = torch.empty(out_shape, dtype=out_dtype, device=a.device)
    else:
        if tuple(out.shape) != tuple(out_shape) or out.dtype != out_dtype or out.device != a.device:
            raise ValueError(f"`out` must be a {out_dtype} tensor of shape {out_shape} on {a.device}")
        if not _row_major_2d(out) or (out.dim() == 3 and out.stride(0) < M * out.stride(-2)):
            raise ValueError("`out` must be row-major")

    d = _b.new_desc()
    d.in_dtype = in_code
    d.out_dtype = _TORCH_TO_SM120[out_dtype]
    d.A, d.B, d.C = a.data_ptr(), b.data_ptr(), out.data_ptr()
    d.M, d.N, d.K = M, N, K
    d.lda = a.stride(-2) if a.shape[-2] > 1 else a.shape[-1]
    d.ldb = b.stride(-2) if b.shape[-2] > 1 else b.shape[-1]
    d.ldc = out.stride(-2) if out.shape[-2] > 1 else out.shape[-1]
    d.batch = batch
    d.stride_a = a.stride(0) if a.dim() == 3 and batch > 1 else 0
    d.stride_b = b.stride(0) if b.dim() == 3 and batch > 1 else 0
    d.stride_c = out.stride(0) if out.dim() == 3 and batch > 1 else 0
    d.transpose_a, d.transpose_b = int(bool(transpose_a)), int(bool(transpose_b))
    d.alpha, d.beta = float(alpha), float(beta)
    keep = [a, b, out]
    for name, s in (("a", scale_a), ("b", scale_b)):
        if s is None:
            continue
        if isinstance(s, torch.Tensor):
            if not s.is_cuda or s.dtype != torch.float32 or s.numel() != 1:
                raise ValueError("a tensor scale must be a one-element float32 CUDA tensor")
            keep.append(s)
            setattr(d, f"scale_{name}_dev", s.data_ptr())
        else:
            if not (float(s) > 0.0):
                raise ValueError("scales must be positive")
            setattr(d, f"scale_{name}", float(s))
    if bias is not None:
        if not isinstance(bias, torch.Tensor):
            raise TypeError("bias must be a tensor")
        if bias.dim() != 1 or bias.shape[0] != N:
            raise InvalidArgumentError(f"bias must have shape [{N}], got {tuple(bias.shape)}")
        if bias.dtype not in (torch.float32, torch.float16, torch.bfloat16):
            raise ValueError(f"bias dtype {bias.dtype} is not supported")
        bias = bias.to(a.device).contiguous()
        keep.append(bias)
        d.bias = bias.data_ptr()
        d.bias_dtype = _TORCH_TO_SM120[bias.dtype]
    d.activation = activation_code(activation)
    if use_tensor_cores is None:
        use_tensor_cores = _config.use_tensor_cores
    if optimization_level is None:
        optimization_level = _config.optimization_level
    if optimization_level not in (0, 1, 2):
        raise ValueError("Optimization level must be 0, 1, or 2")
    d.optimization_level = int(optimization_level)
    d.path = _b.PATH_AUTO if use_tensor_cores else _b.PATH_SIMT
    d.tuning = int(tuning)
    if trace is not None:
        if not (trace.is_cuda and trace.dtype == torch.int64 and trace.is_contiguous() and trace.numel() * 8 >= _b.TRACE_BYTES):
            raise ValueError(f"trace must be a contiguous CUDA int64 tensor of at least {_b.TRACE_BYTES // 8} words")
        keep.append(trace)
        d.tuning |= _b.TUNE_TRACE
        d.workspace, d.workspace_bytes = trace.data_ptr(), trace.numel() * 8
    d.stream = torch.cuda.current_stream(a.device).cuda_stream
    if a.dtype == torch.float32 and K >= 1 and trace is None and use_tensor_cores and fp32_tensor_cores is not False and (
            fp32_tensor_cores or M * N * K * batch >= 1 << 24):
        # 3xTF32: scratch for the split operands comes from the caller's allocator (torch), is kept per
        # stream and grows to the largest request; with it the launcher's AUTO takes the tensor cores
        need = int(_b.load_library().sm120_matmul_workspace_bytes(ctypes.byref(d)))
        ws = _workspace(a.device, max(need, 16))
        keep.append(ws)
        d.workspace, d.workspace_bytes = ws.data_ptr(), ws.numel()
        if fp32_tensor_cores:
            d.path = _b.PATH_TENSOR_CORE
    elif (a.dtype != torch.float32 and batch == 1 and trace is None and use_tensor_cores and not peer_outs and K >= 1024
          and _few_tiles(a.device, M, N)):
        # few output tiles and a long K: the launcher splits K when it is given room for the partial sums
        need = int(_b.load_library().sm120_matmul_workspace_bytes(ctypes.byref(d)))
        if need:
            ws = _workspace(a.device, need)
            keep.append(ws)
            d.workspace, d.workspace_bytes = ws.data_ptr(), ws.numel()

    if peer_outs:
        if host_kind is not None or beta != 0.0:
            raise ValueError("peer_outs needs device operands and beta == 0")
        addrs = []
        for t in peer_outs:
            if isinstance(t, torch.Tensor):
                if not (t.is_cuda and tuple(t.shape) == tuple(out.shape) and t.dtype == out.dtype and t.stride() == out.stride()):
                    raise ValueError("every peer output must match `out` in shape, dtype and strides")
                keep.append(t)
                addrs.append(t.data_ptr())
            else:
                addrs.append(int(t))           # a raw device address (memory of another process, opened through IPC)
        ptrs = (ctypes.c_void_p * len(addrs))(*addrs)
        with torch.cuda.device(a.device):
            rc = _b.load_library().sm120_launch_matmul_gather(ctypes.byref(d), ptrs, len(addrs))
    else:
        with torch.cuda.device(a.device):
            rc = _b.load_library().sm120_launch_matmul_ex(ctypes.byref(d))
    if rc == _b.CUDA_ERROR_INVALID_VALUE:
        raise InvalidArgumentError("SM120MatMul rejected its arguments (cudaErrorInvalidValue)")
    if rc != _b.CUDA_SUCCESS:
        raise InternalError(f"SM120MatMul failed: {_b.error_string(rc)}")

    if host_kind is None:
        return out
    if host_out is not None:
        if tuple(host_out.shape) != tuple(out.shape) or host_out.dtype != out.dtype:
            raise ValueError(f"host `out` must be a {out.dtype} tensor of shape {tuple(out.shape)}")
        host_out.copy_(out, non_blocking=True)
        torch.cuda.current_stream(a.device).synchronize()
        host = host_out
    else:
        host = out.to("cpu")      # synchronises with the launch stream
    return _torch_to_numpy(host) if host_kind == "numpy" else host


def advanced_matmul(
    a,
    b,
    transpose_a: bool = False,
    transpose_b: bool = False,
    use_tensor_cores: Optional[bool] = None,
    optimization_level: Optional[int] = None,
    name: Optional[str] = None,
):
    """Matrix product of two rank-2 tensors: the op ``SM120AdvancedMatMul`` /
    ``SM120MatMul``.  Signature, defaults and the two ``ValueError`` checks are
    those of python/sm120_ops.py:142-184.  ``a`` is [M, K] (or [K, M] with
    ``transpose_a``), ``b`` is [K, N] (or [N, K] with ``transpose_b``); the result
    is [M, N] in the inputs' dtype (bfloat16 for FP8 inputs).

    Raises ``ValueError`` for mixed dtypes or rank != 2, ``InvalidArgumentError``
    for incompatible inner dimensions, ``UnimplementedError`` when no supported
    GPU or library is present (there is no fallback)."""
    del name
    if hasattr(a, "dtype") and hasattr(b, "dtype") and a.dtype != b.dtype:
        raise ValueError(f"Input tensors must have the same dtype, got {a.dtype} and {b.dtype}")
    if len(a.shape) != 2 or len(b.shape) != 2:
        raise ValueError("Input tensors must be 2-dimensional")
    return fused_matmul(a, b, transpose_a=transpose_a, transpose_b=transpose_b, use_tensor_cores=use_tensor_cores,
                        optimization_level=optimization_level)


# names other files of the reference call (python/benchmark.py:65, python/validate.py:158)
sm120_matmul = advanced_matmul


def batched_matmul(a, b, transpose_a: bool = False, transpose_b: bool = False, **kwargs):
    """Strided-batch product C[i] = op(a[i]) @ op(b[i]) for rank-3 operands: the
    semantics of LaunchSM120DynamicMatMul
    (src/cuda_kernels/sm120_dynamic_shapes.cu:107-183,323-383)."""
    if len(a.shape) != 3 and len(b.shape) != 3:
        raise ValueError("batched_matmul needs at least one rank-3 operand")
    return fused_matmul(a, b, transpose_a=transpose_a, transpose_b=transpose_b, **kwargs)


def matmul_grad(grad_c, a, b):
    """Gradients of C = a @ b (no transposes): (grad_c @ b^T, a^T @ grad_c), the
    two products of SM120MatMulGradA / SM120MatMulGradB
    (src/tensorflow_ops/sm120_gradients.cc:22-55)."""
    return (fused_matmul(grad_c, b, transpose_b=True), fused_matmul(a, grad_c, transpose_a=True))


def fused_activation(x: torch.Tensor, activation: Union[None, str, int], bias: Optional[torch.Tensor] = None,
                     out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """act(x + bias) as one HBM-bound pass: the op ``SM120FusedActivation``
    (src/tensorflow_ops/sm120_ops.cc:251-326) over ``sm120_launch_activation``
    (src/cuda_kernels/sm120_c_interface.cu:139-164), with the bias add of
    ``tf.nn.bias_add`` (python/sm120_keras_layers.py:169) folded into the same kernel
    when a bias is given.  `x` is a contiguous CUDA tensor (float32, float16 or
    bfloat16); `bias` has x.shape[-1] entries; `out` may be `x` itself."""
    _require_available()
    if not isinstance(x, torch.Tensor) or not x.is_cuda:
        raise TypeError("fused_activation needs a CUDA tensor")
    if x.dtype not in (torch.float32, torch.float16, torch.bfloat16):
        raise ValueError(f"dtype {x.dtype} is not supported (float32, float16, bfloat16)")
    x = x.contiguous()
    if out is None:
        out = torch.empty_like(x)
    elif not (out.is_cuda and out.is_contiguous() and out.shape == x.shape and out.dtype == x.dtype and out.device == x.device):
        raise ValueError("`out` must be a contiguous CUDA tensor with x's shape, dtype and device")
    code = activation_code(activation)
    cols = x.shape[-1] if x.dim() >= 1 else 1
    rows = x.numel() // cols if cols else 0
    bias_ptr, bias_code = None, 0
    if bias is not None:
        if not (isinstance(bias, torch.Tensor) and bias.is_cuda and bias.dim() == 1 and bias.shape[0] == cols):
            raise InvalidArgumentError(f"bias must be a CUDA tensor of shape [{cols}]")
        if bias.dtype not in (torch.float32, torch.float16, torch.bfloat16):
            raise ValueError(f"bias dtype {bias.dtype} is not supported")
        bias = bias.contiguous()
        bias_ptr, bias_code = bias.data_ptr(), _TORCH_TO_SM120[bias.dtype]
    stream = torch.cuda.current_stream(x.device).cuda_stream
    with torch.cuda.device(x.device):
        rc = _b.load_library().sm120_launch_bias_activation(x.data_ptr(), bias_ptr, bias_code, out.data_ptr(), rows, cols, code,
                                                            _TORCH_TO_SM120[x.dtype], stream)
    if rc == _b.CUDA_ERROR_INVALID_VALUE:
        raise InvalidArgumentError("fused_activation rejected its arguments (cudaErrorInvalidValue)")
    if rc != _b.CUDA_SUCCESS:
        raise InternalError(f"fused_activation failed: {_b.error_string(rc)}")
    return out


def bias_grad(grad_c: torch.Tensor, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """Gradient of a Dense bias: the column sums of `grad_c` (any leading
    dimensions are flattened into rows), accumulated in fp32 in a fixed order
    (``sm120_launch_bias_grad``).  Result dtype: grad_c's, or float32 on request."""
    _require_available()
    if not isinstance(grad_c, torch.Tensor) or not grad_c.is_cuda or grad_c.dim() < 1:
        raise TypeError("bias_grad needs a CUDA tensor of rank >= 1")
    if grad_c.dtype not in (torch.float32, torch.float16, torch.bfloat16):
        raise ValueError(f"dtype {grad_c.dtype} is not supported (float32, float16, bfloat16)")
    out_dtype = out_dtype or grad_c.dtype
    if out_dtype not in (torch.float32, grad_c.dtype):
        raise ValueError("out_dtype must be float32 or grad_c's dtype")
    n = grad_c.shape[-1]
    g = grad_c.reshape(-1, n)
    if g.stride(-1) != 1 or (g.shape[0] > 1 and g.stride(0) < n):
        g = g.contiguous()
    out = torch.empty(n, dtype=out_dtype, device=g.device)
    ld = g.stride(0) if g.shape[0] > 1 else n
    with torch.cuda.device(g.device):
        rc = _b.load_library().sm120_launch_bias_grad(g.data_ptr(), out.data_ptr(), g.shape[0], n, ld, _TORCH_TO_SM120[g.dtype],
                                                      _TORCH_TO_SM120[out_dtype], torch.cuda.current_stream(g.device).cuda_stream)
    if rc == _b.CUDA_ERROR_INVALID_VALUE:
        raise InvalidArgumentError("bias_grad rejected its arguments (cudaErrorInvalidValue)")
    if rc != _b.CUDA_SUCCESS:
        raise InternalError(f"bias_grad failed: {_b.error_string(rc)}")
    return out


def softmax(x: torch.Tensor, axis: int = -1, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Softmax along `axis` (``sm120_launch_softmax``; the reference kernel is
    src/cuda_kernels/sm120_pure_kernels.cu:471-550).  fp32 math, result in x's dtype."""
    _require_available()
    if not isinstance(x, torch.Tensor) or not x.is_cuda:
        raise TypeError("softmax needs a CUDA tensor")
    if x.dtype not in (torch.float32, torch.float16, torch.bfloat16):
        raise ValueError(f"dtype {x.dtype} is not supported (float32, float16, bfloat16)")
    x = x.contiguous()
    axis = axis % x.dim()
    outer = 1
    for e in x.shape[:axis]:
        outer *= int(e)
    inner = 1
    for e in x.shape[axis + 1:]:
        inner *= int(e)
    if max(outer, x.shape[axis], inner) >= 1 << 31:
        raise InvalidArgumentError("softmax extents must fit in 31 bits")
    if out is None:
        out = torch.empty_like(x)
    elif not (out.is_cuda and out.is_contiguous() and out.shape == x.shape and out.dtype == x.dtype):
        raise ValueError("`out` must be a contiguous CUDA tensor with x's shape and dtype")
    with torch.cuda.device(x.device):
        rc = _b.load_library().sm120_launch_softmax(x.data_ptr(), out.data_ptr(), outer, int(x.shape[axis]), inner,
                                                    _TORCH_TO_SM120[x.dtype], torch.cuda.current_stream(x.device).cuda_stream)
    if rc != _b.CUDA_SUCCESS:
        raise (InvalidArgumentError if rc == _b.CUDA_ERROR_INVALID_VALUE else InternalError)(f"softmax failed: {_b.error_string(rc)}")
    return out


def scaled_dot_product_attention(query: torch.Tensor, key: torch.Tensor, value: torch.Tensor, scale: Optional[float] = None,
                                 dropout_rate: float = 0.0, attention_mask: Optional[torch.Tensor] = None,
                                 causal_mask: bool = False, return_attention_scores: bool = False):
    """softmax(scale * Q K^T + mask) V over the last two dimensions: the attention core
    that ``SM120MultiHeadAttention`` calls (python/sm120_keras_layers.py:796-806) and
    ``flash_attention`` wraps (python/sm120_ops.py:315-407).

    query [..., Sq, D], key and value [..., Sk, D] (the same leading dimensions, e.g.
    [batch, heads]).  ``attention_mask`` follows the layer's convention
    (python/sm120_keras_layers.py:815-816): a tensor broadcastable to [..., Sq, Sk] whose
    non-zero entries mark positions to EXCLUDE (it is multiplied by -1e9 and added to the
    scores).  ``causal_mask`` drops keys after the query position (aligned to the end).

    float16 / bfloat16 with D = 64 or 128 and no explicit mask run ONE fused tcgen05
    kernel: the scores never reach HBM.  A mask, float32 tensors, other head sizes and
    ``return_attention_scores`` run as batched GEMM + softmax + batched GEMM on this
    library's kernels.  Returns the output (in the inputs' dtype), or (output, weights)
    with fp32 weights.  Dropout is a training-time feature this build does not have."""
    _require_available()
    if dropout_rate and dropout_rate > 0.0:
        raise NotImplementedError("attention dropout is not implemented in this build")
    for t in (query, key, value):
        if not isinstance(t, torch.Tensor) or not t.is_cuda:
            raise TypeError("query, key and value must be CUDA tensors")
    if not (query.dtype == key.dtype == value.dtype):
        raise ValueError("query, key and value must have the same dtype")
    if query.dtype not in (torch.float32, torch.float16, torch.bfloat16):
        raise ValueError(f"dtype {query.dtype} is not supported (float32, float16, bfloat16)")
    if query.dim() < 2 or key.dim() != query.dim() or value.dim() != query.dim():
        raise ValueError("query, key and value must have the same rank (at least 2)")
    lead = tuple(query.shape[:-2])
    sq, d = int(query.shape[-2]), int(query.shape[-1])
    sk = int(key.shape[-2])
    if tuple(key.shape[:-2]) != lead or tuple(value.shape[:-2]) != lead or key.shape[-1] != d or tuple(value.shape[-2:]) != (sk, d):
        raise InvalidArgumentError("query [..., Sq, D], key [..., Sk, D] and value [..., Sk, D] are required")
    if causal_mask and sq > sk:
        raise InvalidArgumentError("causal attention needs at least as many keys as queries")
    if scale is None:
        scale = 1.0 / float(d) ** 0.5
    bh = 1
    for e in lead:
        bh *= int(e)
    q3, k3, v3 = (t.reshape(bh, -1, d).contiguous() for t in (query, key, value))
    lib = _b.load_library()
    stream = torch.cuda.current_stream(query.device).cuda_stream
    code = _TORCH_TO_SM120[query.dtype]
    out = torch.empty((bh, sq, d), dtype=query.dtype, device=query.device)
    fused_ok = query.dtype != torch.float32 and d in (64, 128) and bh <= 65535
    if attention_mask is None and (fused_ok or query.dtype == torch.float32):
        weights = None
        if return_attention_scores or not fused_ok:
            weights = torch.empty((bh, sq, sk), dtype=torch.float32, device=query.device)
        with torch.cuda.device(query.device):
            rc = lib.sm120_launch_attention_ex(q3.data_ptr(), k3.data_ptr(), v3.data_ptr(), out.data_ptr(),
                                               None if weights is None else weights.data_ptr(), bh, sq, sk, d, float(scale),
                                               int(bool(causal_mask)), code, stream)
        if rc != _b.CUDA_SUCCESS:
            raise (InvalidArgumentError if rc == _b.CUDA_ERROR_INVALID_VALUE else InternalError)(
                f"attention failed: {_b.error_string(rc)}")
        out = out.reshape(*lead, sq, d)
        return (out, weights.reshape(*lead, sq, sk)) if return_attention_scores else out
    # unfused: scores (fp32) = Q K^T, probabilities = softmax(scale * scores + mask) in the inputs' dtype, out = P V
    scores = fused_matmul(q3, k3, transpose_b=True, out_dtype=torch.float32)
    mask_ptr, mask_rows = None, 0
    if attention_mask is not None:
        m = attention_mask.to(device=query.device, dtype=torch.float32)
        m = torch.broadcast_to(m, (*lead, sq, sk)).reshape(-1, sk) if m.dim() > 2 else torch.broadcast_to(m, (sq, sk))
        m = m.contiguous()                                     # [sq, sk] is shared by every batch entry: row r uses r % sq
        mask_ptr, mask_rows = m.data_ptr(), int(m.shape[0])
    p_dtype = query.dtype
    probs = scores if p_dtype == torch.float32 else torch.empty((bh, sq, sk), dtype=p_dtype, device=query.device)
    with torch.cuda.device(query.device):
        rc = lib.sm120_launch_softmax_ex(scores.data_ptr(), probs.data_ptr(), bh * sq, sk, _b.DTYPE_FLOAT32, _TORCH_TO_SM120[p_dtype],
                                         float(scale), mask_ptr, mask_rows, -1e9, int(bool(causal_mask)), sq, stream)
    if rc != _b.CUDA_SUCCESS:
        raise (InvalidArgumentError if rc == _b.CUDA_ERROR_INVALID_VALUE else InternalError)(f"softmax failed: {_b.error_string(rc)}")
    fused_matmul(probs, v3, out=out)
    out = out.reshape(*lead, sq, d)
    if return_attention_scores:
        return out, probs.float().reshape(*lead, sq, sk)
    return out


def flash_attention(queries: torch.Tensor, keys: torch.Tensor, values: torch.Tensor, attention_mask: Optional[torch.Tensor] = None,
                    scale: Optional[float] = None, causal_mask: bool = False, dropout_rate: float = 0.0,
                    name: Optional[str] = None):
    """Signature of python/sm120_ops.py:315-324: 4-dimensional [batch, heads, seq_len, head_dim]
    tensors, returns (attention_output, attention_weights).  Here ``attention_mask`` is ADDED to
    the scaled scores as it is (:400-401), unlike the layer's 0/1 convention."""
    del name
    if queries.dim() != 4 or keys.dim() != 4 or values.dim() != 4:
        raise ValueError("Queries, keys, and values must be 4-dimensional")
    if attention_mask is not None and attention_mask.numel() == 0:
        attention_mask = None
    if attention_mask is not None:
        # an additive mask: hand it to the softmax as (mask / -1e9) * -1e9
        attention_mask = attention_mask.to(torch.float32) / -1e9
    return scaled_dot_product_attention(queries, keys, values, scale=scale, dropout_rate=dropout_rate,
                                        attention_mask=attention_mask, causal_mask=causal_mask, return_attention_scores=True)


class _DenseFunction(torch.autograd.Function):
    """y = relu?(x @ kernel + bias) with this library's kernels in both directions:
    the fused GEMM forward, SM120MatMulGradA / GradB
    (src/tensorflow_ops/sm120_gradients.cc:22-55) and the bias column sum backward."""

    @staticmethod
    def forward(ctx, x, kernel, bias, relu):
        y = fused_matmul(x, kernel, bias=bias, activation="relu" if relu else None)
        ctx.save_for_backward(x, kernel, y if relu else None)
        ctx.has_bias = bias is not None
        return y

    @staticmethod
    def backward(ctx, grad_y):
        x, kernel, y = ctx.saved_tensors
        g = grad_y.contiguous()
        if y is not None:
            g = g * (y > 0).to(g.dtype)
        dx, dk = matmul_grad(g, x, kernel)
        db = bias_grad(g) if ctx.has_bias else None
        return dx, dk, db, None


def dense_trainable(x: torch.Tensor, kernel: torch.Tensor, bias: Optional[torch.Tensor] = None,
                    activation: Union[None, str] = None) -> torch.Tensor:
    """A Dense forward that torch autograd can differentiate through, for training
    loops like the reference's (tests/integration/test_comprehensive_validation.py:346-434):
    x [M, in], kernel [in, units], bias [units]; activation None / "linear" / "relu"."""
    if activation not in (None, "linear", "relu"):
        raise NotImplementedError("dense_trainable differentiates the linear and relu forms only")
    return _DenseFunction.apply(x, kernel, bias, activation == "relu")


def quantize_fp8(x: torch.Tensor, scale: Optional[torch.Tensor] = None):
    """Per-tensor FP8 quantisation for FP8 matmuls, on the device: returns
    (q, scale) with scale = 448 / amax(x) as a one-element float32 CUDA tensor and
    q = x * scale rounded to e4m3 with saturation
    (type and conversion: src/cuda_kernels/sm120_datatype_support.h:71-82,168-171).
    `scale` can be passed to ``fused_matmul(scale_a=...)`` as it is: nothing is
    copied to the host.  When `scale` is given (a one-element float32 CUDA tensor,
    e.g. 448 / the maximum over every shard of a tensor that is split across GPUs),
    only the cast runs and that scale is returned."""
    _require_available()
    if not isinstance(x, torch.Tensor) or not x.is_cuda:
        raise TypeError("quantize_fp8 needs a CUDA tensor")
    if x.dtype not in (torch.float32, torch.float16, torch.bfloat16):
        raise ValueError(f"dtype {x.dtype} cannot be quantised (float32, float16, bfloat16)")
    x = x.contiguous()
    lib = _b.load_library()
    n = x.numel()
    q = torch.empty(x.shape, dtype=torch.float8_e4m3fn, device=x.device)
    if scale is not None:
        if not (isinstance(scale, torch.Tensor) and scale.is_cuda and scale.dtype == torch.float32 and scale.numel() == 1
                and scale.device == x.device):
            raise ValueError("scale must be a one-element float32 CUDA tensor on x's device")
        with torch.cuda.device(x.device):
            rc = lib.sm120_launch_cast_fp8(x.data_ptr(), _TORCH_TO_SM120[x.dtype], n, scale.data_ptr(), q.data_ptr(),
                                           torch.cuda.current_stream(x.device).cuda_stream)
        if rc == _b.CUDA_ERROR_INVALID_VALUE:
            raise InvalidArgumentError("quantize_fp8 rejected its arguments (cudaErrorInvalidValue)")
        if rc != _b.CUDA_SUCCESS:
            raise InternalError(f"quantize_fp8 failed: {_b.error_string(rc)}")
        return q, scale
    scale = torch.empty(1, dtype=torch.float32, device=x.device)
    nbytes = int(lib.sm120_quantize_fp8_scratch_bytes(n))
    scratch = torch.empty(max(nbytes, 4), dtype=torch.uint8, device=x.device)     # the caller's allocator, not the library's
    with torch.cuda.device(x.device):
        rc = lib.sm120_launch_quantize_fp8(x.data_ptr(), _TORCH_TO_SM120[x.dtype], n, q.data_ptr(), scale.data_ptr(),
                                           scratch.data_ptr(), scratch.numel(), torch.cuda.current_stream(x.device).cuda_stream)
    if rc == _b.CUDA_ERROR_INVALID_VALUE:
        raise InvalidArgumentError("quantize_fp8 rejected its arguments (cudaErrorInvalidValue)")
    if rc != _b.CUDA_SUCCESS:
        raise InternalError(f"quantize_fp8 failed: {_b.error_string(rc)}")
    scratch.record_stream(torch.cuda.current_stream(x.device))
    return q, scale


def quantize_fp8_into(x: torch.Tensor, q: torch.Tensor, scale: torch.Tensor) -> None:
    """FP8 quantisation of `x` into buffers the caller already owns, with no
    allocation anywhere on the way (``sm120_launch_quantize_fp8_static``).

    For code that must not allocate device memory while it runs -- a callback
    that may use only the tensors it was given, a serving loop whose memory was
    fixed at start-up.  `q` (float8_e4m3fn, same number of elements as `x`) and
    `scale` (one float32) are written; the intermediate partial maxima live in
    a 16 KB array built into the library, which limits `x` to 268 435 456
    elements and means that two calls running at the same time on one GPU would
    disturb each other: keep them on one stream or order them.  The first call
    on a device also looks up that array's address, so make it before any
    stream capture starts."""
    _require_available()
    if not (isinstance(x, torch.Tensor) and x.is_cuda and x.is_contiguous()):
        raise TypeError("x must be a contiguous CUDA tensor")
    if x.dtype not in (torch.float32, torch.float16, torch.bfloat16):
        raise ValueError(f"dtype {x.dtype} cannot be quantised (float32, float16, bfloat16)")
    if not (q.is_cuda and q.is_contiguous() and q.dtype == torch.float8_e4m3fn and q.numel() == x.numel() and q.device == x.device):
        raise ValueError("q must be a contiguous float8_e4m3fn CUDA tensor with as many elements as x")
    if not (scale.is_cuda and scale.dtype == torch.float32 and scale.numel() == 1 and scale.device == x.device):
        raise ValueError("scale must be a one-element float32 CUDA tensor on x's device")
    if x.numel() > _b.QUANTIZE_FP8_STATIC_MAX_ELEMENTS:
        raise InvalidArgumentError(
            f"x has {x.numel()} elements; the allocation-free quantiser takes at most "
            f"{_b.QUANTIZE_FP8_STATIC_MAX_ELEMENTS} (use quantize_fp8 for larger tensors)")
    with torch.cuda.device(x.device):
        rc = _b.load_library().sm120_launch_quantize_fp8_static(
            x.data_ptr(), _TORCH_TO_SM120[x.dtype], x.numel(), q.data_ptr(), scale.data_ptr(),
            torch.cuda.current_stream(x.device).cuda_stream)
    if rc == _b.CUDA_ERROR_INVALID_VALUE:
        raise InvalidArgumentError("quantize_fp8_into rejected its arguments (cudaErrorInvalidValue)")
    if rc != _b.CUDA_SUCCESS:
        raise InternalError(f"quantize_fp8_into failed: {_b.error_string(rc)}")


class SM120Profiler:
    """Same interface as python/sm120_ops.py:415-445; times with a device
    synchronisation on both sides instead of ``tf.timestamp``."""

    def __init__(self, enabled: bool = True):
        self.enabled = enabled
        self.metrics: Dict[str, Dict[str, Any]] = {}

    def profile_operation(self, operation_name: str, operation_fn, *args, **kwargs):
        if not self.enabled:
            return operation_fn(*args, **kwargs)
        if torch.cuda.is_available():
            torch.cuda.synchronize()
        start = time.perf_counter()
        result = operation_fn(*args, **kwargs)
        if torch.cuda.is_available():
            torch.cuda.synchronize()
        self.metrics[operation_name] = {"execution_time": time.perf_counter() - start, "timestamp": start}
        return result

    def get_metrics(self) -> Dict[str, Any]:
        return self.metrics.copy()

    def clear_metrics(self) -> None:
        self.metrics.clear()


def benchmark_operation(operation_fn: Callable, *args, num_iterations: int = 100, warmup_iterations: int = 10,
                        **kwargs) -> Dict[str, float]:
    """Same arguments and result keys as python/sm120_ops.py:448-490.  Each
    iteration is timed on the device with CUDA events (the reference reads
    ``tf.timestamp`` without synchronising); times are in seconds."""
    for _ in range(warmup_iterations):
        operation_fn(*args, **kwargs)
    times: List[float] = []
    use_events = torch.cuda.is_available()
    for _ in range(num_iterations):
        if use_events:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            operation_fn(*args, **kwargs)
            e1.record()
            e1.synchronize()
            times.append(e0.elapsed_time(e1) * 1e-3)
        else:
            t0 = time.perf_counter()
            operation_fn(*args, **kwargs)
            times.append(time.perf_counter() - t0)
    arr = np.asarray(times, dtype=np.float64)
    return {
        "mean_time": float(arr.mean()),
        "std_time": float(arr.std()),
        "min_time": float(arr.min()),
        "max_time": float(arr.max()),
        "median_time": float(np.median(arr)),
    }


def _initializer(name: str, shape: Sequence[int], dtype: torch.dtype, device, generator=None) -> torch.Tensor:
    name = (name or "zeros").lower()
    if name == "zeros":
        return torch.zeros(*shape, dtype=dtype, device=device)
    if name == "ones":
        return torch.ones(*shape, dtype=dtype, device=device)
    fan_in = shape[0] if len(shape) > 1 else shape[0]
    fan_out = shape[-1]
    if name == "glorot_uniform":
        limit = (6.0 / (fan_in + fan_out)) ** 0.5
        return ((torch.rand(*shape, generator=generator, device="cpu") * 2 - 1) * limit).to(device=device, dtype=dtype)
    if name == "glorot_normal":
        std = (2.0 / (fan_in + fan_out)) ** 0.5
        return (torch.randn(*shape, generator=generator, device="cpu") * std).to(device=device, dtype=dtype)
    if name == "he_normal":
        std = (2.0 / fan_in) ** 0.5
        return (torch.randn(*shape, generator=generator, device="cpu") * std).to(device=device, dtype=dtype)
    if name == "random_normal":
        return (torch.randn(*shape, generator=generator, device="cpu") * 0.05).to(device=device, dtype=dtype)
    raise ValueError(f"unknown initializer {name!r}")


def optimized_dense(inputs, units: int, use_bias: bool = True, activation: Optional[str] = None,
                    kernel_initializer: str = "glorot_uniform", bias_initializer: str = "zeros",
                    name: Optional[str] = None):
    """Stateless dense helper with the signature of python/sm120_ops.py:494-552:
    flattens leading dimensions, draws a fresh kernel [in, units] and bias [units]
    on every call (as the reference does), and computes
    act(inputs @ kernel + bias) in one fused launch."""
    del name
    if len(inputs.shape) < 2:
        raise ValueError("Input must have at least 2 dimensions")
    in_shape = tuple(inputs.shape)
    x = inputs.reshape(-1, in_shape[-1])
    kernel = _initializer(kernel_initializer, (in_shape[-1], units), x.dtype, x.device)
    bias = _initializer(bias_initializer, (units,), x.dtype, x.device) if use_bias else None
    y = fused_matmul(x, kernel, bias=bias, activation=activation)
    return y.reshape(*in_shape[:-1], units)


__all__ = [
    "is_sm120_available",
    "get_sm120_device_info",
    "SM120Config",
    "get_config",
    "advanced_matmul",
    "sm120_matmul",
    "batched_matmul",
    "fused_matmul",
    "matmul_grad",
    "bias_grad",
    "dense_trainable",
    "fused_activation",
    "softmax",
    "scaled_dot_product_attention",
    "flash_attention",
    "quantize_fp8",
    "quantize_fp8_into",
    "SM120Profiler",
    "benchmark_operation",
    "optimized_dense",
    "activation_code",
    "InvalidArgumentError",
    "UnimplementedError",
    "InternalError",
]
