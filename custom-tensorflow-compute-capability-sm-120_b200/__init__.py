"""B200-native build of the SM120 mixed-precision matmul op.

Contents: ``csrc/`` (hand-written sm_100a kernels and the C ABI, built into
``_sm120_ops.so``), ``sm120_ops`` and ``sm120_keras_layers`` (the host-side mirror
of the reference's Python interface for this path), ``mshard`` (M-sharding of
one GEMM across the GPUs of a box) and ``tensorflow_ops/`` (the TensorFlow
OpKernel glue, compiled only where TensorFlow headers exist).

The directory name contains hyphens, so import it with
``importlib.import_module("custom-tensorflow-compute-capability-sm-120_b200")``.
"""
from . import _binding, sm120_ops, sm120_keras_layers, mshard  # noqa: F401
from .sm120_ops import advanced_matmul, fused_matmul, batched_matmul, is_sm120_available  # noqa: F401
from .sm120_keras_layers import SM120Dense, SM120Layer  # noqa: F401

__all__ = ["_binding", "sm120_ops", "sm120_keras_layers", "mshard", "advanced_matmul", "fused_matmul",
           "batched_matmul", "is_sm120_available", "SM120Dense", "SM120Layer"]
