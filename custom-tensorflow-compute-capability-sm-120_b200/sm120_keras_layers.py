"""``SM120Layer``, ``SM120Dense`` and ``SM120MultiHeadAttention`` for the B200 build.

Constructor arguments, weight names and shapes, ``build`` / ``call`` /
``compute_output_shape`` / ``get_config`` and the registered custom-object name
are those of the reference (python/sm120_keras_layers.py:30-56, :59-215,
:967-974).  The layer is framework-neutral here (TensorFlow/Keras is not part
of this build): weights are ``torch`` CUDA tensors and ``call`` takes and returns
``torch`` tensors.

Differences from the reference, all on purpose:

* ``call`` is ONE fused launch, act(x @ kernel + bias), instead of matmul,
  ``tf.nn.bias_add`` and the activation as three ops (:159-174);
* inputs of rank > 2 are flattened to [-1, in] and reshaped back, which is what
  the layer's ``InputSpec(min_ndim=2)`` promises but the reference's rank-2 check
  in ``advanced_matmul`` prevents (python/sm120_ops.py:183-184);
* there is no stock implementation to fall back to.  ``use_sm120`` and
  ``fallback_on_error`` are kept (and serialised) for compatibility;
  ``use_sm120=False`` raises at call time and an error in the SM120 path is
  raised to the caller instead of silently disabling the layer
  (python/sm120_keras_layers.py:46-56).
"""
from __future__ import annotations

from typing import Any, Callable, Dict, Optional, Sequence, Union

import torch

from . import sm120_ops

SM120_AVAILABLE = True

_CUSTOM_OBJECTS: Dict[str, type] = {}


def get_custom_objects() -> Dict[str, type]:
    """Registry of layer classes by serialised name
    (``tf.keras.utils.get_custom_objects()`` in the reference, :967-974)."""
    return _CUSTOM_OBJECTS


class SM120Layer:
    """Base class of SM120 layers (python/sm120_keras_layers.py:30-56)."""

    _name_counts: Dict[str, int] = {}

    def __init__(self, use_sm120: bool = True, fallback_on_error: bool = True, name: Optional[str] = None,
                 dtype: Union[str, torch.dtype, None] = None, trainable: bool = True, **kwargs):
        if kwargs:
            raise TypeError(f"unexpected keyword arguments: {sorted(kwargs)}")
        self.use_sm120 = bool(use_sm120) and SM120_AVAILABLE
        self.fallback_on_error = fallback_on_error
        self._sm120_enabled = self.use_sm120
        base = type(self).__name__.lower()
        if name is None:
            n = SM120Layer._name_counts.get(base, 0)
            SM120Layer._name_counts[base] = n + 1
            name = base if n == 0 else f"{base}_{n}"
        self.name = name
        self.trainable = trainable
        self.dtype = _parse_dtype(dtype)
        self.built = False

    def _try_sm120_operation(self, sm120_func: Callable, fallback_func: Optional[Callable], *args, **kwargs):
        """Runs the SM120 operation.  The reference switches to ``fallback_func`` on
        any exception; this build has none, so the exception propagates."""
        del fallback_func
        if not self._sm120_enabled:
            raise sm120_ops.UnimplementedError(
                f"layer {self.name!r} was created with use_sm120=False and this build has no standard implementation")
        return sm120_func(*args, **kwargs)

    def get_config(self) -> Dict[str, Any]:
        return {"name": self.name, "trainable": self.trainable, "dtype": _dtype_name(self.dtype)}

    @classmethod
    def from_config(cls, config: Dict[str, Any]):
        return cls(**config)

    def __call__(self, inputs):
        if not self.built:
            self.build(tuple(inputs.shape))
        return self.call(inputs)


_DTYPE_NAMES = {"float32": torch.float32, "float16": torch.float16, "bfloat16": torch.bfloat16}


def _parse_dtype(dtype) -> torch.dtype:
    if dtype is None:
        return torch.float32            # tf.keras.backend.floatx()
    if isinstance(dtype, torch.dtype):
        return dtype
    if str(dtype) in _DTYPE_NAMES:
        return _DTYPE_NAMES[str(dtype)]
    raise TypeError(f"A Dense layer can only be built with a floating-point dtype, got {dtype}")


def _dtype_name(dtype: torch.dtype) -> str:
    for k, v in _DTYPE_NAMES.items():
        if v == dtype:
            return k
    return str(dtype)


class SM120Dense(SM120Layer):
    """Dense layer y = activation(x @ kernel + bias) on the SM120 matmul op.

    Args (python/sm120_keras_layers.py:81-96): units, activation, use_bias,
    kernel_initializer, bias_initializer, kernel_regularizer, bias_regularizer,
    activity_regularizer, kernel_constraint, bias_constraint, use_sm120,
    fallback_on_error, plus the base-layer keywords name / dtype / trainable.

    ``activation`` may be None, a name the fused epilogue implements (linear,
    relu, gelu = erf GELU as in Keras, gelu_tanh, tanh, sigmoid, swish/silu, elu,
    selu, leaky_relu, mish) or a callable, which is applied after the fused
    matmul + bias.  Regularizers and constraints are stored and serialised; they
    act on training loops, not on the forward product."""

    def __init__(self, units: int, activation: Union[None, str, Callable] = None, use_bias: bool = True,
                 kernel_initializer: str = "glorot_uniform", bias_initializer: str = "zeros",
                 kernel_regularizer=None, bias_regularizer=None, activity_regularizer=None,
                 kernel_constraint=None, bias_constraint=None, use_sm120: bool = True,
                 fallback_on_error: bool = True, **kwargs):
        super().__init__(use_sm120=use_sm120, fallback_on_error=fallback_on_error, **kwargs)
        self.units = int(units) if not isinstance(units, int) else units
        if self.units <= 0:
            raise ValueError(f"Expected units > 0, got {units}")
        if isinstance(activation, str) or activation is None:
            sm120_ops.activation_code(activation)      # raises ValueError for unknown names
        elif not callable(activation):
            raise ValueError(f"activation must be None, a name or a callable, got {activation!r}")
        self.activation = activation
        self.use_bias = use_bias
        self.kernel_initializer = kernel_initializer
        self.bias_initializer = bias_initializer
        self.kernel_regularizer = kernel_regularizer
        self.bias_regularizer = bias_regularizer
        self.activity_regularizer = activity_regularizer
        self.kernel_constraint = kernel_constraint
        self.bias_constraint = bias_constraint
        self.supports_masking = True
        self.kernel: Optional[torch.Tensor] = None
        self.bias: Optional[torch.Tensor] = None
        self.input_spec: Optional[Dict[str, Any]] = None

    # -- weights ---------------------------------------------------------------
    def build(self, input_shape: Sequence[int], device: Union[str, torch.device, None] = None, seed: Optional[int] = None):
        if not self.dtype.is_floating_point:
            raise TypeError(f"A Dense layer can only be built with a floating-point dtype, got {self.dtype}")
        input_shape = tuple(input_shape)
        if len(input_shape) < 2:
            raise ValueError(f"Dense expects inputs of rank >= 2, got shape {input_shape}")
        last_dim = input_shape[-1]
        if last_dim is None:
            raise ValueError(f"The last dimension of the inputs to a Dense layer should be defined, got {input_shape}")
        self.input_spec = {"min_ndim": 2, "axes": {-1: int(last_dim)}}
        if device is None:
            device = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
        gen = None
        if seed is not None:
            gen = torch.Generator(device="cpu")
            gen.manual_seed(int(seed))
        self.kernel = sm120_ops._initializer(self.kernel_initializer, (int(last_dim), self.units), self.dtype, device, gen)
        self.bias = sm120_ops._initializer(self.bias_initializer, (self.units,), self.dtype, device, gen) if self.use_bias else None
        self.built = True

    @property
    def weights(self):
        return [w for w in (self.kernel, self.bias) if w is not None]

    def get_weights(self):
        return [w.detach().clone() for w in self.weights]

    def set_weights(self, weights: Sequence[torch.Tensor]):
        expected = 2 if self.use_bias else 1
        if len(weights) != expected:
            raise ValueError(f"expected {expected} weight tensors, got {len(weights)}")
        k = torch.as_tensor(weights[0])
        if self.kernel is not None and tuple(k.shape) != tuple(self.kernel.shape):
            raise ValueError(f"kernel shape {tuple(k.shape)} does not match {tuple(self.kernel.shape)}")
        device = self.kernel.device if self.kernel is not None else k.device
        self.kernel = k.to(device=device, dtype=self.dtype).contiguous()
        if self.use_bias:
            b = torch.as_tensor(weights[1])
            if tuple(b.shape) != (self.units,):
                raise ValueError(f"bias shape {tuple(b.shape)} does not match ({self.units},)")
            self.bias = b.to(device=device, dtype=self.dtype).contiguous()
        self.built = True

    # -- forward ---------------------------------------------------------------
    def call(self, inputs: torch.Tensor) -> torch.Tensor:
        if inputs.dim() < 2:
            raise ValueError(f"Dense expects inputs of rank >= 2, got shape {tuple(inputs.shape)}")
        if inputs.shape[-1] != self.kernel.shape[0]:
            raise sm120_ops.InvalidArgumentError(
                f"last dimension of the inputs ({inputs.shape[-1]}) does not match the kernel ({self.kernel.shape[0]})")
        fused_act = self.activation if (self.activation is None or isinstance(self.activation, str)) else None

        def sm120_dense():
            x = inputs.reshape(-1, inputs.shape[-1])
            y = sm120_ops.fused_matmul(x, self.kernel, bias=self.bias if self.use_bias else None, activation=fused_act)
            return y.reshape(*inputs.shape[:-1], self.units)

        outputs = self._try_sm120_operation(sm120_dense, None)
        if callable(self.activation):
            outputs = self.activation(outputs)
        return outputs

    def compute_output_shape(self, input_shape: Sequence[int]):
        input_shape = tuple(input_shape)
        if len(input_shape) < 2:
            raise ValueError(f"input shape must have rank >= 2, got {input_shape}")
        if input_shape[-1] is None:
            raise ValueError(f"The last dimension of the input shape must be defined, got {input_shape}")
        return input_shape[:-1] + (self.units,)

    def get_config(self) -> Dict[str, Any]:
        config = super().get_config()
        act = self.activation
        config.update({
            "units": self.units,
            "activation": ("linear" if act is None else act) if not callable(act) else getattr(act, "__name__", repr(act)),
            "use_bias": self.use_bias,
            "kernel_initializer": self.kernel_initializer,
            "bias_initializer": self.bias_initializer,
            "kernel_regularizer": self.kernel_regularizer,
            "bias_regularizer": self.bias_regularizer,
            "activity_regularizer": self.activity_regularizer,
            "kernel_constraint": self.kernel_constraint,
            "bias_constraint": self.bias_constraint,
            "use_sm120": self.use_sm120,
            "fallback_on_error": self.fallback_on_error,
        })
        return config


class SM120MultiHeadAttention(SM120Layer):
    """Multi-head attention on the SM120 ops (python/sm120_keras_layers.py:636-886):
    four ``SM120Dense`` projections (query, key, value: num_heads * key_dim / value_dim
    units; output: ``output_shape`` or the query's last dimension) around
    ``sm120_ops.scaled_dot_product_attention``, which for float16 / bfloat16 heads of 64 or
    128 is one fused tcgen05 kernel.  Constructor arguments and ``get_config`` keys are the
    reference's (:643-684, :858-886).  ``call(inputs, attention_mask=None,
    return_attention_scores=False, training=None)`` takes one tensor [batch, seq, dim]
    (self-attention) or a list [query, key, value]; the mask marks EXCLUDED positions with
    non-zero entries, as in the reference (:815-816).  Dropout is not implemented: a
    non-zero rate raises when ``training`` is true."""

    def __init__(self, num_heads: int, key_dim: int, value_dim: Optional[int] = None, dropout: float = 0.0, use_bias: bool = True,
                 output_shape=None, attention_axes=None, kernel_initializer: str = "glorot_uniform",
                 bias_initializer: str = "zeros", kernel_regularizer=None, bias_regularizer=None, activity_regularizer=None,
                 kernel_constraint=None, bias_constraint=None, use_sm120: bool = True, fallback_on_error: bool = True,
                 use_flash_attention: bool = True, **kwargs):
        super().__init__(use_sm120=use_sm120, fallback_on_error=fallback_on_error, **kwargs)
        if num_heads < 1 or key_dim < 1:
            raise ValueError("num_heads and key_dim must be positive")
        self.num_heads = int(num_heads)
        self.key_dim = int(key_dim)
        self.value_dim = int(value_dim) if value_dim is not None else int(key_dim)
        self.dropout = float(dropout)
        self.use_bias = use_bias
        self.output_shape = output_shape
        self.attention_axes = attention_axes
        self.kernel_initializer = kernel_initializer
        self.bias_initializer = bias_initializer
        self.kernel_regularizer = kernel_regularizer
        self.bias_regularizer = bias_regularizer
        self.activity_regularizer = activity_regularizer
        self.kernel_constraint = kernel_constraint
        self.bias_constraint = bias_constraint
        self.use_flash_attention = use_flash_attention
        self.supports_masking = True
        self.query_dense = self.key_dense = self.value_dense = self.output_dense = None

    def _dense(self, units: int, name: str) -> SM120Dense:
        return SM120Dense(units, use_bias=self.use_bias, kernel_initializer=self.kernel_initializer,
                          bias_initializer=self.bias_initializer, kernel_regularizer=self.kernel_regularizer,
                          bias_regularizer=self.bias_regularizer, kernel_constraint=self.kernel_constraint,
                          bias_constraint=self.bias_constraint, use_sm120=self.use_sm120,
                          fallback_on_error=self.fallback_on_error, name=f"{self.name}/{name}", dtype=self.dtype)

    def build(self, input_shape, device=None, seed: Optional[int] = None):
        if isinstance(input_shape, list):
            if len(input_shape) != 3:
                raise ValueError("MultiHeadAttention expects exactly 3 inputs: [query, key, value]")
            query_shape, key_shape, value_shape = (tuple(s) for s in input_shape)
        else:
            query_shape = key_shape = value_shape = tuple(input_shape)
        self.query_dense = self._dense(self.num_heads * self.key_dim, "query")
        self.key_dense = self._dense(self.num_heads * self.key_dim, "key")
        self.value_dense = self._dense(self.num_heads * self.value_dim, "value")
        output_dim = self.output_shape if self.output_shape is not None else query_shape[-1]
        self.output_dense = self._dense(int(output_dim), "output")
        seeds = [None] * 4 if seed is None else [seed, seed + 1, seed + 2, seed + 3]
        self.query_dense.build(query_shape, device=device, seed=seeds[0])
        self.key_dense.build(key_shape, device=device, seed=seeds[1])
        self.value_dense.build(value_shape, device=device, seed=seeds[2])
        self.output_dense.build(tuple(query_shape[:-1]) + (self.num_heads * self.value_dim,), device=device, seed=seeds[3])
        self.built = True

    @property
    def weights(self):
        return [w for layer in (self.query_dense, self.key_dense, self.value_dense, self.output_dense) for w in layer.weights]

    def __call__(self, inputs, attention_mask=None, return_attention_scores=False, training=None):
        if not self.built:
            self.build([tuple(t.shape) for t in inputs] if isinstance(inputs, list) else tuple(inputs.shape))
        return self.call(inputs, attention_mask=attention_mask, return_attention_scores=return_attention_scores, training=training)

    def call(self, inputs, attention_mask=None, return_attention_scores=False, training=None):
        if isinstance(inputs, list):
            if len(inputs) != 3:
                raise ValueError("MultiHeadAttention expects exactly 3 inputs: [query, key, value]")
            query, key, value = inputs
        else:
            query = key = value = inputs
        if query.dim() != 3 or key.dim() != 3 or value.dim() != 3:
            raise ValueError("MultiHeadAttention expects [batch, seq, dim] tensors")
        if value.shape[-1] != self.num_heads * self.value_dim and self.value_dense is None:
            raise ValueError("layer is not built")
        batch, seq_q, seq_k = query.shape[0], query.shape[1], key.shape[1]
        # projections, then [batch, seq, heads, dim] -> [batch, heads, seq, dim] (:780-794)
        q = self.query_dense(query).reshape(batch, seq_q, self.num_heads, self.key_dim).permute(0, 2, 1, 3)
        k = self.key_dense(key).reshape(batch, seq_k, self.num_heads, self.key_dim).permute(0, 2, 1, 3)
        v = self.value_dense(value).reshape(batch, seq_k, self.num_heads, self.value_dim).permute(0, 2, 1, 3)
        if self.value_dim != self.key_dim:
            raise NotImplementedError("value_dim != key_dim is not implemented by the attention kernels")

        def sm120_attention():
            return sm120_ops.scaled_dot_product_attention(
                q, k, v, scale=1.0 / float(self.key_dim) ** 0.5, dropout_rate=self.dropout if training else 0.0,
                attention_mask=attention_mask, return_attention_scores=return_attention_scores)

        result = self._try_sm120_operation(sm120_attention, None)
        attention_output, attention_weights = result if return_attention_scores else (result, None)
        attention_output = attention_output.permute(0, 2, 1, 3).reshape(batch, seq_q, self.num_heads * self.value_dim)
        output = self.output_dense(attention_output)
        return (output, attention_weights) if return_attention_scores else output

    def get_config(self) -> Dict[str, Any]:
        config = super().get_config()
        config.update({
            "num_heads": self.num_heads, "key_dim": self.key_dim, "value_dim": self.value_dim, "dropout": self.dropout,
            "use_bias": self.use_bias, "output_shape": self.output_shape, "attention_axes": self.attention_axes,
            "kernel_initializer": self.kernel_initializer, "bias_initializer": self.bias_initializer,
            "kernel_regularizer": self.kernel_regularizer, "bias_regularizer": self.bias_regularizer,
            "activity_regularizer": self.activity_regularizer, "kernel_constraint": self.kernel_constraint,
            "bias_constraint": self.bias_constraint, "use_sm120": self.use_sm120, "fallback_on_error": self.fallback_on_error,
            "use_flash_attention": self.use_flash_attention,
        })
        return config


_CUSTOM_OBJECTS.update({"SM120Dense": SM120Dense, "SM120MultiHeadAttention": SM120MultiHeadAttention})

__all__ = ["SM120Layer", "SM120Dense", "SM120MultiHeadAttention", "get_custom_objects", "SM120_AVAILABLE"]
