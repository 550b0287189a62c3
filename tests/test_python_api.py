"""CPU tests of the Python surface that mirrors python/sm120_ops.py and
python/sm120_keras_layers.py: names, signatures, error behaviour, config."""
import inspect

import numpy as np
import pytest
import torch


def test_public_names(ops):
    for name in ("is_sm120_available", "get_sm120_device_info", "SM120Config", "get_config", "advanced_matmul",
                 "SM120Profiler", "benchmark_operation", "optimized_dense", "sm120_matmul"):
        assert name in ops.__all__ and hasattr(ops, name)
    sig = inspect.signature(ops.advanced_matmul)
    assert list(sig.parameters) == ["a", "b", "transpose_a", "transpose_b", "use_tensor_cores", "optimization_level", "name"]
    assert [p.default for p in list(sig.parameters.values())[2:]] == [False, False, None, None, None]
    sig = inspect.signature(ops.optimized_dense)
    assert list(sig.parameters) == ["inputs", "units", "use_bias", "activation", "kernel_initializer", "bias_initializer", "name"]
    sig = inspect.signature(ops.benchmark_operation)
    assert sig.parameters["num_iterations"].default == 100 and sig.parameters["warmup_iterations"].default == 10


def test_config_defaults_and_validation(ops):
    # tests/test_sm120_operations.py:550-572
    cfg = ops.SM120Config()
    assert (cfg.optimization_level, cfg.use_tensor_cores, cfg.enable_profiling, cfg.memory_optimization,
            cfg.fallback_to_standard) == (1, True, False, True, True)
    cfg.set_optimization_level(2)
    assert cfg.optimization_level == 2
    with pytest.raises(ValueError):
        cfg.set_optimization_level(3)
    cfg.enable_tensor_cores(False)
    assert cfg.use_tensor_cores is False
    assert ops.get_config() is ops.get_config()


def test_matmul_argument_errors(ops):
    # tests/test_sm120_operations.py:200-214: mixed dtype -> ValueError, bad inner dim -> InvalidArgument|ValueError
    a = torch.zeros(4, 8, dtype=torch.float32)
    with pytest.raises(ValueError, match="same dtype"):
        ops.advanced_matmul(a, torch.zeros(8, 4, dtype=torch.float16))
    with pytest.raises(ValueError, match="2-dimensional"):
        ops.advanced_matmul(torch.zeros(2, 4, 8), torch.zeros(8, 4))
    with pytest.raises(ops.InvalidArgumentError):
        ops.advanced_matmul(a, torch.zeros(7, 4))
    assert issubclass(ops.InvalidArgumentError, ValueError)
    with pytest.raises(ops.InvalidArgumentError):
        ops.advanced_matmul(a, torch.zeros(4, 9), transpose_b=True)
    with pytest.raises(ValueError):
        ops.fused_matmul(torch.zeros(4, 8, dtype=torch.int32), torch.zeros(8, 4, dtype=torch.int32))
    with pytest.raises(ops.InvalidArgumentError):
        ops.batched_matmul(torch.zeros(2, 4, 8), torch.zeros(3, 8, 4))
    with pytest.raises(ValueError):
        ops.activation_code("softmax")
    assert ops.activation_code("gelu") == 9 and ops.activation_code("gelu_tanh") == 4 and ops.activation_code(None) == -1


@pytest.mark.skipif(torch.cuda.is_available(), reason="checks the no-GPU behaviour")
def test_no_fallback_without_a_gpu(ops):
    assert ops.is_sm120_available() is False
    info = ops.get_sm120_device_info()
    assert info["available"] is False and info["library_loaded"] is True
    with pytest.raises(ops.UnimplementedError):
        ops.advanced_matmul(torch.zeros(4, 8), torch.zeros(8, 4))
    with pytest.raises(ops.UnimplementedError):
        ops.advanced_matmul(np.zeros((4, 8), np.float32), np.zeros((8, 4), np.float32))


def test_benchmark_operation_keys(ops):
    r = ops.benchmark_operation(lambda x: x + 1, 1, num_iterations=5, warmup_iterations=1)
    assert sorted(r) == ["max_time", "mean_time", "median_time", "min_time", "std_time"]
    assert r["min_time"] <= r["median_time"] <= r["max_time"]


def test_dense_layer_config_round_trip(pkg):
    layers = pkg.sm120_keras_layers
    sig = inspect.signature(layers.SM120Dense.__init__)
    assert list(sig.parameters)[1:13] == ["units", "activation", "use_bias", "kernel_initializer", "bias_initializer",
                                          "kernel_regularizer", "bias_regularizer", "activity_regularizer",
                                          "kernel_constraint", "bias_constraint", "use_sm120", "fallback_on_error"]
    layer = layers.SM120Dense(64, activation="gelu", name="proj", dtype="bfloat16")
    cfg = layer.get_config()
    for key in ("name", "trainable", "dtype", "units", "activation", "use_bias", "kernel_initializer", "bias_initializer",
                "kernel_regularizer", "bias_regularizer", "activity_regularizer", "kernel_constraint", "bias_constraint",
                "use_sm120", "fallback_on_error"):
        assert key in cfg
    clone = layers.SM120Dense.from_config(cfg)
    assert clone.get_config() == cfg
    assert layers.get_custom_objects()["SM120Dense"] is layers.SM120Dense
    assert layer.compute_output_shape((8, 16, 32)) == (8, 16, 64)
    with pytest.raises(ValueError):
        layers.SM120Dense(0)
    with pytest.raises(ValueError):
        layers.SM120Dense(8, activation="softmax")
    with pytest.raises(ValueError):
        layer.compute_output_shape((32,))


def test_dense_layer_weights_on_cpu(pkg):
    layers = pkg.sm120_keras_layers
    layer = layers.SM120Dense(24, use_bias=True, dtype="float32")
    layer.build((None, 5, 16), device="cpu", seed=3)
    assert tuple(layer.kernel.shape) == (16, 24) and tuple(layer.bias.shape) == (24,)
    limit = (6.0 / (16 + 24)) ** 0.5
    assert float(layer.kernel.abs().max()) <= limit and float(layer.bias.abs().max()) == 0.0
    other = layers.SM120Dense(24, dtype="float32")
    other.build((4, 16), device="cpu", seed=3)
    assert torch.equal(other.kernel, layer.kernel)            # seeded initialisation is reproducible
    w = [torch.ones(16, 24), torch.zeros(24)]
    layer.set_weights(w)
    assert torch.equal(layer.get_weights()[0], w[0])
    with pytest.raises(ValueError):
        layer.set_weights([torch.ones(3, 3), torch.zeros(24)])
    off = layers.SM120Dense(4, use_sm120=False)
    off.build((2, 8), device="cpu")
    with pytest.raises(pkg.sm120_ops.UnimplementedError):
        off.call(torch.zeros(2, 8))


def test_host_pipeline_chunk_schedule(ops):
    H = ops._HostPipeline
    for m in (512, 513, 700, 1024, 2048, 4096, 8192, 5000, 100003):
        rows = H.chunk_rows(m)
        assert sum(rows) == m and all(r > 0 for r in rows)
        assert all(r % H.MIN_ROWS == 0 for r in rows[:-1])
        assert rows[:-1] == sorted(rows[:-1], reverse=True)        # the big chunks first, a short tail
    assert H.chunk_rows(4096) == [1536, 1024, 768, 512, 256]
