#!/usr/bin/env python
"""Benchmark of the SM120 matmul op on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

One "step" is one GEMM of the workload through the C ABI.  The default workload
is the fp16 product M = N = K = 4096 with A row-major and B stored [N, K] (fp32
accumulate, fp16 out).  With N > 1 (one process per GPU, launched by torchrun)
every rank multiplies its own 4096-row slab of A by the replicated B: the
M-sharded product with M = 4096 * N, no data-path collective, weak scaling.

Rank 0 prints ONE JSON line.  `value` is whole-job TFLOP/s with the operands
resident in HBM; `e2e` is the same product through the public Python API from
pinned host buffers (host->device and device->host copies inside the timed
region); `roofline` compares the kernel with the measured cuBLAS bf16 peak of
this pool; `cublas_same_process` is torch.matmul on the same buffers, timed the
same way right after (a yardstick only); `cpu_baseline` is the oracle's fp32
host-BLAS product of the whole workload timed on this box's cores;
`fp8_m_sharded` is the FP8 product M = 65536, N = K = 8192 split by rows over
the N ranks (strong scaling: the whole M on one GPU at N = 1), with the fused
and the NCCL gather of C beside it at N > 1; `all_configs` (N = 1) lists every
benchmark workload and `small_shapes` four products with few output tiles (GPU time
from CUDA-graph replays, the K parts chosen, cuBLAS beside them).  `--impl reference`
times only the CPU product.

Other workloads (`--workload`): f32_1024, f16_4096_tn, bf16_4096_tn,
bf16_dense_gelu, bf16_batched_qk, fp8_65536 (M split over the ranks), fp8_8192,
f32_1024_ffma, f32_4096, f32_4096_ffma, bf16_8192_tn, bf16_1024x1024x8192 (split along K), and the HBM-bound kernels quant_fp8_64m,
activation_gelu_64m, bias_grad_8192x11008, softmax_131072x2048 and the fused attention
attention_<batch x heads>x<sequence>x<head size>[_causal] (bf16; the listed shapes, default 64x2048x128).  `--trace FILE` also writes the
launch timeline (SM120_TUNE_TRACE) of one launch of the workload to FILE.
"""
import argparse
import importlib
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
PACKAGE_NAME = "custom-tensorflow-compute-capability-sm-120_b200"

METRIC = "gemm_tflops"          # GEMM TFLOP/s, whole job; % of the dense tensor peak is reported beside it
UNIT = "TFLOP/s"
NOMINAL_PEAK = {"f16": 2250.0, "bf16": 2250.0, "f8e4m3": 4500.0, "f32": 80.0}   # dense, per GPU, datasheet
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}

# name -> shape, types, operand layout ("tn": B stored [N, K]; "nn": B stored [K, N]) and epilogue.
# `oracle_idx` is the index of the same workload in oracle/reference.py's seeded generators.
WORKLOADS = {
    "f32_1024":        dict(M=1024, N=1024, K=1024, batch=1, dtype="f32", layout="nn", oracle_idx=1),
    "f16_4096_tn":     dict(M=4096, N=4096, K=4096, batch=1, dtype="f16", layout="tn", oracle_idx=2),
    "bf16_4096_tn":    dict(M=4096, N=4096, K=4096, batch=1, dtype="bf16", layout="tn", oracle_idx=2),
    "bf16_dense_gelu": dict(M=8192, N=11008, K=4096, batch=1, dtype="bf16", layout="nn", epilogue="bias+gelu", oracle_idx=3),
    "bf16_batched_qk": dict(M=2048, N=2048, K=128, batch=64, dtype="bf16", layout="nn", oracle_idx=4),
    "fp8_65536":       dict(M=65536, N=8192, K=8192, batch=1, dtype="f8e4m3", layout="tn", sharded=True, oracle_idx=5),
    "fp8_8192":        dict(M=8192, N=8192, K=8192, batch=1, dtype="f8e4m3", layout="tn", oracle_idx=5),
    "f32_1024_ffma":   dict(M=1024, N=1024, K=1024, batch=1, dtype="f32", layout="nn", ffma=True, oracle_idx=1),
    "f32_4096":        dict(M=4096, N=4096, K=4096, batch=1, dtype="f32", layout="nn", oracle_idx=1),
    "f32_4096_ffma":   dict(M=4096, N=4096, K=4096, batch=1, dtype="f32", layout="nn", ffma=True, oracle_idx=1),
    "bf16_8192_tn":    dict(M=8192, N=8192, K=8192, batch=1, dtype="bf16", layout="tn", oracle_idx=2),   # the shape the measured peak is taken on
    "bf16_1024x1024x8192": dict(M=1024, N=1024, K=8192, batch=1, dtype="bf16", layout="tn", oracle_idx=2),   # few tiles, long K: split-K
}
# attention_<batch x heads>x<sequence>x<head size>[_causal], bf16
ATTENTION_WORKLOADS = ("attention_64x2048x128", "attention_64x2048x128_causal", "attention_16x8192x128", "attention_16x8192x128_causal",
                       "attention_8x16384x128_causal", "attention_256x512x128", "attention_128x2048x64", "attention_16x16384x64")
AUX_WORKLOADS = ("quant_fp8_64m", "activation_gelu_64m", "bias_grad_8192x11008", "softmax_131072x2048") + ATTENTION_WORKLOADS
ALIASES = {"cfg1": "f32_1024", "cfg2": "f16_4096_tn", "cfg2bf16": "bf16_4096_tn", "cfg3": "bf16_dense_gelu",
           "cfg4": "bf16_batched_qk", "cfg5": "fp8_65536"}
IN_BYTES = {"f32": 4, "f16": 2, "bf16": 2, "f8e4m3": 1}
OUT_BYTES = {"f32": 4, "f16": 2, "bf16": 2, "f8e4m3": 2}

# dram__bytes_read.sum + dram__bytes_write.sum per launch of the workload's kernel, from the ncu
# captures summarised under profiles/ (the file named beside each figure); None = not captured.
NCU_TRAFFIC_BYTES = {
    "f16_4096_tn": 91455744,        # profiles/gemm_tcgen05_f16_4096x4096x4096.txt: 74.30 MB read + 17.16 MB written
    "bf16_4096_tn": 91455744,       # same kernel, shape and byte counts
    "bf16_dense_gelu": 517800000,   # profiles/gemm_tcgen05_bf16_dense_gelu_8192x11008x4096.txt: 351.7 MB read + 166.1 MB written
    "bf16_batched_qk": 547412224,   # profiles/gemm_tcgen05_bf16_batched_qk_96x1024x1024x128.txt: 67.2 MB read + 480.2 MB written
    "fp8_8192": 402100000,          # profiles/gemm_tcgen05_fp8_8192x8192x8192.txt: 284.4 MB read + 117.7 MB written
    "attention_64x2048x128": 115489280,   # profiles/attention_tcgen05_64x2048x128_bf16.txt: 100.7 MB read + 14.7 MB written
}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            d = json.load(f)
        return d, "measured"
    except Exception:
        return dict(FALLBACK_PEAKS), "fallback"


# ---------------------------------------------------------------------------
# workloads
# ---------------------------------------------------------------------------
def workload_spec(name: str, world: int):
    """Shapes of one rank's share, FLOPs and algorithmic bytes per step (per rank)."""
    name = ALIASES.get(name, name)
    if name not in WORKLOADS:
        raise SystemExit(f"unknown workload {name}")
    s = dict(WORKLOADS[name])
    s["name"] = name
    s["scaling"] = "weak"
    s["M_total"] = s["M"] * world
    if s.get("sharded"):
        if s["M"] % world != 0:
            raise SystemExit(f"{name} needs a world size that divides {s['M']}")
        s["M_total"] = s["M"]
        s["M"] //= world
        s["scaling"] = "strong"
    s["in_bytes"], s["out_bytes"] = IN_BYTES[s["dtype"]], OUT_BYTES[s["dtype"]]
    s["flops"] = 2.0 * s["M"] * s["N"] * s["K"] * s["batch"]
    s["bytes"] = s["batch"] * ((s["M"] * s["K"] + s["K"] * s["N"]) * s["in_bytes"] + s["M"] * s["N"] * s["out_bytes"])
    return s


def make_device_operands(spec, seed, device, ops, reduce_max=None):
    """Synthetic operands with the workload's shapes and value distributions, drawn on
    the device from a seeded generator.  FP8 operands come from the library's own
    quantiser (scale = 448 / amax)."""
    import torch
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    M, N, K, B = spec["M"], spec["N"], spec["K"], spec["batch"]
    dt = spec["dtype"]
    kw = {}
    if dt == "f32":
        a = torch.rand(M, K, generator=g, device=device) * 2 - 1
        b = torch.rand(K, N, generator=g, device=device) * 2 - 1
        if spec.get("ffma"):
            kw["use_tensor_cores"] = False          # the exact FFMA kernel instead of 3xTF32 on the tensor cores
    elif dt in ("f16", "bf16") and spec["layout"] == "tn":
        tdt = torch.float16 if dt == "f16" else torch.bfloat16
        a = (torch.randn(M, K, generator=g, device=device) / K ** 0.5).to(tdt)
        b = (torch.randn(N, K, generator=g, device=device) / K ** 0.5).to(tdt)      # stored [N, K]
        kw["transpose_b"] = True
    elif spec["name"] == "bf16_dense_gelu":
        a = torch.randn(M, K, generator=g, device=device).bfloat16()
        b = (0.02 * torch.randn(K, N, generator=g, device=device)).bfloat16()
        kw["bias"] = (0.02 * torch.randn(N, generator=g, device=device)).bfloat16()
        kw["activation"] = "gelu"
    elif spec["name"] == "bf16_batched_qk":
        a = torch.randn(B, M, K, generator=g, device=device).bfloat16()
        b = torch.randn(B, K, N, generator=g, device=device).bfloat16()
    elif dt != "f8e4m3":
        raise SystemExit(f"no operand recipe for workload {spec['name']}")
    else:   # FP8: N(0,1) before quantisation, per-tensor scales that map amax to 448
        b32 = torch.randn(N, K, generator=g, device=device)
        b, sb = ops.quantize_fp8(b32)
        del b32
        a32 = torch.randn(M, K, generator=g, device=device)
        if reduce_max is not None:      # A is one tensor split over the ranks: one scale, from the maximum over all slabs
            a, sa = ops.quantize_fp8(a32, scale=(448.0 / reduce_max(a32.abs().max().reshape(1))).float())
        else:
            a, sa = ops.quantize_fp8(a32)
        del a32
        kw.update(transpose_b=True, scale_a=sa, scale_b=sb)
    return a, b, kw


# ---------------------------------------------------------------------------
# clocks during the timed region (NVML: the source nvidia-smi reads)
# ---------------------------------------------------------------------------
class ClockSampler:
    REASONS = {
        0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap",
        0x80: "hw_power_brake_slowdown",
    }

    def __init__(self, index: int, period_s: float = 0.002):
        self.index, self.period = index, period_s
        self.samples, self.reasons = [], set()
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nvml = pynvml
            self.handle = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nvml = None

    def _loop(self):
        n = self.nvml
        while not self._stop.is_set():
            try:
                self.samples.append(n.nvmlDeviceGetClockInfo(self.handle, n.NVML_CLOCK_SM))
                mask = n.nvmlDeviceGetCurrentClocksThrottleReasons(self.handle)
                for bit, name in self.REASONS.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop.wait(self.period)

    def start(self):
        if self.nvml is not None:
            self._stop.clear()
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()

    def stop(self):
        if self._thread is not None:
            self._stop.set()
            self._thread.join()
            self._thread = None

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": 0}
        return {"sm_mhz": statistics.median(self.samples), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


def config_dict(args, spec, world, l2_note):
    """The `config` object, identical for both arms."""
    layout = "A row-major [M,K], B stored [N,K]" if spec["layout"] == "tn" else "A row-major [M,K], B row-major [K,N]"
    return {"workload": spec["name"], "layout": layout, "epilogue": spec.get("epilogue", "none"),
            "gather": getattr(args, "gather", "none"), "M_per_gpu": spec["M"], "M_total": spec["M_total"],
            "N": spec["N"], "K": spec["K"], "batch": spec["batch"],
            "sharding": "M-slabs, B replicated; collective only with --gather", "l2": l2_note}


# ---------------------------------------------------------------------------
# reference arm / CPU baseline: the oracle's fp32 host-BLAS product
# ---------------------------------------------------------------------------
def cpu_operands(spec):
    """The workload's own seeded inputs (oracle/reference.py's generators: same shapes and value
    distributions as the GPU arm), as the arrays the CPU product consumes, and a description."""
    import numpy as np
    from oracle import reference as ref

    idx = spec["oracle_idx"]
    full = ref.config_shapes(idx)
    same = (spec["M"], spec["N"], spec["K"], spec["batch"]) == (full["M"], full["N"], full["K"], full["batch"])
    if same and idx != 5:
        cfg = ref.make_config(idx)
        if spec["dtype"] == "bf16" and idx == 2:       # the fp16 workload's values, stored as bf16
            cfg["a"] = ref.quantize(cfg["a"].astype(np.float32), "bfloat16")
            cfg["b"] = ref.quantize(cfg["b"].astype(np.float32), "bfloat16")
        text = "the whole workload per step: fp32 torch.matmul (host BLAS) + the epilogue on the workload's own seeded inputs"
        return cfg["a"], cfg["b"], cfg["bias"], cfg["act"], cfg["transpose_b"], spec["M"], text
    # sizes the generators do not hold, and the FP8 workload (8.8 TFLOP per step): drawn here with the
    # same distributions; the FP8 workload is timed on the first 8192 rows of A
    rng = np.random.default_rng(idx - 1)
    N, K, B = spec["N"], spec["K"], spec["batch"]
    tb = spec["layout"] == "tn"
    rows = min(spec["M"], 8192) if spec["dtype"] == "f8e4m3" else spec["M"]
    lead = (B,) if B > 1 else ()
    if spec["dtype"] == "f32":
        a = rng.uniform(-1, 1, lead + (rows, K)).astype(np.float32)
        b = rng.uniform(-1, 1, lead + ((N, K) if tb else (K, N))).astype(np.float32)
    else:
        a = rng.standard_normal(lead + (rows, K), dtype=np.float32)
        b = rng.standard_normal(lead + ((N, K) if tb else (K, N)), dtype=np.float32)
    if rows == spec["M"]:
        text = "the whole workload per step: fp32 torch.matmul (host BLAS) on inputs of the workload's distribution"
    else:
        text = (f"first {rows} of {spec['M']} rows of A per step (all of B), fp32 torch.matmul (host BLAS) on the unquantised "
                "N(0,1) inputs; the rate is what a whole step would run at (extrapolated)")
    return a, b, None, -1, tb, rows, text


def cpu_product(spec, steps, warmup):
    """Times `steps` CPU products; returns (TFLOP/s, ms/step, cores, sample text)."""
    from oracle import reference as ref

    a, b, bias, act, tb, rows, text = cpu_operands(spec)
    cores = os.cpu_count() or 1
    times = []
    for i in range(warmup + steps):
        _, secs, cores = ref.cpu_baseline_fp32(a, b, transpose_b=tb, bias=bias, act=act, threads=cores, repeats=1)
        if i >= warmup:
            times.append(secs)
    total = sum(times)
    flops = 2.0 * rows * spec["N"] * spec["K"] * spec["batch"]
    return flops * len(times) / total / 1e12, 1e3 * total / len(times) * (spec["M"] / rows), cores, text


def run_reference(args, rank, world):
    spec = workload_spec(args.workload, world)
    if rank != 0:
        return
    tflops, ms, cores, text = cpu_product(spec, args.steps, args.warmup)
    line = {
        "impl": "reference", "metric": METRIC, "value": tflops, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": spec["scaling"],
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": config_dict(args, spec, world, "host memory"),
        "note": "CPU restatement (oracle port) of the reference's fallback path tf.linalg.matmul + bias_add + activation, "
                "fp32 host BLAS on all cores; TensorFlow itself cannot be installed here",
        "cpu_baseline": {"value": tflops, "unit": UNIT, "cores": cores, "kind": "port", "sample": text},
        "e2e": {"value": tflops, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------
def nvml_index(torch, dev_index):
    """NVML index of torch device `dev_index` (they differ under CUDA_VISIBLE_DEVICES)."""
    try:
        import pynvml
        pynvml.nvmlInit()
        uuid = "GPU-" + str(torch.cuda.get_device_properties(dev_index).uuid)
        return pynvml.nvmlDeviceGetIndex(pynvml.nvmlDeviceGetHandleByUUID(uuid.encode()))
    except Exception:
        return dev_index


def time_device_steps(torch, step_fn, sets, steps, warmup, barrier):
    """W warm-up steps, then K steps rotating over the buffer sets, timed with CUDA
    events on the launch stream.  Returns seconds for the K steps."""
    for i in range(warmup):
        step_fn(*sets[i % len(sets)])
    torch.cuda.synchronize()
    barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(steps):
        step_fn(*sets[i % len(sets)])
    e1.record()
    torch.cuda.synchronize()
    barrier()
    return e0.elapsed_time(e1) * 1e-3


def build_sets(torch, ops, spec, device, min_total_bytes=3 * 126e6, max_sets=4, reduce_max=None):
    """Buffer sets (A, B, C) so that consecutive steps never find their operands in
    the 126 MB L2: at least 2 sets and at least ~380 MB in total, unless one set
    alone is larger than that."""
    out_dt = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16, "f8e4m3": torch.bfloat16}[spec["dtype"]]
    n_sets = int(min(max_sets, max(2, -(-min_total_bytes // spec["bytes"])))) if spec["bytes"] < min_total_bytes else 1
    sets, kw = [], {}
    for s in range(n_sets):
        a, b, kw = make_device_operands(spec, 1234 + s, device, ops, reduce_max=reduce_max)
        shape = ((spec["batch"],) if spec["batch"] > 1 else ()) + (spec["M"], spec["N"])
        sets.append((a, b, torch.empty(shape, dtype=out_dt, device=device)))
    return sets, kw


def rank_stats(torch, dist, world, device, secs, steps):
    """(max over ranks in seconds, {min, median, max} of ms per step over the ranks)."""
    per = [secs]
    if world > 1:
        t = torch.tensor([secs], device=device, dtype=torch.float64)
        allr = [torch.zeros_like(t) for _ in range(world)]
        dist.all_gather(allr, t)
        per = [float(x.item()) for x in allr]
    ms = sorted(1e3 * s / steps for s in per)
    return max(per), {"min": ms[0], "median": statistics.median(ms), "max": ms[-1]}


def measure_e2e(torch, ops, spec, sets, kw, steps, warmup):
    """The same product through the public API with HOST operands: every step copies
    A and B from pinned host memory to the device, multiplies, and copies C back into
    a pinned host buffer (the API pipelines the three over row chunks).  Wall-clock
    around `steps` calls, device synchronised on both sides.  Returns (seconds, h2d
    bytes per step, d2h bytes per step)."""
    a_d, b_d, c_d = sets[0]
    a_h = torch.empty(a_d.shape, dtype=a_d.dtype, pin_memory=True).copy_(a_d)
    b_h = torch.empty(b_d.shape, dtype=b_d.dtype, pin_memory=True).copy_(b_d)
    c_h = torch.empty(c_d.shape, dtype=c_d.dtype, pin_memory=True)
    kw_h = dict(kw)
    for name in ("scale_a", "scale_b"):                 # host operands take host scales
        if isinstance(kw_h.get(name), torch.Tensor):
            kw_h[name] = float(kw_h[name].item())
    if kw_h.get("bias") is not None:
        kw_h["bias"] = torch.empty(kw["bias"].shape, dtype=kw["bias"].dtype, pin_memory=True).copy_(kw["bias"])
    h2d = a_h.numel() * a_h.element_size() + b_h.numel() * b_h.element_size()
    if kw_h.get("bias") is not None:
        h2d += kw_h["bias"].numel() * kw_h["bias"].element_size()
    d2h = c_h.numel() * c_h.element_size()
    for _ in range(warmup):
        ops.fused_matmul(a_h, b_h, out=c_h, **kw_h)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(steps):
        ops.fused_matmul(a_h, b_h, out=c_h, **kw_h)
    torch.cuda.synchronize()
    return time.perf_counter() - t0, h2d, d2h


def pcie_probe(torch, device, nbytes=64 << 20):
    """Raw copy rates of this GPU's PCIe link with pinned memory (GB/s): host->device alone, device->host
    alone, and both at once on two streams (each direction's own rate while the other runs)."""
    h_in = torch.empty(nbytes, dtype=torch.uint8, pin_memory=True)
    h_out = torch.empty(nbytes, dtype=torch.uint8, pin_memory=True)
    d_in = torch.empty(nbytes, dtype=torch.uint8, device=device)
    d_out = torch.zeros(nbytes, dtype=torch.uint8, device=device)
    s1, s2 = torch.cuda.Stream(device=device), torch.cuda.Stream(device=device)

    def run(up, down, reps=4):
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(reps):
            if up:
                with torch.cuda.stream(s1):
                    d_in.copy_(h_in, non_blocking=True)
            if down:
                with torch.cuda.stream(s2):
                    h_out.copy_(d_out, non_blocking=True)
        torch.cuda.synchronize()
        return reps * nbytes / (time.perf_counter() - t0) / 1e9

    run(True, True, 1)
    return {"h2d_gbs": run(True, False), "d2h_gbs": run(False, True), "each_direction_when_both_gbs": run(True, True),
            "bytes_per_copy": nbytes}


def host_overhead(torch, ops, binding, device):
    """Host time of one launch (microseconds) on a product so small that the GPU is never the bottleneck:
    through the Python API, and through the C ABI alone (ctypes call with a prepared descriptor)."""
    import ctypes
    a = torch.randn(256, 64, device=device).bfloat16()
    b = torch.randn(64, 256, device=device).bfloat16()
    out = torch.empty(256, 256, dtype=torch.bfloat16, device=device)
    n = 2000
    for _ in range(50):
        ops.fused_matmul(a, b, out=out)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(n):
        ops.fused_matmul(a, b, out=out)
    t_api = time.perf_counter() - t0
    torch.cuda.synchronize()
    d = binding.new_desc()
    d.in_dtype = d.out_dtype = binding.DTYPE_BFLOAT16
    d.A, d.B, d.C = a.data_ptr(), b.data_ptr(), out.data_ptr()
    d.M, d.N, d.K = 256, 256, 64
    d.stream = torch.cuda.current_stream(device).cuda_stream
    fn, ref_d = binding.load_library().sm120_launch_matmul_ex, ctypes.byref(d)
    t0 = time.perf_counter()
    for _ in range(n):
        fn(ref_d)
    t_abi = time.perf_counter() - t0
    torch.cuda.synchronize()
    return {"python_api_us": 1e6 * t_api / n, "c_abi_us": 1e6 * t_abi / n,
            "what": "bf16 256x256x64, 2000 back-to-back launches, host wall-clock of the enqueue loop"}


def cublas_yardstick(torch, spec, sets, kw, steps, warmup):
    """torch.matmul (cuBLAS) on the same buffers, same rotation, same events: TFLOP/s, or None where
    torch has no plain matmul for the type.  A yardstick for the bench only; the package never calls it."""
    tb = bool(kw.get("transpose_b"))
    if spec["dtype"] == "f8e4m3":
        # FP8: torch._scaled_mm (cuBLASLt) wants A [M, K] row-major and B column-major, i.e. B stored [N, K]
        if not tb or not hasattr(torch, "_scaled_mm"):
            return None
        one = torch.ones((), device=sets[0][0].device)

        def step8(a, b, out):
            torch._scaled_mm(a, b.t(), scale_a=one, scale_b=one, out_dtype=out.dtype)

        try:
            secs = time_device_steps(torch, step8, sets, steps, warmup, lambda: None)
        except Exception as e:
            return {"error": str(e)[:160]}
        return {"tflops": spec["flops"] / (secs / steps) / 1e12, "ms_per_step": 1e3 * secs / steps,
                "what": "torch._scaled_mm (cuBLASLt FP8) on the same buffer sets, unit scales, product only"}

    def step(a, b, out):
        torch.matmul(a, b.transpose(-1, -2) if tb else b, out=out)

    try:
        prev = torch.backends.cuda.matmul.allow_tf32
        torch.backends.cuda.matmul.allow_tf32 = False
        secs = time_device_steps(torch, step, sets, steps, warmup, lambda: None)
        torch.backends.cuda.matmul.allow_tf32 = prev
    except Exception as e:
        return {"error": str(e)[:160]}
    return {"tflops": spec["flops"] / (secs / steps) / 1e12, "ms_per_step": 1e3 * secs / steps,
            "what": "torch.matmul on the same buffer sets, product only (no bias / activation)"}


def side_table(torch, ops, binding, device):
    """Single-GPU TFLOP/s of every benchmark workload (after 3 warm-ups, CUDA events),
    reported beside the headline."""
    table = {}
    for name in ("f32_1024", "f16_4096_tn", "bf16_4096_tn", "bf16_dense_gelu", "bf16_batched_qk", "fp8_8192", "f32_1024_ffma"):
        spec = workload_spec(name, 1)
        try:
            sets, kw = build_sets(torch, ops, spec, device)
            steps = 20

            def step(a, b, out):
                ops.fused_matmul(a, b, out=out, **kw)
            secs = time_device_steps(torch, step, sets, steps, 3, lambda: None)
            tf = spec["flops"] / (secs / steps) / 1e12
            row = {"ms": round(1e3 * secs / steps, 4), "tflops": round(tf, 1),
                   "gbs": round(spec["bytes"] / (secs / steps) / 1e9, 1),
                   "pct_nominal_peak": round(100 * tf / NOMINAL_PEAK[spec["dtype"]], 1),
                   "kernel": binding.last_kernel_name(),
                   "shape": [spec["batch"], spec["M"], spec["N"], spec["K"]]}
            yard = cublas_yardstick(torch, spec, sets, kw, steps, 3)
            if yard and "tflops" in yard:
                row["cublas_tflops"] = round(yard["tflops"], 1)
            table[name] = row
            del sets
            torch.cuda.empty_cache()
        except Exception as e:  # keep the headline even if a side measurement fails
            table[name] = {"error": str(e)[:200]}
    return table


def small_shapes(torch, ops, binding, device):
    """Products with few output tiles (projection, decode-time and weight-gradient shapes, bf16, B stored [N, K]):
    GPU time per call with the host taken out (24 calls captured into a CUDA graph, the graph replayed), the K
    parts the launcher chose, and cuBLAS through torch.matmul timed the same way."""
    def graph_time(fn, calls=24):
        for _ in range(6):
            fn()
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        side = torch.cuda.Stream(device=device)
        side.wait_stream(torch.cuda.current_stream(device))
        with torch.cuda.stream(side):
            with torch.cuda.graph(g, stream=side):
                for _ in range(calls):
                    fn()
        torch.cuda.synchronize()
        g.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(3):
            g.replay()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / (3 * calls) * 1e-3

    table = {}
    for (M, N, K) in ((1024, 1024, 8192), (128, 4096, 4096), (64, 8192, 8192), (256, 8192, 8192)):
        key = f"bf16_{M}x{N}x{K}"
        try:
            nsets = min(6, max(2, int(400e6 // ((M * K + N * K + M * N) * 2)) + 1))
            sets = [(torch.randn(M, K, device=device, dtype=torch.bfloat16), torch.randn(N, K, device=device, dtype=torch.bfloat16),
                     torch.empty(M, N, device=device, dtype=torch.bfloat16)) for _ in range(nsets)]
            turn = [0]

            def ours():
                a, b, c = sets[turn[0] % nsets]
                turn[0] += 1
                ops.fused_matmul(a, b, out=c, transpose_b=True)

            def cublas():
                a, b, c = sets[turn[0] % nsets]
                turn[0] += 1
                torch.matmul(a, b.t(), out=c)
            t_ours = graph_time(ours)
            kernel, parts = binding.last_kernel_name(), binding.last_split_k()
            t_cublas = graph_time(cublas)
            flops = 2.0 * M * N * K
            table[key] = {"us": round(t_ours * 1e6, 1), "tflops": round(flops / t_ours / 1e12, 1), "kernel": kernel, "k_parts": parts,
                          "cublas_us": round(t_cublas * 1e6, 1), "cublas_tflops": round(flops / t_cublas / 1e12, 1)}
            del sets
            torch.cuda.empty_cache()
        except Exception as e:  # keep the headline even if a side measurement fails
            table[key] = {"error": str(e)[:200]}
    return table


def fp8_m_sharded(torch, dist, pkg, device, rank, world, barrier, steps=64, warmup=5):
    """The FP8 product M = 65536, N = K = 8192 split by rows over the ranks (the whole M on one GPU
    at world 1): one scale for all of A from the maximum over every rank's slab, B replicated.
    Times the product alone and, for world > 1, with the gather of C fused into the kernel and
    with the chunked NCCL all-gather."""
    ops, ms = pkg.sm120_ops, pkg.mshard
    spec = workload_spec("fp8_65536", world)
    M, N, K = spec["M"], spec["N"], spec["K"]
    g = torch.Generator(device=device)
    g.manual_seed(777)                                   # B: the same on every rank
    b, sb = ops.quantize_fp8(torch.randn(N, K, generator=g, device=device))
    g.manual_seed(1000 + rank)                           # A: this rank's slab
    a32 = torch.randn(M, K, generator=g, device=device)
    amax = a32.abs().max().reshape(1)
    if world > 1:
        dist.all_reduce(amax, op=dist.ReduceOp.MAX)      # set-up: every rank quantises with the same scale
    sa = (448.0 / amax).float()
    a, _ = ops.quantize_fp8(a32, scale=sa)
    del a32
    kw = dict(transpose_b=True, scale_a=sa, scale_b=sb)
    n_sets = 1 if spec["bytes"] > 3 * 126e6 else 2       # slabs of 8 ranks: alternate two outputs, operands exceed L2 with them
    sets = [(a, b, torch.empty(M, N, dtype=torch.bfloat16, device=device)) for _ in range(n_sets)]

    def local_step(a_, b_, out):
        ops.fused_matmul(a_, b_, out=out, **kw)

    secs = time_device_steps(torch, local_step, sets, steps, warmup, barrier)
    worst, per_rank = rank_stats(torch, dist, world, device, secs, steps)
    block = {
        "workload": "fp8_65536", "scaling": "strong", "M_total": spec["M_total"], "M_per_gpu": M, "N": N, "K": K,
        "steps": steps, "warmup": warmup, "ms_per_step": 1e3 * worst / steps, "per_rank_ms": per_rank,
        "tflops_total": world * spec["flops"] / (worst / steps) / 1e12,
        "pct_of_nominal_fp8_peak_per_gpu": 100.0 * spec["flops"] / (worst / steps) / 1e12 / NOMINAL_PEAK["f8e4m3"],
        "kernel": pkg._binding.last_kernel_name(),
        "operands": "N(0,1) quantised by the library's quantiser, scale 448/amax (A: amax over all ranks)",
    }
    if world > 1:
        sh = ms.MShardedMatmul(spec["M_total"], N)
        slab_bytes = M * N * 2
        gathers = {}
        del sets
        bufs = ms.PeerBuffers(sh, torch.bfloat16, device)

        def fused_step(a_, b_, out):
            sh.gathered_fused(a_, b_, bufs, **kw)

        def nccl_step(a_, b_, out):
            sh.gathered(a_, b_, out_dtype=torch.bfloat16, chunks=4, **kw)

        for name, fn in (("fused", fused_step), ("nccl", nccl_step)):
            s = time_device_steps(torch, fn, [(a, b, None)], max(16, steps // 2), 3, barrier)
            w, pr = rank_stats(torch, dist, world, device, s, max(16, steps // 2))
            t_step = w / max(16, steps // 2)
            gathers[name] = {"ms_per_step": 1e3 * t_step, "per_rank_ms": pr,
                             "nvlink_bytes_out_per_rank": (world - 1) * slab_bytes,
                             "nvlink_gbs_out_per_rank": (world - 1) * slab_bytes / t_step / 1e9,
                             "nvlink_floor_ms_at_770gbs": 1e3 * (world - 1) * slab_bytes / 770e9}
        gathers["fused"]["what"] = "one kernel per rank: the GEMM epilogue stores every C block to every rank (TMA stores over NVLink)"
        gathers["nccl"]["what"] = "GEMM in 4 row chunks, NCCL all-gather of chunk c on a side stream under the GEMM of chunk c+1"
        block["gather"] = gathers
        bufs.close()
    return block


def run_aux(args, torch, pkg, device, peaks, peak_kind):
    """HBM-bound kernels of the library: one JSON line with a bandwidth roofline."""
    ops, binding = pkg.sm120_ops, pkg._binding
    hbm = float(peaks.get("hbm_gbs", FALLBACK_PEAKS["hbm_gbs"]))
    n = 64 * 1024 * 1024
    if args.workload == "quant_fp8_64m":
        xs = [torch.randn(n, device=device).bfloat16() for _ in range(3)]
        nbytes = n * (2 + 2 + 1)          # x read twice (amax, cast), q written once
        what = "amax + scale + cast of 64 Mi bf16 elements to e4m3 (two launches)"

        def step(i):
            ops.quantize_fp8(xs[i % 3])
    elif args.workload == "activation_gelu_64m":
        xs = [torch.randn(n, device=device).bfloat16() for _ in range(3)]
        outs = [torch.empty_like(x) for x in xs]
        nbytes = n * 4
        what = "tanh-GELU of 64 Mi bf16 elements (sm120_launch_activation)"

        def step(i):
            ops.fused_activation(xs[i % 3], "gelu_tanh", out=outs[i % 3])
    elif args.workload == "softmax_131072x2048":
        xs = [torch.randn(131072, 2048, device=device).bfloat16() for _ in range(2)]
        outs = [torch.empty_like(x) for x in xs]
        nbytes = 131072 * 2048 * 4
        what = "row softmax of a bf16 [64 x 2048, 2048] score matrix (sm120_launch_softmax)"

        def step(i):
            ops.softmax(xs[i % 2], out=outs[i % 2])
    elif args.workload in ATTENTION_WORKLOADS:
        return run_attention(args, torch, pkg, device, peaks, peak_kind)
    else:
        xs = [torch.randn(8192, 11008, device=device).bfloat16() for _ in range(3)]
        nbytes = 8192 * 11008 * 2
        what = "column sums of a bf16 [8192, 11008] gradient (sm120_launch_bias_grad)"

        def step(i):
            ops.bias_grad(xs[i % 3])
    for i in range(args.warmup):
        step(i)
    torch.cuda.synchronize()
    launches0 = binding.launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        step(i)
    e1.record()
    torch.cuda.synchronize()
    secs = e0.elapsed_time(e1) * 1e-3 / args.steps
    line = {"metric": "hbm_bandwidth", "value": nbytes / secs / 1e9, "unit": "GB/s", "n_gpus": 1, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": secs * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic", "config": {"workload": args.workload, "what": what,
                                                             "l2": "three buffer sets of >= 128 MB rotate"},
            "roofline": {"bound": "hbm", "achieved": nbytes / secs / 1e9, "peak": hbm, "unit": "GB/s",
                         "frac": nbytes / secs / 1e9 / hbm, "traffic": None, "kernel": binding.last_kernel_name(),
                         "algorithmic_bytes_per_step": nbytes, "peak_source": f"{peak_kind}: hbm_gbs (copy)"},
            "gpu_launches": int(binding.launch_count() - launches0)}
    print(json.dumps(line), flush=True)


def run_attention(args, torch, pkg, device, peaks, peak_kind):
    """Fused attention forward, bf16; the default shape is the attention-score benchmark's (batch x heads = 64, sequence
    2048, head 128).  4 S^2 D FLOPs per batch entry (half of that with the causal mask); beside it the same result as
    GEMM + softmax + GEMM on this library (scores through HBM; sequences up to 4096) and the framework's own attention
    (torch.nn.functional.scaled_dot_product_attention, a yardstick only)."""
    ops, binding = pkg.sm120_ops, pkg._binding
    dims = args.workload.split("_")[1].split("x")
    bh, s, d = int(dims[0]), int(dims[1]), int(dims[2])
    causal = args.workload.endswith("_causal")
    sets = [tuple(torch.randn(bh, s, d, device=device).bfloat16() for _ in range(3)) for _ in range(3)]
    flops = 4.0 * s * s * d * bh * (0.5 if causal else 1.0)

    def timed(fn, steps, warmup):
        for i in range(warmup):
            fn(*sets[i % 3])
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(steps):
            fn(*sets[i % 3])
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) * 1e-3 / steps

    launches0 = binding.launch_count()
    secs = timed(lambda q, k, v: ops.scaled_dot_product_attention(q, k, v, causal_mask=causal), args.steps, args.warmup)
    launches = (binding.launch_count() - launches0) * args.steps // (args.steps + args.warmup)
    kernel = binding.last_kernel_name()
    unfused = None
    if s <= 4096 and not args.lean:
        zero_mask = torch.zeros(s, s, device=device)        # an explicit mask takes the unfused route
        unfused = timed(lambda q, k, v: ops.scaled_dot_product_attention(q, k, v, attention_mask=zero_mask, causal_mask=causal),
                        max(3, args.steps // 5), 2)
    library = None
    if not args.lean:
        try:
            sdpa = torch.nn.functional.scaled_dot_product_attention
            library = timed(lambda q, k, v: sdpa(q.unsqueeze(0), k.unsqueeze(0), v.unsqueeze(0), is_causal=causal), args.steps, args.warmup)
        except Exception:                                    # a yardstick only: absent or unsupported is not an error
            library = None
    peak = float(peaks.get("bf16_tflops", FALLBACK_PEAKS["bf16_tflops"]))
    tf = flops / secs / 1e12
    line = {"metric": METRIC, "value": tf, "unit": UNIT, "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": secs * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic",
            "config": {"workload": args.workload, "batch_x_heads": bh, "seq": s, "head_dim": d, "causal": causal,
                       "what": "softmax(Q K^T / sqrt(d)) V in one kernel", "l2": "three sets of Q, K, V rotate"},
            "roofline": {"bound": "tensor", "achieved": tf, "peak": peak, "unit": "TFLOP/s", "frac": tf / peak, "traffic": NCU_TRAFFIC_BYTES.get(args.workload),
                         "kernel": kernel, "algorithmic_flops_per_launch": flops, "algorithmic_bytes_per_launch": 4 * bh * s * d * 2,
                         "peak_source": f"{peak_kind}: bf16_tflops (cuBLAS bf16 8192^3 burst)"},
            "pct_of_nominal_dense_peak": 100.0 * tf / NOMINAL_PEAK["bf16"],
            "unfused_gemm_softmax_gemm": None if unfused is None else {"ms_per_step": unfused * 1e3, "tflops": flops / unfused / 1e12,
                                                                       "hbm_bytes_of_scores": bh * s * s * (4 + 4 + 2 + 2)},
            "torch_sdpa_same_process": None if library is None else {"ms_per_step": library * 1e3, "tflops": flops / library / 1e12},
            "gpu_launches": int(launches)}
    print(json.dumps(line), flush=True)


def write_trace(torch, ops, binding, spec, sets, kw, path):
    """One traced launch of the workload (after the timed region): per-CTA timeline as JSON, plus a summary."""
    a, b, out = sets[0]
    trace = torch.zeros(binding.TRACE_BYTES // 8, dtype=torch.int64, device=a.device)
    for _ in range(3):
        ops.fused_matmul(a, b, out=out, **kw)
    ops.fused_matmul(a, b, out=out, trace=trace, **kw)
    ops.fused_matmul(a, b, out=out, **kw)
    torch.cuda.synchronize()
    t = trace.cpu().numpy().reshape(binding.TRACE_MAX_CTAS, binding.TRACE_WORDS_PER_CTA)
    used = t[t[:, 4] != 0]
    if len(used) == 0:
        return None
    t_first = int(used[:, 0].min())
    rows = []
    for r in used:
        mhz = 1e3 * (int(r[5]) - int(r[1])) / max(1, int(r[4]) - int(r[0]))
        rows.append({"sm": int(r[7]), "tiles": int(r[6]), "enter_ns": int(r[0]) - t_first, "ready_ns": int(r[2]) - t_first,
                     "exit_ns": int(r[4]) - t_first, "cycles_alive": int(r[5]) - int(r[1]), "mhz": round(mhz, 1),
                     "setup_cycles": int(r[3]) - int(r[1]),
                     "tiles_cycles": [[int(r[8 + 4 * i + j]) - int(r[1]) if r[8 + 4 * i + j] else None for j in range(4)]
                                      for i in range(min(8, int(r[6])))]})
    summary = {"workload": spec["name"], "kernel": binding.last_kernel_name(), "ctas": len(rows),
               "launch_span_ns": int(used[:, 4].max()) - t_first,
               "median_cycles_alive": statistics.median(r["cycles_alive"] for r in rows),
               "median_mhz": statistics.median(r["mhz"] for r in rows)}
    with open(path, "w") as f:
        json.dump({"summary": summary, "ctas": rows}, f)
    return summary


def run_gpu(args, rank, world, local_rank):
    import torch
    import torch.distributed as dist

    pkg = importlib.import_module(PACKAGE_NAME)
    ops, binding = pkg.sm120_ops, pkg._binding
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if not ops.is_sm120_available():
        raise SystemExit("bench: no supported GPU or _sm120_ops.so missing (there is no fallback)")
    peaks, peak_kind = measured_peaks()
    if args.workload in AUX_WORKLOADS:
        if world > 1:
            raise SystemExit(f"{args.workload} is a single-GPU workload")
        return run_aux(args, torch, pkg, device, peaks, peak_kind)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
        token = torch.zeros(1, device=device)

        def barrier():
            dist.all_reduce(token)
            torch.cuda.synchronize()
    else:
        def barrier():
            return None

    spec = workload_spec(args.workload, world)
    reduce_max = None
    if spec.get("sharded") and world > 1:
        def reduce_max(t):
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            return t
    sets, kw = build_sets(torch, ops, spec, device, reduce_max=reduce_max)
    n_sets = len(sets)

    def plain_step(a, b, out):
        ops.fused_matmul(a, b, out=out, **kw)

    # optional gather of the M-sharded product (N > 1): NCCL all-gather per row chunk, or fused into the GEMM epilogue
    step_fn = plain_step
    if args.gather != "none":
        if world == 1:
            raise SystemExit("--gather needs --gpus N > 1")
        sh = pkg.mshard.MShardedMatmul(spec["M"] * world, spec["N"])
        out_dt = sets[0][2].dtype
        if args.gather == "fused":
            bufs = pkg.mshard.PeerBuffers(sh, out_dt, device)

            def step_fn(a, b, out):
                sh.gathered_fused(a, b, bufs, **kw)
        else:
            def step_fn(a, b, out):
                sh.gathered(a, b, out_dtype=out_dt, chunks=4, **kw)

    sampler = ClockSampler(nvml_index(torch, local_rank)) if rank == 0 else None
    launches0 = binding.launch_count()
    maps0 = binding.tensor_map_stats()
    if sampler:
        sampler.start()
    secs = time_device_steps(torch, step_fn, sets, args.steps, args.warmup, barrier)
    if sampler:
        sampler.stop()
    launches = binding.launch_count() - launches0
    launches = launches * args.steps // (args.steps + args.warmup)      # the same kernels run in every step, warm-up included
    maps1 = binding.tensor_map_stats()
    kernel = binding.last_kernel_name()
    kernel_mhz = binding.kernel_clock_mhz(local_rank) if kernel.startswith("tc_") else None
    if sampler and len(sampler.samples) < 5 and not args.lean:
        # the timed region was shorter than a few sampling periods: sample the same launches for ~0.3 s more
        sampler.start()
        t_end = time.perf_counter() + 0.3
        while time.perf_counter() < t_end:
            time_device_steps(torch, plain_step, sets, max(10, args.steps), 0, lambda: None)
        sampler.stop()
    secs, per_rank = rank_stats(torch, dist, world, device, secs, args.steps)

    yard = None
    if not args.lean and args.gather == "none":
        yard = cublas_yardstick(torch, spec, sets, kw, min(args.steps, 200), 3)

    # end to end from host buffers, every rank at once, max over ranks
    e2e = None
    if not args.lean:
        e2e_steps = max(1, min(args.steps, 100))
        e2e_secs, h2d, d2h = measure_e2e(torch, ops, spec, sets, kw, e2e_steps, min(args.warmup, 3))
        e2e_secs, e2e_per_rank = rank_stats(torch, dist, world, device, e2e_secs, e2e_steps)
        e2e = {"value": world * spec["flops"] / (e2e_secs / e2e_steps) / 1e12, "unit": UNIT,
               "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "ms_per_step": 1e3 * e2e_secs / e2e_steps,
               "per_rank_ms": e2e_per_rank, "steps": e2e_steps,
               "pcie_gbs_per_gpu": (h2d + d2h) / (e2e_secs / e2e_steps) / 1e9,
               "how": "fused_matmul on pinned host operands: B first, then row chunks of A in / product / C out on three streams"}

    probes = None
    if not args.lean and rank == 0:
        probes = {"pcie": pcie_probe(torch, device), "host_overhead": host_overhead(torch, ops, binding, device)}

    trace_summary = None
    if args.trace and rank == 0 and kernel.startswith("tc_"):
        trace_summary = write_trace(torch, ops, binding, spec, sets, kw, args.trace)

    status = __import__("ctypes").c_uint(0)
    binding.load_library().sm120_get_kernel_status(local_rank, __import__("ctypes").byref(status), 0)

    strong = None
    if not args.lean and not args.no_fp8_block and args.gather == "none":
        del sets
        torch.cuda.empty_cache()
        sets = None
        strong = fp8_m_sharded(torch, dist, pkg, device, rank, world, barrier)

    if rank == 0:
        per_launch = secs / args.steps
        tf_gpu = spec["flops"] / per_launch / 1e12
        peak = float(peaks.get("bf16_tflops", FALLBACK_PEAKS["bf16_tflops"]))
        hbm = float(peaks.get("hbm_gbs", FALLBACK_PEAKS["hbm_gbs"]))
        store_bound = spec["name"] == "bf16_batched_qk"
        if store_bound:
            roof = {"bound": "hbm", "achieved": spec["bytes"] / per_launch / 1e9, "peak": hbm, "unit": "GB/s"}
        else:
            # the e4m3 rate of the tensor pipe is twice the bf16 rate: scale the measured bf16 peak for the FP8 workload
            tpeak = peak * (2.0 if spec["dtype"] == "f8e4m3" else 1.0)
            roof = {"bound": "tensor", "achieved": tf_gpu, "peak": tpeak, "unit": "TFLOP/s"}
        roof["frac"] = roof["achieved"] / roof["peak"]
        roof["traffic"] = NCU_TRAFFIC_BYTES.get(spec["name"])
        roof["peak_source"] = f"{peak_kind}: MEASURED_PEAKS.json " + (
            "hbm_gbs (copy)" if store_bound else
            ("2 x bf16_tflops (cuBLAS bf16 8192^3 burst; e4m3 runs at twice the bf16 rate)" if spec["dtype"] == "f8e4m3"
             else "bf16_tflops (cuBLAS bf16 8192^3 burst)"))
        roof["kernel"] = kernel
        roof["algorithmic_flops_per_launch"] = spec["flops"]
        roof["algorithmic_bytes_per_launch"] = spec["bytes"]
        roof["launch_us"] = per_launch * 1e6
        # launch time in SM cycles at the clock the kernel itself saw: comparable between differently power-capped boxes
        roof["cycles_per_launch"] = per_launch * 1e6 * kernel_mhz if kernel_mhz else None

        cpu_tf, cpu_ms, cores, sample = (None, None, os.cpu_count(), "skipped (N > 1)")
        if world == 1 and not args.lean:
            cpu_tf, cpu_ms, cores, sample = cpu_product(spec, 3, 1)
        elif args.lean:
            sample = "skipped (--lean)"

        line = {
            "metric": METRIC, "value": world * tf_gpu, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": per_launch * 1e3, "higher_is_better": True,
            "scaling": spec["scaling"], "vs_baseline": None, "dtype": spec["dtype"], "data": "synthetic",
            "config": config_dict(args, spec, world,
                                  f"operands rotate over {n_sets} buffer set(s) of {spec['bytes'] / 1e6:.0f} MB; "
                                  "consecutive steps never reuse a set, total exceeds the 126 MB L2"),
            "tflops_per_gpu": tf_gpu,
            "per_rank_ms": per_rank,
            "pct_of_nominal_dense_peak": 100.0 * tf_gpu / NOMINAL_PEAK[spec["dtype"]],
            "pct_of_measured_bf16_peak": 100.0 * tf_gpu / peak,
            "roofline": roof,
            "cublas_same_process": yard,
            "cpu_baseline": {"value": cpu_tf, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample,
                             "ms_per_step": cpu_ms},
            "e2e": e2e,
            "gpu_launches": int(launches),
            "host_overhead": probes["host_overhead"] if probes else None,
            "pcie_probe": probes["pcie"] if probes else None,
            "tensor_maps": {"encoded": maps1[0] - maps0[0], "reused": maps1[1] - maps0[1]},
            "clocks": dict(sampler.summary(), sm_mhz_in_kernel=kernel_mhz) if sampler else None,
            "kernel_status": int(status.value),
            "fp8_m_sharded": strong,
        }
        if trace_summary:
            line["trace"] = trace_summary
        if world == 1 and not args.no_side_table and not args.lean:
            line["all_configs"] = side_table(torch, ops, binding, device)
            line["small_shapes"] = small_shapes(torch, ops, binding, device)
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=500)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--workload", default="f16_4096_tn",
                    choices=sorted(WORKLOADS) + sorted(ALIASES) + list(AUX_WORKLOADS))
    ap.add_argument("--impl", default="sm120", choices=["sm120", "reference"])
    ap.add_argument("--gather", default="none", choices=["none", "nccl", "fused"],
                    help="N > 1 only: also produce the whole C on every rank inside the timed step, by an NCCL "
                         "all-gather (per row chunk, overlapped) or by the GEMM epilogue's own peer stores")
    ap.add_argument("--no-side-table", action="store_true", help="skip the per-workload table at N=1")
    ap.add_argument("--no-fp8-block", action="store_true", help="skip the M-sharded FP8 measurement")
    ap.add_argument("--trace", default=None, help="write the launch timeline of one launch to this file (JSON)")
    ap.add_argument("--lean", action="store_true",
                    help="for runs under a profiler: the timed launches only (no CPU baseline, cuBLAS yardstick, "
                         "end-to-end, FP8 block, side table or extra launches for clock sampling)")
    args = ap.parse_args()
    args.workload = ALIASES.get(args.workload, args.workload)
    args.warmup = max(3, args.warmup) if args.impl == "sm120" else args.warmup
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus and world > 1:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    if args.gpus > 1 and world == 1:
        raise SystemExit("for --gpus N > 1 launch with: python -m torch.distributed.run --nproc-per-node N bench.py --gpus N ...")
    if args.impl == "reference":
        if args.workload in AUX_WORKLOADS:
            raise SystemExit("the reference arm times the matmul workloads")
        run_reference(args, rank, world)
    else:
        run_gpu(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
