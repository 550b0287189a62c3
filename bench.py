#!/usr/bin/env python
"""Benchmark of the SM120 matmul op on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload cfg2] [--impl reference]

One "step" is one GEMM of the workload through the C ABI.  The default workload
is BASELINE configuration 2 (fp16, M=N=K=4096, A row-major, B stored [N,K],
fp32 accumulate, fp16 out).  With N > 1 (one process per GPU, launched by
torchrun) every rank multiplies its own 4096-row slab of A by the replicated B:
the M-sharded product with M = 4096*N, no data-path collective, weak scaling.
`--workload cfg5` runs the FP8 configuration (M = 65536 split over the ranks,
strong scaling); cfg1/cfg3/cfg4 are single-GPU.

Rank 0 prints ONE JSON line.  `value` is whole-job TFLOP/s with the operands
resident in HBM; `e2e` is the same product through the public Python API from
pinned host buffers (host->device and device->host copies inside the timed
region); `roofline` compares the kernel with the measured cuBLAS bf16 peak of
this pool; `cpu_baseline` is the oracle's fp32 host-BLAS product timed on this
box's cores.  `--impl reference` times only that CPU product.
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

METRIC = "gemm_tflops"          # BASELINE.json: GEMM TFLOP/s per GPU and % of B200 dense tensor peak at 1/2/4/8 GPUs
UNIT = "TFLOP/s"
NOMINAL_PEAK = {"f16": 2250.0, "bf16": 2250.0, "f8e4m3": 4500.0, "f32": 80.0}   # dense, per GPU, datasheet
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}

# dram__bytes_read.sum + dram__bytes_write.sum per launch of the dominant kernel,
# from the ncu capture summarised under profiles/ (None until captured).
NCU_TRAFFIC_BYTES = {
    "cfg2": 93319680,       # profiles/gemm_tcgen05_cfg2_fp16_4096.txt: 74.60 MB read + 18.72 MB written
    "cfg2bf16": 93319680,   # same kernel, shape and byte counts as cfg2
    "cfg3": 529810176,      # profiles/gemm_tcgen05_cfg3_bf16_dense_gelu.txt: 366.6 MB read + 163.2 MB written
    "cfg4": 546989312,      # profiles/gemm_tcgen05_cfg4_bf16_batched.txt: 67.2 MB read + 479.8 MB written
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
    if name == "cfg1":
        s = dict(M=1024, N=1024, K=1024, batch=1, dtype="f32", in_bytes=4, out_bytes=4, scaling="weak")
    elif name == "cfg2":
        s = dict(M=4096, N=4096, K=4096, batch=1, dtype="f16", in_bytes=2, out_bytes=2, scaling="weak")
    elif name == "cfg2bf16":
        s = dict(M=4096, N=4096, K=4096, batch=1, dtype="bf16", in_bytes=2, out_bytes=2, scaling="weak")
    elif name == "cfg3":
        s = dict(M=8192, N=11008, K=4096, batch=1, dtype="bf16", in_bytes=2, out_bytes=2, scaling="weak")
    elif name == "cfg4":
        s = dict(M=2048, N=2048, K=128, batch=64, dtype="bf16", in_bytes=2, out_bytes=2, scaling="weak")
    elif name == "cfg5":
        if 65536 % world != 0:
            raise SystemExit("cfg5 needs a world size that divides 65536")
        s = dict(M=65536 // world, N=8192, K=8192, batch=1, dtype="f8e4m3", in_bytes=1, out_bytes=2, scaling="strong")
    else:
        raise SystemExit(f"unknown workload {name}")
    s["name"] = name
    s["flops"] = 2.0 * s["M"] * s["N"] * s["K"] * s["batch"]
    s["bytes"] = s["batch"] * ((s["M"] * s["K"] + s["K"] * s["N"]) * s["in_bytes"] + s["M"] * s["N"] * s["out_bytes"])
    return s


def make_device_operands(spec, seed, device):
    """Synthetic operands with the configuration's shapes and value distributions,
    drawn on the device from a seeded generator."""
    import torch
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    M, N, K, B = spec["M"], spec["N"], spec["K"], spec["batch"]
    name = spec["name"]
    kw = {}
    if name == "cfg1":
        a = torch.rand(M, K, generator=g, device=device) * 2 - 1
        b = torch.rand(K, N, generator=g, device=device) * 2 - 1
    elif name in ("cfg2", "cfg2bf16"):
        dt = torch.float16 if name == "cfg2" else torch.bfloat16
        a = (torch.randn(M, K, generator=g, device=device) / K ** 0.5).to(dt)
        b = (torch.randn(N, K, generator=g, device=device) / K ** 0.5).to(dt)      # stored [N, K]
        kw["transpose_b"] = True
    elif name == "cfg3":
        a = torch.randn(M, K, generator=g, device=device).bfloat16()
        b = (0.02 * torch.randn(K, N, generator=g, device=device)).bfloat16()
        kw["bias"] = (0.02 * torch.randn(N, generator=g, device=device)).bfloat16()
        kw["activation"] = "gelu"
    elif name == "cfg4":
        a = torch.randn(B, M, K, generator=g, device=device).bfloat16()
        b = torch.randn(B, K, N, generator=g, device=device).bfloat16()
    else:  # cfg5: N(0,1) quantised with s = 448/amax; amax of N(0,1) over these sizes is ~5.5-6
        a32 = torch.randn(M, K, generator=g, device=device)
        b32 = torch.randn(N, K, generator=g, device=device)
        sa, sb = 448.0 / 6.0, 448.0 / 6.0       # one scale for every rank, fixed in advance
        a = (a32 * sa).clamp_(-448, 448).to(torch.float8_e4m3fn)
        b = (b32 * sb).clamp_(-448, 448).to(torch.float8_e4m3fn)
        del a32, b32
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
    return {"workload": args.workload, "gather": getattr(args, "gather", "none"), "M_per_gpu": spec["M"], "M_total": spec["M"] * world, "N": spec["N"],
            "K": spec["K"], "batch": spec["batch"], "sharding": "M-slabs, B replicated; collective only with --gather", "l2": l2_note}


# ---------------------------------------------------------------------------
# reference arm / CPU baseline: the oracle's fp32 host-BLAS product
# ---------------------------------------------------------------------------
def cpu_sample_shapes(spec):
    """A bounded sample of the workload for the CPU: the first rows of A only,
    sized to ~35 GFLOP per step so that a run of many steps ends within minutes."""
    per_row = 2.0 * spec["N"] * spec["K"] * spec["batch"]
    rows = int(max(64, min(spec["M"], 3.5e10 // per_row)))
    return rows, f"first {rows} of {spec['M']} rows of A per step (all of B), fp32 torch.matmul (MKL) + the epilogue"


def cpu_product(spec, steps, warmup):
    """Times `steps` CPU products of the sample; returns (TFLOP/s, ms/step, cores, sample text)."""
    import numpy as np
    import torch
    from oracle import reference as ref

    rows, text = cpu_sample_shapes(spec)
    rng = np.random.default_rng(0)
    N, K, B = spec["N"], spec["K"], spec["batch"]
    lead = (B,) if B > 1 else ()
    name = spec["name"]
    tb = name in ("cfg2", "cfg2bf16", "cfg5")
    a = rng.standard_normal(lead + (rows, K), dtype=np.float32)
    b = rng.standard_normal(lead + ((N, K) if tb else (K, N)), dtype=np.float32)
    bias = rng.standard_normal((N,), dtype=np.float32) if name == "cfg3" else None
    act = 9 if name == "cfg3" else -1
    cores = os.cpu_count() or 1
    times = []
    for i in range(warmup + steps):
        _, secs, cores = ref.cpu_baseline_fp32(a, b, transpose_b=tb, bias=bias, act=act, threads=cores, repeats=1)
        if i >= warmup:
            times.append(secs)
    total = sum(times)
    flops = 2.0 * rows * N * K * B
    return flops * len(times) / total / 1e12, 1e3 * total / len(times), cores, text


def run_reference(args, rank, world):
    spec = workload_spec(args.workload, world)
    if rank != 0:
        return
    tflops, ms, cores, text = cpu_product(spec, args.steps, min(args.warmup, 2))
    line = {
        "impl": "reference", "metric": METRIC, "value": tflops, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": min(args.warmup, 2), "ms_per_step": ms, "higher_is_better": True, "scaling": spec["scaling"],
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": config_dict(args, spec, world, "host memory; every step multiplies the same bounded sample"),
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


def time_device_steps(torch, ops, sets, kw, steps, warmup, barrier, step_fn=None):
    """W warm-up steps, then K steps rotating over the buffer sets, timed with CUDA
    events on the launch stream.  A step is one product (step_fn may add the gather
    of an M-sharded product).  Returns seconds for the K steps."""
    if step_fn is None:
        def step_fn(a, b, out):
            ops.fused_matmul(a, b, out=out, **kw)
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


def build_sets(torch, spec, device, min_total_bytes=3 * 126e6, max_sets=4):
    """Buffer sets (A, B, C) so that consecutive steps never find their operands in
    the 126 MB L2: at least 2 sets and at least ~380 MB in total, unless one set
    alone is larger than that."""
    out_dt = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16, "f8e4m3": torch.bfloat16}[spec["dtype"]]
    n_sets = int(min(max_sets, max(2, -(-min_total_bytes // spec["bytes"])))) if spec["bytes"] < min_total_bytes else 1
    sets, kw = [], {}
    for s in range(n_sets):
        a, b, kw = make_device_operands(spec, 1234 + s, device)
        shape = ((spec["batch"],) if spec["batch"] > 1 else ()) + (spec["M"], spec["N"])
        sets.append((a, b, torch.empty(shape, dtype=out_dt, device=device)))
    return sets, kw


def measure_e2e(torch, ops, spec, sets, kw, steps, warmup):
    """The same product through the public API with HOST operands: every step copies
    A and B from pinned host memory to the device, multiplies, and copies C back into
    a pinned host buffer.  Wall-clock around `steps` calls, device synchronised on
    both sides.  Returns (seconds, h2d bytes per step, d2h bytes per step)."""
    a_d, b_d, c_d = sets[0]
    a_h = torch.empty(a_d.shape, dtype=a_d.dtype, pin_memory=True).copy_(a_d)
    b_h = torch.empty(b_d.shape, dtype=b_d.dtype, pin_memory=True).copy_(b_d)
    c_h = torch.empty(c_d.shape, dtype=c_d.dtype, pin_memory=True)
    kw_h = dict(kw)
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


def side_table(torch, ops, binding, device, peaks):
    """Single-GPU TFLOP/s of every BASELINE configuration (10 launches each after 3
    warm-ups, CUDA events), reported beside the headline."""
    table = {}
    for name in ("cfg1", "cfg2", "cfg2bf16", "cfg3", "cfg4", "cfg5"):
        spec = workload_spec(name, 8 if name == "cfg5" else 1)      # cfg5: one rank's slab of the 8-way shard
        try:
            sets, kw = build_sets(torch, spec, device)
            secs = time_device_steps(torch, ops, sets, kw, 10, 3, lambda: None)
            ms = 1e3 * secs / 10
            tf = spec["flops"] / (secs / 10) / 1e12
            table[name] = {"ms": round(ms, 4), "tflops": round(tf, 1), "gbs": round(spec["bytes"] / (secs / 10) / 1e9, 1),
                           "pct_nominal_peak": round(100 * tf / NOMINAL_PEAK[spec["dtype"]], 1),
                           "kernel": binding.last_kernel_name(),
                           "shape": [spec["batch"], spec["M"], spec["N"], spec["K"]]}
            del sets
            torch.cuda.empty_cache()
        except Exception as e:  # keep the headline even if a side measurement fails
            table[name] = {"error": str(e)[:200]}
    return table


def run_gpu(args, rank, world, local_rank):
    import torch
    import torch.distributed as dist

    pkg = importlib.import_module(PACKAGE_NAME)
    ops, binding = pkg.sm120_ops, pkg._binding
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if not ops.is_sm120_available():
        raise SystemExit("bench: no supported GPU or _sm120_ops.so missing (there is no fallback)")
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
    peaks, peak_kind = measured_peaks()
    sets, kw = build_sets(torch, spec, device)
    n_sets = len(sets)

    # optional gather of the M-sharded product (N > 1): NCCL all-gather per row chunk, or fused into the GEMM epilogue
    step_fn = None
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
    if sampler:
        sampler.start()
    secs = time_device_steps(torch, ops, sets, kw, args.steps, args.warmup, barrier, step_fn)
    if sampler:
        sampler.stop()
    launches = binding.launch_count() - launches0 - args.warmup
    kernel = binding.last_kernel_name()
    if sampler and len(sampler.samples) < 5 and not args.lean:
        # the timed region was shorter than a few sampling periods: sample the same launches for ~0.3 s more
        sampler.start()
        t_end = time.perf_counter() + 0.3
        while time.perf_counter() < t_end:
            time_device_steps(torch, ops, sets, kw, max(10, args.steps), 0, lambda: None)
        sampler.stop()

    if world > 1:
        t = torch.tensor([secs], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        secs = float(t.item())

    # end to end from host buffers, every rank at once, max over ranks
    e2e_steps = max(1, min(args.steps, 100))
    e2e_secs, h2d, d2h = measure_e2e(torch, ops, spec, sets, kw, e2e_steps, min(args.warmup, 3))
    if world > 1:
        t = torch.tensor([e2e_secs], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_secs = float(t.item())

    # SM clock seen from inside the last launch (%clock64 over %globaltimer of CTA 0)
    probe = (__import__("ctypes").c_ulonglong * 2)()
    lib = binding.load_library()
    lib.sm120_debug_read_probe.argtypes = [__import__("ctypes").c_void_p]
    lib.sm120_debug_read_probe(probe)
    kernel_mhz = 1e3 * probe[0] / probe[1] if probe[1] else None

    status = __import__("ctypes").c_uint(0)
    binding.load_library().sm120_get_kernel_status(local_rank, __import__("ctypes").byref(status), 0)

    if rank == 0:
        per_launch = secs / args.steps
        tf_gpu = spec["flops"] / per_launch / 1e12
        peak = float(peaks.get("bf16_tflops", FALLBACK_PEAKS["bf16_tflops"]))
        hbm = float(peaks.get("hbm_gbs", FALLBACK_PEAKS["hbm_gbs"]))
        store_bound = spec["name"] == "cfg4"
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
            "pct_of_nominal_dense_peak": 100.0 * tf_gpu / NOMINAL_PEAK[spec["dtype"]],
            "pct_of_measured_bf16_peak": 100.0 * tf_gpu / peak,
            "roofline": roof,
            "cpu_baseline": {"value": cpu_tf, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample,
                             "ms_per_step": cpu_ms},
            "e2e": {"value": world * spec["flops"] / (e2e_secs / e2e_steps) / 1e12, "unit": UNIT,
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "ms_per_step": 1e3 * e2e_secs / e2e_steps,
                    "steps": e2e_steps},
            "gpu_launches": int(launches),
            "clocks": dict(sampler.summary(), sm_mhz_in_kernel=kernel_mhz) if sampler else None,
            "kernel_status": int(status.value),
        }
        if world == 1 and not args.no_side_table and not args.lean:
            del sets
            torch.cuda.empty_cache()
            line["all_configs"] = side_table(torch, ops, binding, device, peaks)
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=500)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--workload", default="cfg2", choices=["cfg1", "cfg2", "cfg2bf16", "cfg3", "cfg4", "cfg5"])
    ap.add_argument("--impl", default="sm120", choices=["sm120", "reference"])
    ap.add_argument("--gather", default="none", choices=["none", "nccl", "fused"],
                    help="N > 1 only: also produce the whole C on every rank inside the timed step, by an NCCL "
                         "all-gather (per row chunk, overlapped) or by the GEMM epilogue's own peer stores")
    ap.add_argument("--no-side-table", action="store_true", help="skip the per-configuration table at N=1")
    ap.add_argument("--lean", action="store_true",
                    help="for runs under a profiler: also skip the CPU baseline and the extra launches that lengthen a "
                         "short timed region for clock sampling")
    args = ap.parse_args()
    args.warmup = max(3, args.warmup) if args.impl == "sm120" else args.warmup
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus and world > 1:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    if args.gpus > 1 and world == 1:
        raise SystemExit("for --gpus N > 1 launch with: python -m torch.distributed.run --nproc-per-node N bench.py --gpus N ...")
    if args.impl == "reference":
        run_reference(args, rank, world)
    else:
        run_gpu(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
