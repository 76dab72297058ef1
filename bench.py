"""Throughput of the NF4 + LoRA training hot path on B200.

    python bench.py --gpus N --steps K --warmup W              # this repository's CUDA path
    python bench.py --impl reference --gpus N --steps K ...     # the reference's own CPU implementation

Default workload `step7b` (BASELINE.json configs[4]): one optimizer update of the 7B-class MQA decoder -
32 layers, hidden 4096, 32 + 1 heads of 128, SwiGLU MLP 14336, vocab 49152, NF4 base weights in 64-element
blocks with fp32 absmax, rank-256 adapters on all seven projections, bf16 compute, fp32 adapters / gradients
/ Adam state, 4 packed rows of 4096 tokens per GPU with document lengths log-uniform in [64, 4096] - through
`Trainer.update`: batch to the device, forward, tiled lm_head loss, backward, (N > 1) NCCL all-reduce of
the adapter gradients, clip, AdamW, loss back to the host. `--workload step1b` is configs[3], `--workload
projection` is configs[1] (one gate/up-shaped projection, forward + backward). All data is synthetic and
seeded.

Rank 0 prints ONE JSON line. `value` is whole-job tokens/s with the batch resident in HBM; `e2e` is the same
update fed from pinned host memory with the loss read back; `roofline` is the tcgen05 GEMM kernels'
algorithmic FLOP/s over their own CUDA-event time against the measured cuBLAS bf16 peak, with the DRAM
traffic of those kernels from an ncu capture of one decoder layer scaled to the step; `projection_op` is
configs[1] timed in the same process (the "projection TFLOP/s vs peak" half of the metric);
`reference_gpu` is the unmodified reference (oracle/_ref: cuBLAS + Triton + FlashAttention-2) timed on the
same GPU with the same weights and batch - reported beside the line, never used in it; `cpu_baseline` and
`--impl reference` time the unmodified reference's CPU branch on the host cores on a bounded sample.
"""

import argparse
import json
import os
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

ROWS, INNER, OUTER, RANK = 16384, 4096, 14336, 256
CPU_SAMPLE_ROWS = 512
METRIC = "train tokens/s (NF4 r256 LoRA projection fwd+bwd, 7B gate/up shape)"
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def projection_flops(rows):
    """Algorithmic work of one step: 4TKN + 6TKr + 6TNr (no recomputation counted)."""
    return 4 * rows * INNER * OUTER + 6 * rows * INNER * RANK + 6 * rows * OUTER * RANK


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return json.load(f), "measured"
    return dict(FALLBACK_PEAKS), "fallback"


def world():
    return int(os.environ.get("RANK", 0)), int(os.environ.get("LOCAL_RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))


# ---------------------------------------------------------------------------------------------
class ClockSampler(threading.Thread):
    """Reads SM clock and throttle reasons of one GPU through NVML. It is started before the warm-up
    (NVML start-up takes tens of milliseconds); `window()` keeps the samples taken between `mark()` and
    `stop()`, i.e. during the timed region."""

    def __init__(self, index, period=0.004):
        super().__init__(daemon=True)
        self.index, self.period = index, period
        self.samples, self.max_mhz, self.error = [], None, None
        self._stop_event = threading.Event()
        self._start_time = None

    def run(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            handle = pynvml.nvmlDeviceGetHandleByIndex(self.index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(handle, pynvml.NVML_CLOCK_SM)
            names = {"HwSlowdown": "hw_slowdown", "HwThermalSlowdown": "hw_thermal_slowdown",
                     "SwThermalSlowdown": "sw_thermal_slowdown", "SwPowerCap": "sw_power_cap"}
            masks = {}
            for suffix, label in names.items():
                for prefix in ("nvmlClocksEventReason", "nvmlClocksThrottleReason"):
                    if hasattr(pynvml, prefix + suffix):
                        masks[getattr(pynvml, prefix + suffix)] = label
            read = getattr(pynvml, "nvmlDeviceGetCurrentClocksEventReasons", None) or \
                pynvml.nvmlDeviceGetCurrentClocksThrottleReasons
            while not self._stop_event.is_set():
                clock = pynvml.nvmlDeviceGetClockInfo(handle, pynvml.NVML_CLOCK_SM)
                active = read(handle)
                labels = tuple(label for mask, label in masks.items() if active & mask)
                self.samples.append((time.perf_counter(), clock, labels))
                time.sleep(self.period)
        except Exception as error:  # NVML missing: report that instead of clocks
            self.error = f"nvml_unavailable:{type(error).__name__}"

    def mark(self):
        self._start_time = time.perf_counter()

    def stop(self):
        end = time.perf_counter()
        self._stop_event.set()
        self.join(timeout=2)
        inside = [s for s in self.samples if self._start_time is not None and self._start_time <= s[0] <= end]
        if not inside and self.samples:   # region shorter than one sampling period: nearest sample
            inside = [min(self.samples, key=lambda s: abs(s[0] - end))]
        ordered = sorted(s[1] for s in inside)
        reasons = sorted({label for s in inside for label in s[2]})
        if self.error:
            reasons.append(self.error)
        return {"sm_mhz": ordered[len(ordered) // 2] if ordered else None, "sm_max_mhz": self.max_mhz,
                "reasons": reasons, "samples": len(ordered)}


def physical_gpu_index(local_rank):
    visible = os.environ.get("CUDA_VISIBLE_DEVICES")
    if visible:
        try:
            return int(visible.split(",")[local_rank])
        except (ValueError, IndexError):
            pass
    return local_rank


# ---------------------------------------------------------------------------------------------
class CpuProjection:
    """The reference's CPU branch of one projection (modeling/lora.py:29-39 + torch autograd) on `rows` tokens of the
    workload: the unmodified `Projection` from oracle/_ref when it is installed (kind "reference"), else the oracle's
    restatement of that branch (kind "port")."""

    def __init__(self, rows, dtype, threads):
        from oracle import ref_bridge
        torch.set_num_threads(threads)
        generator = torch.Generator().manual_seed(1234)
        self.rows, self.dtype = rows, dtype
        weight = (torch.randn(OUTER, INNER, generator=generator) * .02).to(dtype)
        a = torch.randn(RANK, INNER, generator=generator) * .02
        b = torch.randn(OUTER, RANK, generator=generator) * .01
        self.x = torch.randn(rows, INNER, generator=generator).to(dtype).requires_grad_(True)
        self.dy = torch.randn(rows, OUTER, generator=generator).to(dtype)
        self.kind = "reference" if ref_bridge.available() else "port"
        if self.kind == "reference":
            ref_bridge.load()
            from causal_tuner.modeling.lora import Projection
            self.module = Projection(INNER, OUTER, rank=RANK, base_dtype=dtype, compute_dtype=dtype, device="cpu")
            with torch.no_grad():
                self.module.weight.copy_(weight)
                self.module.lora_A.copy_(a)
                self.module.lora_B.copy_(b)
            self.a, self.b = self.module.lora_A, self.module.lora_B
        else:
            self.weight, self.a, self.b = weight, a.requires_grad_(True), b.requires_grad_(True)

    def step(self):
        if self.kind == "reference":
            y = self.module(self.x)
        else:
            from oracle import ops
            y = ops.projection(self.x, self.weight, self.a, self.b, None, self.dtype)
        return torch.autograd.grad(y, (self.x, self.a, self.b), self.dy)

    def seconds_per_step(self, steps):
        start = time.perf_counter()
        for _ in range(steps):
            self.step()
        return (time.perf_counter() - start) / steps


def faster_cpu_projection(threads):
    """bf16 and fp32 compute are both legitimate reference settings; keep whichever this host runs faster."""
    best = None
    for name, dtype in (("bf16", torch.bfloat16), ("fp32", torch.float32)):
        candidate = CpuProjection(CPU_SAMPLE_ROWS, dtype, threads)
        candidate.step()
        seconds = candidate.seconds_per_step(1)
        if best is None or seconds < best[0]:
            best = (seconds, name, candidate)
    return best[1], best[2]


def cpu_sample_text(name, steps, kind="port"):
    source = ("the reference's own Projection (oracle/_ref, unmodified), CPU branch modeling/lora.py:29-39 + autograd"
              if kind == "reference" else "oracle/ops.py restating the reference CPU branch modeling/lora.py:29-39 + autograd")
    return (f"{steps} steps of {CPU_SAMPLE_ROWS} of the {ROWS} rows (full K, N, rank; cost is linear in rows), "
            f"{name} compute, {source}")


def cpu_baseline(seconds=12.0):
    threads = os.cpu_count() or 1
    name, problem = faster_cpu_projection(threads)
    one = problem.seconds_per_step(1)
    steps = max(3, min(200, int(seconds / max(one, 1e-3))))
    per_step = problem.seconds_per_step(steps)
    return {"value": CPU_SAMPLE_ROWS / per_step, "unit": "tokens/s", "cores": threads, "kind": problem.kind,
            "sample": cpu_sample_text(name, steps, problem.kind)}


def run_reference(args):
    """The reference arm of the projection workload: the reference's CPU branch on this machine's host cores,
    all threads; each step is one pass over a bounded sample of the workload's rows."""
    rank, _, _ = world()
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    name, problem = faster_cpu_projection(threads)
    for _ in range(max(args.warmup, 1)):
        problem.step()
    per_step = problem.seconds_per_step(args.steps)
    value = CPU_SAMPLE_ROWS / per_step
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1000.0 * per_step,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": name, "data": "synthetic",
            "config": workload_config(args.gpus, bool(args.keep_low_rank)),
            "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": threads, "kind": problem.kind,
                             "sample": cpu_sample_text(name, args.steps, problem.kind)},
            "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


def workload_config(gpus, keep_low_rank=True):
    return {"workload": "projection_fwd_bwd_7b_gate (BASELINE.json configs[1])", "rows_per_gpu": ROWS, "in_features": INNER,
            "out_features": OUTER, "rank": RANK, "nf4_blocksize": 64, "absmax": "fp32",
            "low_rank_input": ("x.A^T kept for backward" if keep_low_rank
                               else "recomputed in backward (as the reference does)"),
            "parallelism": f"dp{gpus}", "l2": "inputs (134 MB X + 470 MB dY per step) are larger than the 126 MB L2"}


# ---------------------------------------------------------------------------------------------
def run_ours(args):
    rank, local_rank, world_size = world()
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the operators have no CPU path "
                         "(use --impl reference for the CPU composition)")
    import torch.distributed as dist
    from causal_tuner_b200 import _lib
    from causal_tuner_b200.dp import GradientExchange
    from causal_tuner_b200.kernels.linear import project_group
    from causal_tuner_b200.modeling.lora import Projection

    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    distributed = world_size > 1
    if distributed:
        dist.init_process_group("nccl", device_id=device)
    _lib.load()

    torch.manual_seed(2024)  # identical weights on every rank
    module = Projection(INNER, OUTER, rank=RANK, device=device)
    module.install_nf4(module.weight.detach().clone(), device, blocksize=64, nested=False)
    module.keep_low_rank = bool(args.keep_low_rank)
    with torch.no_grad():
        module.lora_A.normal_(std=.02)
        module.lora_B.normal_(std=.01)
    generator = torch.Generator(device="cpu").manual_seed(77 + rank)  # rank-specific rows
    x_host = torch.randn(ROWS, INNER, generator=generator).bfloat16().pin_memory()
    dy_host = torch.randn(ROWS, OUTER, generator=generator).bfloat16().pin_memory()
    x = x_host.to(device).requires_grad_(True)
    dy = dy_host.to(device)
    parameters = (module.lora_A, module.lora_B)

    def step(inputs=x, upstream=dy):
        y = project_group((module,), inputs)[0]
        dx, da, db = torch.autograd.grad(y, (inputs, *parameters), upstream)
        if distributed:
            exchange = GradientExchange()
            exchange.add(da)
            exchange.add(db)
            exchange.finish()
        return y, dx, da, db

    def barrier():
        if distributed:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(function, steps):
        barrier()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(steps):
            function()
        stop.record()
        barrier()
        elapsed = torch.tensor([start.elapsed_time(stop)], device=device, dtype=torch.float64)
        if distributed:
            dist.all_reduce(elapsed, op=dist.ReduceOp.MAX)
        return elapsed.item() / steps

    # ---- device-resident throughput --------------------------------------------------------
    sampler = ClockSampler(physical_gpu_index(local_rank))
    sampler.start()
    for _ in range(max(args.warmup, 3)):
        step()
    _lib.check_device()
    sampler.mark()
    launches_before = _lib.launch_count()
    _lib.timing_enable(True)
    ms_per_step = timed(step, args.steps)
    kernel_ms, kernel_flops, kernel_launches = _lib.timing_collect()
    _lib.timing_enable(False)
    launches = _lib.launch_count() - launches_before
    clocks = sampler.stop()
    _lib.check_device()

    e2e_ms, e2e_steps, h2d, d2h = None, 0, 0, 0
    if not args.no_e2e:
        e2e_ms, e2e_steps, h2d, d2h = end_to_end(args, module, parameters, x, dy, x_host, dy_host, distributed, timed)
    _lib.check_device()
    finish(args, rank, world_size, distributed, ms_per_step, e2e_ms, e2e_steps, h2d, d2h, launches, kernel_ms,
           kernel_flops, kernel_launches, clocks)


def end_to_end(args, module, parameters, x, dy, x_host, dy_host, distributed, timed):
    """Host buffers in, every result back out, copies overlapped with compute on two side streams."""
    from causal_tuner_b200.dp import GradientExchange
    from causal_tuner_b200.kernels.linear import project_group
    device = x.device
    y_host = torch.empty(ROWS, OUTER, dtype=torch.bfloat16).pin_memory()
    dx_host = torch.empty(ROWS, INNER, dtype=torch.bfloat16).pin_memory()
    da_host = torch.empty(RANK, INNER, dtype=torch.float32).pin_memory()
    db_host = torch.empty(OUTER, RANK, dtype=torch.float32).pin_memory()
    x_dev = torch.empty_like(x, requires_grad=True)
    dy_dev = torch.empty_like(dy)
    upload, download = torch.cuda.Stream(device), torch.cuda.Stream(device)

    def e2e_step():
        compute = torch.cuda.current_stream()
        upload.wait_stream(compute)
        with torch.cuda.stream(upload):
            x_dev.data.copy_(x_host, non_blocking=True)
            x_ready = torch.cuda.Event()
            x_ready.record(upload)
            dy_dev.copy_(dy_host, non_blocking=True)
            dy_ready = torch.cuda.Event()
            dy_ready.record(upload)
        compute.wait_event(x_ready)
        y = project_group((module,), x_dev)[0]
        download.wait_stream(compute)
        with torch.cuda.stream(download):
            y_host.copy_(y, non_blocking=True)   # overlaps the upload of dY and the backward pass
        compute.wait_event(dy_ready)
        dx, da, db = torch.autograd.grad(y, (x_dev, *parameters), dy_dev)
        if distributed:
            exchange = GradientExchange()
            exchange.add(da)
            exchange.add(db)
            exchange.finish()
        download.wait_stream(compute)
        with torch.cuda.stream(download):
            dx_host.copy_(dx, non_blocking=True)
            da_host.copy_(da, non_blocking=True)
            db_host.copy_(db, non_blocking=True)
        compute.wait_stream(download)
        for tensor in (y, dx, da, db):
            tensor.record_stream(download)
        torch.cuda.current_stream().synchronize()  # the host owns the results before the next step

    e2e_steps = max(2, min(args.steps, 10))
    for _ in range(2):
        e2e_step()
    e2e_ms = timed(e2e_step, e2e_steps)
    h2d = x_host.numel() * 2 + dy_host.numel() * 2
    d2h = y_host.numel() * 2 + dx_host.numel() * 2 + da_host.numel() * 4 + db_host.numel() * 4
    if not (torch.isfinite(y_host[:64].float()).all() and torch.isfinite(da_host).all()):
        raise RuntimeError("end-to-end leg produced non-finite results")
    return e2e_ms, e2e_steps, h2d, d2h


def finish(args, rank, world_size, distributed, ms_per_step, e2e_ms, e2e_steps, h2d, d2h, launches, kernel_ms,
           kernel_flops, kernel_launches, clocks):
    import torch.distributed as dist
    if rank != 0:
        if distributed:
            dist.destroy_process_group()
        return
    peaks, peak_kind = measured_peaks()
    tokens = ROWS * world_size
    achieved = kernel_flops / (kernel_ms * 1e-3) / 1e12 if kernel_ms > 0 else None
    peak = float(peaks["bf16_tflops"])
    line = {
        "metric": METRIC, "value": tokens / (ms_per_step * 1e-3), "unit": "tokens/s", "n_gpus": world_size,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": workload_config(world_size, bool(args.keep_low_rank)),
        "step_tflops_per_gpu": projection_flops(ROWS) / (ms_per_step * 1e-3) / 1e12,
        "step_frac_of_bf16_peak": projection_flops(ROWS) / (ms_per_step * 1e-3) / 1e12 / peak,
        "e2e": None if e2e_ms is None else {
            "value": tokens / (e2e_ms * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": h2d,
            "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms, "steps": e2e_steps},
        "gpu_launches": launches,
        "roofline": {"bound": "tensor", "kernel": "gemm_tcgen05_kernel", "achieved": achieved, "peak": peak,
                     "unit": "TFLOP/s", "frac": (achieved / peak) if achieved else None,
                     "peak_source": f"{peak_kind} cuBLAS bf16 burst (MEASURED_PEAKS.json)",
                     "launches": kernel_launches, "kernel_ms_per_step": kernel_ms / args.steps,
                     "traffic": None},
        "clocks": clocks,
    }
    if world_size == 1 and not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_baseline()
    print(json.dumps(line), flush=True)
    if distributed:
        dist.destroy_process_group()


STEP_METRIC = "train tokens/s (NF4 r256 LoRA, MQA decoder, one optimizer update)"


def step_config(name, gpus, mlp_cache_gib=0, execution=None, keep_low_rank=False):
    import bench_step
    spec = bench_step.WORKLOADS[name]
    config = spec["config"]
    per_layer = spec["rows"] * spec["length"] * 2 * (2 * config["intermediate_size"] + 2 * bench_step.RANK)
    planned = min(config["num_hidden_layers"], int(mlp_cache_gib * 2**30) // per_layer)   # MLP.cache_bytes per layer
    cached = planned if execution is None else execution.get("mlp_cache_layers", 0)
    kept_mb = 5 * bench_step.RANK * 2 * spec["rows"] * spec["length"] / 1e6
    return {"workload": f"{name} ({spec['reference']})", **spec["config"], "rank": bench_step.RANK,
            "rows_per_gpu": spec["rows"], "seq_len": spec["length"], "global_batch": spec["rows"] * gpus,
            "nf4_blocksize": 64, "absmax": "fp32", "attention": "flash_attention_2 (library, as in the reference)",
            "activation_checkpointing": False,
            "mlp": (f"gate/up kept for backward in {cached} layers ({mlp_cache_gib} GiB budget, last layers first), "
                    f"recomputed in backward in the others"),
            "low_rank_inputs": (f"x.A^T of q/k/v/o and (with the MLP cache) down kept for backward ({kept_mb:.1f} MB per layer)" if keep_low_rank
                                else "recomputed in backward (as the reference does)"),
            "parallelism": f"dp{gpus}",
            "rows": ("one global batch of n_gpus x rows_per_gpu packed rows (seed 1000); ranks take rows_per_gpu rows "
                     "each from the cost-balanced assignment (tokens + document length^2 / (12 x seq_len))"),
            "l2": "per-layer operands (>= 134 MB activations + 117 MB decoded weight) exceed the 126 MB L2"}


def reference_cpu_line(workload, steps, warmup):
    """Times `steps` whole updates of the unmodified reference on the host cores (after `warmup`). Returns
    (tokens/s, seconds per update, cpu_baseline record). Falls back to the oracle's restatement of one layer
    + head (kind "port") on a machine where oracle/_ref was never installed."""
    import bench_step
    threads = os.cpu_count() or 1
    if not bench_step.reference_cpu_available():
        estimate = bench_step.cpu_estimate(workload, passes=max(1, min(steps, 5)))
        return estimate["value"], bench_step.CPU_SAMPLE_TOKENS / estimate["value"], estimate
    problem = bench_step.ReferenceCpuStep(workload, threads)
    started = time.perf_counter()
    problem.step()
    first = time.perf_counter() - started
    # A host on which steps + warm-up would take more than about five minutes gets a smaller sample.
    while problem.tokens > 128 and first * (steps + warmup) > 300:
        problem.resize(problem.tokens // 2)
        first /= 2
    for _ in range(max(warmup - 1, 0) if problem.tokens == bench_step.CPU_SAMPLE_TOKENS else warmup):
        problem.step()
    start = time.perf_counter()
    for _ in range(steps):
        metrics = problem.step()
    seconds = (time.perf_counter() - start) / steps
    rate = metrics["valid_tokens"] / seconds
    record = {"value": rate, "unit": "tokens/s", "cores": threads, "kind": "reference",
              "sample": problem.sample_text(steps), "seconds_per_update": seconds, "loss": metrics["loss"]}
    return rate, seconds, record


def run_step_reference(args):
    """The reference arm: rank 0 alone runs the reference's CPU implementation; each step is one whole
    optimizer update on a bounded sample (one 512-token packed row) of the workload's batch."""
    rank, _, _ = world()
    if rank != 0:
        return
    rate, seconds, record = reference_cpu_line(args.workload, args.steps, max(args.warmup, 1))
    config = step_config(args.workload, args.gpus, args.mlp_cache_gib, None, bool(args.keep_low_rank))
    config["reference_step"] = ("ms_per_step is one update on a 512-token sample of the per-GPU batch, not on the whole "
                                "batch; tokens/s is what compares")
    line = {"impl": "reference", "metric": STEP_METRIC, "value": rate, "unit": "tokens/s",
            "n_gpus": args.gpus, "steps": args.steps, "warmup": max(args.warmup, 1),
            "ms_per_step": 1000.0 * seconds, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": config,
            "cpu_baseline": record,
            "e2e": {"value": rate, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


def projection_op_record(device, steps=20):
    """BASELINE.json configs[1] inside the same process: one fused NF4 + LoRA projection (M = 16384, K = 4096,
    N = 14336, rank 256), forward Y and backward dX, dA, dB through `project_group`, CUDA events, inputs larger
    than L2. Algorithmic FLOP 4TKN + 6TKr + 6TNr against the measured cuBLAS burst peak (a kernel timed alone)."""
    from causal_tuner_b200.kernels.linear import project_group
    from causal_tuner_b200.modeling.lora import Projection
    torch.manual_seed(2024)
    module = Projection(INNER, OUTER, rank=RANK, device=device)
    module.install_nf4(module.weight.detach().clone(), device, blocksize=64, nested=False)
    module.keep_low_rank = True
    with torch.no_grad():
        module.lora_A.normal_(std=.02)
        module.lora_B.normal_(std=.01)
    generator = torch.Generator(device=device).manual_seed(77)
    x = torch.randn(16384, INNER, device=device, generator=generator).bfloat16().requires_grad_(True)
    dy = torch.randn(16384, OUTER, device=device, generator=generator).bfloat16()

    def step():
        y = project_group((module,), x)[0]
        torch.autograd.grad(y, (x, module.lora_A, module.lora_B), dy)

    for _ in range(3):
        step()
    torch.cuda.synchronize(device)
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(steps):
        step()
    stop.record()
    torch.cuda.synchronize(device)
    ms = start.elapsed_time(stop) / steps
    peaks, kind = measured_peaks()
    tflops = projection_flops(16384) / (ms * 1e-3) / 1e12
    record = {"workload": "projection_fwd_bwd_7b_gate (BASELINE.json configs[1])", "ms": ms, "tflops": tflops,
              "frac_of_bf16_burst_peak": tflops / float(peaks["bf16_tflops"]), "peak_source": kind,
              "tokens_per_s": 16384 / (ms * 1e-3), "steps": steps}
    return record, module, x, dy


def reference_gpu_record(model, device, batch, tokens, projection=None, table=None):
    """The unmodified reference (oracle/_ref) on this GPU: its Triton kernels, cuBLAS and FlashAttention-2 through
    its own `Trainer.update`, on a replica that shares this model's packed NF4 weights and starts from copies of
    its adapters, same batch; and its `project_group` on configs[1]. A reported comparison only."""
    from oracle import ref_bridge
    if not ref_bridge.available():
        return {"unavailable": "oracle/_ref is not installed on this machine"}
    try:
        import triton  # noqa: F401
    except ImportError:
        return {"unavailable": "triton is not importable; the reference's CUDA path needs it"}
    record = {}
    ref_bridge.load()
    if projection is not None:
        from causal_tuner.kernels.linear import project_group as reference_group
        module, x, dy = projection
        theirs = ref_bridge.mirror_projection(module)

        def step():
            y = reference_group((theirs,), x)[0]
            torch.autograd.grad(y, (x, theirs.lora_A, theirs.lora_B), dy)
        for _ in range(3):
            step()
        torch.cuda.synchronize(device)
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(10):
            step()
        stop.record()
        torch.cuda.synchronize(device)
        ms = start.elapsed_time(stop) / 10
        record["projection_op"] = {"ms": ms, "tflops": projection_flops(16384) / (ms * 1e-3) / 1e12}
        del theirs
    # Policy pinned to this arm's: no layer checkpointing, the same MLP activation-cache budget.
    theirs = ref_bridge.mirror_model(model)
    trainer = ref_bridge.reference_trainer(theirs, device, loss_token_budget=4096)
    for index in range(2):              # Triton compiles its kernels in the first update
        metrics = trainer.update([dict(batch)], step=index, total_steps=1 << 20)
    torch.cuda.synchronize(device)
    steps = 3
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for index in range(steps):
        metrics = trainer.update([dict(batch)], step=2 + index, total_steps=1 << 20)
    stop.record()
    torch.cuda.synchronize(device)
    ms = start.elapsed_time(stop) / steps
    if table:
        kernel_table(lambda: trainer.update([dict(batch)], step=5, total_steps=1 << 20), table,
                     "one update of the unmodified reference (oracle/_ref: Triton + cuBLAS + FlashAttention-2), same weights and batch")
    record.update({"value": tokens / (ms * 1e-3), "unit": "tokens/s", "ms_per_step": ms, "steps": steps,
                   "loss": metrics["loss"], "execution": {k: v for k, v in metrics["execution"][0].items()},
                   "what": "reference CausalLM + Trainer.update from oracle/_ref (Triton + cuBLAS + FlashAttention-2), "
                           "same packed NF4 weights, adapters and batch, same GPU, 1 GPU"})
    return record


def kernel_table(update, path, title):
    """Device time per kernel of ONE update under torch.profiler (CUPTI), written to `path` as a text table.
    Diagnostic: kernels run serialised and slightly slower under the profiler; compare rows, not the total
    with a bench value."""
    from torch.profiler import ProfilerActivity, profile
    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA]) as session:
        update()
        torch.cuda.synchronize()
    rows = []
    for event in session.key_averages():
        total = getattr(event, "device_time_total", None)
        if total is None:
            total = getattr(event, "cuda_time_total", 0)
        if total > 0:
            rows.append((total, event.count, event.key))
    rows.sort(reverse=True)
    grand = sum(row[0] for row in rows) or 1
    with open(path, "w") as handle:
        handle.write(f"{title}\ntotal device time {grand / 1000:.2f} ms in {sum(r[1] for r in rows)} launches\n")
        for total, count, name in rows[:60]:
            handle.write(f"{total / 1000:10.2f} ms {100 * total / grand:5.1f} %  n={count:5d}  {name[:140]}\n")


# The GEMM shapes of one decoder layer of step7b (16384 tokens): (name, M, N, K, layout). NT: B given as [N, K]
# (forward products); NN: B given as [K, N] (input gradients, dy . W); TN: both operands token-major, fp32 output
# (adapter gradients).
STEP_SHAPES = [("fwd gate/up", 16384, 14336, 4352, "NT"), ("fwd q/o", 16384, 4096, 4352, "NT"),
               ("fwd down", 16384, 4096, 14592, "NT"), ("dx down", 16384, 14336, 4352, "NN"),
               ("dx gate+up", 16384, 4096, 29184, "NN"), ("dx o", 16384, 4096, 4352, "NN"),
               ("x.A^T", 16384, 256, 4096, "NT"), ("x.A^T q/k/v", 16384, 768, 4096, "NT"),
               ("dy.B gate", 16384, 256, 14336, "NN"), ("k/v forward", 16384, 128, 4352, "NT"),
               ("dB gate", 14336, 256, 16384, "TN"), ("dA down", 256, 14336, 16384, "TN"),
               ("dB q", 4096, 256, 16384, "TN"), ("dA q/k/v", 768, 4096, 16384, "TN")]


def run_shapes(args):
    """`--workload shapes`: every GEMM shape of a step7b layer through this library's tcgen05 kernels and through
    torch.matmul (cuBLAS) on the same operands, alternating bursts of about 60 ms, best of two; one JSON line.
    A same-device yardstick for the kernels, not a bench line."""
    from causal_tuner_b200.kernels import linear
    torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False
    device = torch.device("cuda", 0)
    make = lambda *shape: (torch.randn(*shape, device=device) * .1).bfloat16()

    def burst(function, count):
        function()
        function()
        torch.cuda.synchronize()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(count):
            function()
        stop.record()
        torch.cuda.synchronize()
        return start.elapsed_time(stop) / count * 1000

    table = {}
    for name, m, n, k, layout in STEP_SHAPES:
        if layout == "TN":
            left, right = make(k, m), make(k, n)
            ours_out, library_out = (torch.empty(m, n, device=device) for _ in range(2))
            ours = lambda: linear.token_gradient(left, right, ours_out)
            library = lambda: torch.mm(left.T, right, out_dtype=torch.float32, out=library_out)
        else:
            left = make(m, k)
            right = make(n, k).T if layout == "NT" else make(k, n)
            ours_out, library_out = (torch.empty(m, n, device=device, dtype=torch.bfloat16) for _ in range(2))
            ours = lambda: linear.matmul(left, right, out=ours_out)
            library = lambda: torch.mm(left, right, out=library_out)
        flop = 2 * m * n * k
        count = max(20, int(6e4 / (flop / 1.3e15 * 1e6)))
        best = [min(burst(f, count) for _ in range(2)) for f in (ours, library)]
        table[name] = {"M": m, "N": n, "K": k, "layout": layout, "ours_us": best[0], "cublas_us": best[1],
                       "ours_tflops": flop / best[0] / 1e6, "cublas_tflops": flop / best[1] / 1e6,
                       "rel_diff": ((ours_out.float() - library_out.float()).norm() / library_out.float().norm()).item()}
        del left, right, ours_out, library_out
    # Where should the NF4 decode run? The gate/up base product x . dequant(W)^T (K = 4096, N = 14336) with the
    # decode as its own kernel into a dense scratch followed by the GEMM (what the operators do), against the
    # decode inside the GEMM's producer stage (ct_matmul_nf4), which repeats it for every 256-row tile of x.
    from causal_tuner_b200.kernels.nf4_cuda import dequantize_nf4
    from causal_tuner_b200.quant import quantize_nf4
    packed, state = quantize_nf4((torch.randn(OUTER, INNER, device=device) * .02).bfloat16(), blocksize=64, nested=False)
    placement = {}
    for tokens in (256, 512, 1024, 4096, 16384):
        x = make(tokens, INNER)
        out_once, out_fused = (torch.empty(tokens, OUTER, device=device, dtype=torch.bfloat16) for _ in range(2))
        once = lambda: linear.matmul(x, dequantize_nf4(packed, state, torch.bfloat16).T, out=out_once)
        fused = lambda: linear.matmul_nf4(x, packed, state, out=out_fused)
        count = max(20, int(6e4 / (2 * tokens * OUTER * INNER / 1.3e15 * 1e6 + 30)))
        best = [min(burst(f, count) for _ in range(2)) for f in (once, fused)]
        placement[str(tokens)] = {"decode_then_gemm_us": best[0], "decode_inside_gemm_us": best[1],
                                  "identical": bool(torch.equal(out_once, out_fused))}
        del x, out_once, out_fused
    print(json.dumps({"workload": "shapes (GEMMs of one step7b layer, ours vs torch.matmul on the same GPU)", "shapes": table,
                      "nf4_decode_placement": placement}), flush=True)


# DRAM traffic of the tcgen05 GEMM kernels (profiles/step7b_gemm_dram_traffic_ncu.md): `dram__bytes_read.sum +
# dram__bytes_write.sum` summed over the GEMM launches of one update of this workload cut to ONE and to TWO decoder
# layers (16384 tokens, forward + backward, MLP activations kept, the lm_head's GEMMs included). The difference
# is one layer, the rest is the head; every layer launches the same GEMMs, so a step is layers x layer + head.
# `operands` is the least those launches could move: every operand read once and every result written once.
GEMM_DRAM_TRAFFIC = {"step7b": {"layer_bytes": 19.03e9, "head_bytes": 10.30e9, "layer_launches": 25, "head_launches": 12,
                                "operands_bytes_per_step": 348e9}}


def gemm_traffic(workload, config, launches_per_step):
    """`traffic`: DRAM bytes per GEMM launch, averaged over the launches of a step, for the roofline record; None
    for a workload of which no capture is on file."""
    capture = GEMM_DRAM_TRAFFIC.get(workload)
    if not capture or not launches_per_step:
        return {"traffic": None}
    layers = config["num_hidden_layers"]
    step_bytes = layers * capture["layer_bytes"] + capture["head_bytes"]
    launches = layers * capture["layer_launches"] + capture["head_launches"]
    return {"traffic": step_bytes / launches, "traffic_per_step": step_bytes,
            "operand_bytes_per_step": capture["operands_bytes_per_step"],
            "traffic_note": (f"ncu dram__bytes_read.sum + dram__bytes_write.sum over the GEMM launches of this workload with 1 "
                             f"and with 2 decoder layers; step = {layers} x (difference) + head = {launches} launches "
                             f"(this run: {launches_per_step:.0f}); operand bytes = every operand read once, every result "
                             f"written once")}


def run_step(args):
    """One optimizer update per step through `Trainer.update`: host batch -> device, forward, tiled loss,
    backward, (N > 1: NCCL all-reduce of the fp32 adapter gradients), clip, AdamW, loss back to the host."""
    import torch.distributed as dist
    import bench_step
    from causal_tuner_b200 import _lib
    from causal_tuner_b200.training import Trainer, make_optimizer
    rank, local_rank, world_size = world()
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the operators have no CPU path "
                         "(use --impl reference for the CPU composition)")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    distributed = world_size > 1
    if distributed:
        dist.init_process_group("nccl", device_id=device)
    _lib.load()
    spec = bench_step.WORKLOADS[args.workload]
    if args.layers:        # profiler-sized case: fewer layers of the same shapes (not a bench value)
        spec = dict(spec, config=dict(spec["config"], num_hidden_layers=args.layers))
        bench_step.WORKLOADS[args.workload] = spec
    model = bench_step.build_model(args.workload, device, args.mlp_cache_gib, keep_low_rank=bool(args.keep_low_rank))
    optimizer = make_optimizer(model, learning_rate=2e-5)
    trainer = Trainer(model, optimizer, device=device, loss_token_budget=4096)
    # One global batch of world_size x rows packed rows, the same on every rank; each rank takes the rows
    # the cost-balanced assignment gives it (rows per rank fixed, so the per-GPU token count does not
    # change with N, but no rank is left with all the long documents).
    host_batch = bench_step.synthetic_batch(spec["rows"] * world_size, spec["length"], spec["config"]["vocab_size"],
                                            seed=1000)
    if world_size > 1:
        from causal_tuner_b200.dp import balance_rows, row_costs
        costs = row_costs(host_batch["attention_mask"], host_batch["segment_ids"], width=spec["length"])
        mine = torch.tensor(balance_rows(costs, world_size)[rank])
        host_batch = {key: value[mine].contiguous() for key, value in host_batch.items()}
    host_batch = {k: v.pin_memory() for k, v in host_batch.items()}
    device_batch = {k: v.to(device) for k, v in host_batch.items()}
    tokens_per_rank = spec["rows"] * spec["length"]

    def barrier():
        if distributed:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(batch, steps):
        barrier()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        losses = [trainer.update([batch])["loss"] for _ in range(steps)]
        stop.record()
        barrier()
        elapsed = torch.tensor([start.elapsed_time(stop)], device=device, dtype=torch.float64)
        if distributed:
            dist.all_reduce(elapsed, op=dist.ReduceOp.MAX)
        return elapsed.item() / steps, losses

    sampler = ClockSampler(physical_gpu_index(local_rank))
    sampler.start()
    for _ in range(max(args.warmup, 3)):
        trainer.update([device_batch])
    _lib.check_device()
    sampler.mark()
    launches_before = _lib.launch_count()
    _lib.timing_enable(True)
    ms_per_step, losses = timed(device_batch, args.steps)
    kernel_ms, kernel_flops, kernel_launches = _lib.timing_collect()
    _lib.timing_enable(False)
    launches = _lib.launch_count() - launches_before
    clocks = sampler.stop()
    e2e_ms, _ = timed(host_batch, max(2, min(args.steps, 5)))   # ids from pinned host memory, loss back to host
    _lib.check_device()
    peak_memory = torch.cuda.max_memory_allocated(device)
    # The same update with every layer recomputing its MLP activations in backward (no cache budget):
    # the low-memory end of the policy, reported beside the headline so that both are on record.
    recompute = None
    if args.mlp_cache_gib and model.last_execution.get("mlp_cache_layers") and not args.no_recompute_arm:
        execution = dict(model.last_execution)
        model.runtime.mlp_cache_budget_bytes = None
        for module in model.modules():
            if hasattr(module, "keep_low_rank"):
                module.keep_low_rank = False       # the reference's policy: nothing kept beyond x and the parameters
        torch.cuda.reset_peak_memory_stats(device)
        trainer.update([device_batch])
        recompute_ms, _ = timed(device_batch, max(2, min(args.steps, 3)))
        recompute = {"value": tokens_per_rank * world_size / (recompute_ms * 1e-3), "unit": "tokens/s",
                     "ms_per_step": recompute_ms, "peak_memory_gb": torch.cuda.max_memory_allocated(device) / 1e9}
        model.last_execution = execution
        model.runtime.mlp_cache_budget_bytes = int(args.mlp_cache_gib * 2**30) or None
        for module in model.modules():
            if hasattr(module, "keep_low_rank"):
                module.keep_low_rank = bool(args.keep_low_rank)
    if rank != 0:
        if distributed:
            dist.destroy_process_group()
        return
    # Reported beside the line, measured after it (N = 1 only): configs[1] in this process, and the unmodified
    # reference's CUDA path on the same GPU, weights and batch.
    if args.kernel_table:
        kernel_table(lambda: trainer.update([device_batch]), args.kernel_table + "_ours.txt",
                     f"{args.workload}: one update of this library (MLP cache budget {args.mlp_cache_gib} GiB)")
    projection_op, reference_gpu = None, None
    if world_size == 1 and not args.no_extras:
        trainer.optimizer.zero_grad(set_to_none=True)
        projection_op, module, x, dy = projection_op_record(device)
        try:
            reference_gpu = reference_gpu_record(model, device, device_batch, tokens_per_rank, (module, x, dy),
                                                 table=args.kernel_table and args.kernel_table + "_reference_gpu.txt")
        except Exception as error:      # a reported extra must not take the bench line down with it
            reference_gpu = {"unavailable": f"{type(error).__name__}: {error}"[:300]}
        del module, x, dy
    peaks, peak_kind = measured_peaks()
    peak = float(peaks.get("bf16_tflops_sustained", peaks["bf16_tflops"]))
    tokens = tokens_per_rank * world_size
    flops = bench_step.step_flops(spec["config"], tokens_per_rank)
    achieved = kernel_flops / (kernel_ms * 1e-3) / 1e12 if kernel_ms > 0 else None
    h2d = sum(v.numel() * v.element_size() for v in host_batch.values())
    line = {
        "metric": STEP_METRIC, "value": tokens / (ms_per_step * 1e-3), "unit": "tokens/s", "n_gpus": world_size,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": step_config(args.workload, world_size, args.mlp_cache_gib, model.last_execution,
                              bool(args.keep_low_rank)),
        "step_tflops_per_gpu": flops / (ms_per_step * 1e-3) / 1e12,
        "step_frac_of_bf16_peak": flops / (ms_per_step * 1e-3) / 1e12 / peak,
        "e2e": {"value": tokens / (e2e_ms * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": 4, "ms_per_step": e2e_ms},
        "gpu_launches": launches,
        "roofline": {"bound": "tensor", "kernel": "gemm_tcgen05_{pair,wide,gated,group}_kernel (one body, gemm_tc.cu)",
                     "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": (achieved / peak) if achieved else None,
                     "peak_source": f"{peak_kind} cuBLAS bf16 sustained (kernel timed inside a long step)",
                     "launches": kernel_launches, "kernel_ms_per_step": kernel_ms / args.steps,
                     **gemm_traffic(args.workload, spec["config"], kernel_launches / args.steps)},
        "clocks": clocks, "loss_first": losses[0], "loss_last": losses[-1],
        "peak_memory_gb": peak_memory / 1e9, "mlp_recompute_everywhere": recompute,
        "projection_op": projection_op, "reference_gpu": reference_gpu,
    }
    if world_size == 1 and not args.no_cpu_baseline:
        line["cpu_baseline"] = reference_cpu_line(args.workload, steps=3, warmup=1)[2]
    print(json.dumps(line), flush=True)
    if distributed:
        dist.destroy_process_group()


def main():
    global ROWS
    parser = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=20)
    parser.add_argument("--warmup", type=int, default=3)
    parser.add_argument("--impl", choices=("ours", "reference"), default="ours")
    parser.add_argument("--rows", type=int, default=ROWS,
                        help="tokens per GPU; anything but the default is a profiler-sized case, not a bench value")
    parser.add_argument("--no-e2e", action="store_true", help="skip the host-buffer leg (profiler captures)")
    parser.add_argument("--no-cpu-baseline", action="store_true", help="skip the CPU leg (profiler captures)")
    parser.add_argument("--no-extras", action="store_true",
                        help="skip the projection_op and reference_gpu records (profiler captures)")
    parser.add_argument("--layers", type=int, default=0,
                        help="decoder layers of a step workload; anything but the default is a profiler-sized case")
    parser.add_argument("--keep-low-rank", type=int, choices=(0, 1), default=1,
                        help="keep the low-rank inputs x.A^T (q/k/v/o in the step workloads) for backward (1) or recompute them as the reference does (0)")
    parser.add_argument("--no-recompute-arm", action="store_true",
                        help="skip the second measurement with every MLP recomputing its activations (profiler captures)")
    parser.add_argument("--mlp-cache-gib", type=float, default=64.0,
                        help="per-GPU byte budget for keeping MLP gate/up activations instead of recomputing them "
                             "(0: always recompute)")
    parser.add_argument("--workload", choices=("step7b", "step1b", "projection", "shapes"), default="step7b",
                        help="step7b: 7B-class decoder update (the headline metric); step1b: the 1.3B decoder; "
                             "projection: one fused NF4+LoRA projection, forward+backward; shapes: the GEMM shapes of a "
                             "step7b layer against torch.matmul (a diagnostic table, not a bench line)")
    parser.add_argument("--kernel-table", default=None, metavar="PREFIX",
                        help="also write per-kernel device-time tables of one update (torch.profiler) to PREFIX_ours.txt "
                             "and, with the reference_gpu record, PREFIX_reference_gpu.txt")
    args = parser.parse_args()
    ROWS = args.rows
    if args.workload == "shapes":
        run_shapes(args)
    elif args.workload == "projection":
        run_reference(args) if args.impl == "reference" else run_ours(args)
    else:
        run_step_reference(args) if args.impl == "reference" else run_step(args)


if __name__ == "__main__":
    main()
