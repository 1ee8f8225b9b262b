"""Benchmark of the PINN training step: collocation points per second per full
Adam step (forward, reverse pass, gradient all-reduce, optimizer update).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

Launched under `python -m torch.distributed.run` for N > 1 (one rank per GPU).
Prints ONE JSON line on rank 0.

The default workload is the 2-D Poisson configuration (float32, tanh MLP
2-64x4-1, 65,536 interior + 4,096 boundary points per GPU).  Inputs are seeded
synthetic points and Xavier-normal weights.  With N GPUs every rank holds its
own 65,536 + 4,096 points (weak scaling) and the step ends with one all-reduce
of the flat [loss, gradients] buffer.

  value  device-resident step: points and parameters already in HBM;
  e2e    the same step through `optim.Trainer.step(batch)` with the batch
         copied from pinned host memory every step and the step's loss read
         back, both inside the timed region.
"""

from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "collocation_points_per_second_per_adam_step"
UNIT = "points/s"


def parse_args():
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=20)
    parser.add_argument("--warmup", type=int, default=5)
    parser.add_argument("--impl", default="ours", choices=["ours", "reference"])
    parser.add_argument("--workload", default="poisson2d")
    parser.add_argument("--points", type=int, default=None, help="interior points per GPU (default: the workload's)")
    parser.add_argument("--cpu-seconds", type=float, default=12.0, help="target CPU time of the bounded CPU sample")
    parser.add_argument("--no-cpu-baseline", action="store_true")
    return parser.parse_args()


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as handle:
            return json.load(handle), "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}, "fallback"


class ClockSampler:
    """Samples the SM clock and the throttle reasons of one GPU while the timed region runs:
    NVML from a thread every 10 ms (plus one reading at the start and one at the end, so that
    even a region of a few milliseconds is covered); nvidia-smi when NVML cannot be loaded.
    Read-only: no setting of the GPU is touched."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    REASONS = {0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown"}

    def __init__(self, index: int, uuid: str | None = None) -> None:
        self.index = index
        self.process = None
        self.lines: list[str] = []
        self.sm: list[float] = []
        self.reasons: set[str] = set()
        self.sm_max = None
        self.nvml = None
        self.handle = None
        self.stop_flag = threading.Event()
        self.thread = None
        try:
            import pynvml

            pynvml.nvmlInit()
            handle = None
            if uuid:
                try:
                    handle = pynvml.nvmlDeviceGetHandleByUUID(uuid if uuid.startswith("GPU-") else "GPU-" + uuid)
                except Exception:
                    handle = None
            self.handle = handle if handle is not None else pynvml.nvmlDeviceGetHandleByIndex(index)
            self.sm_max = float(pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM))
            self.nvml = pynvml
        except Exception:
            self.nvml = None

    def _read_nvml(self) -> None:
        nv = self.nvml
        try:
            self.sm.append(float(nv.nvmlDeviceGetClockInfo(self.handle, nv.NVML_CLOCK_SM)))
            getter = getattr(nv, "nvmlDeviceGetCurrentClocksEventReasons", None) or nv.nvmlDeviceGetCurrentClocksThrottleReasons
            mask = int(getter(self.handle))
            for bit, name in self.REASONS.items():
                if mask & bit:
                    self.reasons.add(name)
        except Exception:
            pass

    def _loop(self) -> None:
        while not self.stop_flag.wait(0.01):
            self._read_nvml()

    def start(self) -> None:
        if self.nvml is not None:
            self._read_nvml()
            self.thread = threading.Thread(target=self._loop, daemon=True)
            self.thread.start()
            return
        try:
            self.process = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.process = None

    def _read(self) -> None:
        for line in self.process.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.nvml is not None:
            self._read_nvml()
            self.stop_flag.set()
            if self.thread is not None:
                self.thread.join(timeout=1.0)
            return {"sm_mhz": float(np.median(self.sm)) if self.sm else None, "sm_max_mhz": self.sm_max,
                    "samples": len(self.sm), "reasons": sorted(self.reasons), "source": "nvml, 10 ms"}
        if self.process is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "samples": 0, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.process.terminate()
        sm, sm_max, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            fields = [f.strip() for f in line.split(",")]
            if len(fields) < 9:
                continue
            try:
                sm.append(float(fields[1]))
                sm_max.append(float(fields[2]))
            except ValueError:
                continue
            for name, flag in zip(names, fields[5:9]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(sm_max) if sm_max else None,
                "samples": len(sm), "reasons": sorted(reasons), "source": "nvidia-smi, 100 ms"}


def cpu_sample(workload_name: str, seconds: float, threads: int):
    """Times the CPU oracle's value-and-gradient on a bounded sample of the
    workload's interior points; returns (points/s, sample description)."""
    from oracle import contracted
    from quabla_b200 import workloads
    from quabla_b200._transforms import CompiledLoss

    contracted.build()
    probe_points = 256
    w = workloads.make(workload_name, probe_points)
    args = (w.params, *w.data)
    traced = CompiledLoss(w.loss, args, (0,), 0, build_plan=False)
    inputs = traced.named_inputs(args)
    t0 = time.perf_counter()
    contracted.value_and_grad(traced.spec, inputs, threads=threads)
    probe = max(time.perf_counter() - t0, 1e-4)
    full = workloads.make(workload_name).interior_points
    points = int(min(full, max(probe_points, probe_points * seconds / probe)))
    w = workloads.make(workload_name, points)
    args = (w.params, *w.data)
    traced = CompiledLoss(w.loss, args, (0,), 0, build_plan=False)
    inputs = traced.named_inputs(args)
    t0 = time.perf_counter()
    contracted.value_and_grad(traced.spec, inputs, threads=threads)
    elapsed = time.perf_counter() - t0
    sample = (f"{w.interior_points} of {full} interior points (+ proportionally scaled boundary sets), one "
              f"value-and-gradient pass, float64, oracle/contracted.c, {threads} thread(s), {elapsed:.2f} s")
    return w.interior_points / elapsed, sample


def run_reference(args) -> None:
    """The reference arm: the reference's CPU algorithm for the path on the host
    cores.  The reference itself is Rust and cannot be built in this image (no
    cargo/rustc), so this times the oracle port with every host thread."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import contracted
    from quabla_b200 import workloads

    threads = contracted.max_threads()
    per_step = max(1.0, min(8.0, 120.0 / max(1, args.steps + args.warmup)))
    values = []
    sample = ""
    for step in range(args.warmup + args.steps):
        value, sample = cpu_sample(args.workload, per_step, threads)
        if step >= args.warmup:
            values.append(value)
    value = float(np.median(values))
    w = workloads.make(args.workload, 64)
    full = workloads.make(args.workload).interior_points if args.points is None else args.points
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * full / value, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f64", "data": "synthetic",
        "config": {"workload": args.workload, "description": w.description,
                   "note": "CPU oracle port of the reference plan interpreter; optimizer update not included"},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


def main() -> None:
    args = parse_args()
    if args.impl == "reference":
        run_reference(args)
        return

    import torch

    import quabla_b200 as qb
    from quabla_b200 import _lib, workloads
    from quabla_b200._plan import nccl_unique_id

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the qb200 backend has no CPU fallback")
    torch.cuda.set_device(local_rank)
    device = f"cuda:{local_rank}"
    if world > 1:
        torch.distributed.init_process_group("nccl", device_id=torch.device(device))

    # Workload: every rank draws the same global point sets and keeps its shard.
    base = workloads.make(args.workload, args.points)
    per_gpu = base.interior_points
    if world > 1:
        big = workloads.make(args.workload, per_gpu * world)
        data = []
        for full_array, local_array in zip(big.data, base.data):
            if full_array.shape[0] == local_array.shape[0] * world:
                n = local_array.shape[0]
                data.append(np.ascontiguousarray(full_array[rank * n:(rank + 1) * n]))
            else:
                data.append(local_array)  # tiny exact sets (two boundary points) are replicated
        data = tuple(data)
    else:
        data = base.data
    w = base
    optimizer = qb.optim.Adam(learning_rate=1e-3)
    batch_argnums = tuple(range(len(data)))
    trainer = qb.optim.Trainer(w.loss, w.params, optimizer, *data, device=device, batch_argnums=batch_argnums)
    plan = trainer._executor.plan
    if world > 1:
        ids = [nccl_unique_id() if rank == 0 else None]
        torch.distributed.broadcast_object_list(ids, src=0)
        plan.attach_comm(ids[0], rank, world, "mean")
    stream = torch.cuda.ExternalStream(plan.query(_lib.Q_STREAM), device=device)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=device)  # larger than the 126 MB L2
    align_token = torch.zeros(1, device=device)

    kernel_ns: list = []  # device time of the interior point set's kernels, one entry per timed step
    allreduce_ns: list = []  # device time of the gradient all-reduce (waits for the other ranks included)

    def barrier():
        if world > 1:
            torch.distributed.barrier()
        torch.cuda.synchronize()

    def timed_steps(step_fn, count: int) -> float:
        """Milliseconds of `count` steps, each bracketed by events on the plan's
        stream; L2 is flushed between steps, outside the timed brackets."""
        starts = [torch.cuda.Event(enable_timing=True) for _ in range(count)]
        stops = [torch.cuda.Event(enable_timing=True) for _ in range(count)]
        for i in range(count):
            flush.fill_(i & 0xFF)
            barrier()  # ranks enter the step together: the bracket times the step, not the ranks' skew
            if world > 1:
                # ... and their streams too: a one-element all-reduce on the plan's stream releases every
                # rank's stream at the same moment, so host jitter after the barrier stays outside the bracket.
                with torch.cuda.stream(stream):
                    torch.distributed.all_reduce(align_token)
            starts[i].record(stream)
            step_fn()
            stops[i].record(stream)
            stops[i].synchronize()
            kernel_ns.append(plan.query(_lib.Q_SET0_NANOSECONDS))
            allreduce_ns.append(plan.query(_lib.Q_ALLREDUCE_NANOSECONDS))
        return sum(a.elapsed_time(b) for a, b in zip(starts, stops))

    def device_step():
        trainer.step()

    pinned = [torch.from_numpy(np.ascontiguousarray(a)).pin_memory() for a in data]
    pinned_np = [p.numpy() for p in pinned]

    def e2e_step():
        trainer.step(*pinned_np)  # host -> device copy of the batch, step, ...
        _ = trainer.value         # ... and the step's loss read back

    for _ in range(max(args.warmup, 3)):
        device_step()
    plan.synchronize()
    barrier()
    try:
        gpu_uuid = str(torch.cuda.get_device_properties(local_rank).uuid)
    except Exception:
        gpu_uuid = None
    sampler = ClockSampler(local_rank, gpu_uuid)
    sampler.start()
    launches0 = plan.query(_lib.Q_KERNEL_LAUNCHES)
    device_ms = timed_steps(device_step, args.steps)
    launches = plan.query(_lib.Q_KERNEL_LAUNCHES) - launches0
    barrier()
    for _ in range(3):
        e2e_step()
    barrier()
    t0 = time.perf_counter()
    e2e_ms = 0.0
    for i in range(args.steps):
        flush.fill_(i & 0xFF)
        barrier()
        t1 = time.perf_counter()
        e2e_step()
        plan.synchronize()
        e2e_ms += 1e3 * (time.perf_counter() - t1)
    clocks = sampler.stop()
    barrier()

    times = torch.tensor([device_ms, e2e_ms], dtype=torch.float64, device=device)
    if world > 1:
        torch.distributed.all_reduce(times, op=torch.distributed.ReduceOp.MAX)
    device_ms, e2e_ms = (float(t) for t in times.cpu())
    total_points = per_gpu * world
    ms_per_step = device_ms / args.steps
    value = total_points / (ms_per_step * 1e-3)
    e2e_value = total_points / (e2e_ms / args.steps * 1e-3)
    h2d = int(sum(a.nbytes for a in data))
    d2h = int(np.dtype(w.dtype).itemsize)

    peaks, peak_kind = measured_peaks()
    dtype_name = "f32" if np.dtype(w.dtype) == np.float32 else "f64"
    # Roofline of the dominant kernel: the kernels of the interior point set (one fused launch on
    # narrow networks), timed live with CUDA events on the plan's stream inside the timed steps.
    kernel_s = float(np.mean(kernel_ns)) * 1e-9
    # Matmul FLOPs one launch EXECUTES: the streams the plan carries (a Laplacian carried as one merged
    # second-order stream is fewer streams than the reference formulation's one per direction).
    interior = plan.spec.sets[0]
    streams = interior.streams
    flops = w.flops_per_point(streams) * per_gpu
    step_flops = flops + sum(w.flops_per_point(s) * n for n, s in w.extra)
    achieved_tflops = flops / kernel_s / 1e12
    if dtype_name == "f32":
        # 3xTF32 on the tensor pipe: TF32 runs at half the bf16 rate, three passes per product.
        # Burst figure for a kernel timed alone in a short step; the sustained one (seconds-long loop under the
        # power cap) when the timed kernels run for tens of milliseconds per step.
        sustained = kernel_s > 0.02 and "bf16_tflops_sustained" in peaks
        peak_tflops = peaks["bf16_tflops_sustained" if sustained else "bf16_tflops"] / 2.0 / 3.0
        peak_note = f"{peak_kind} bf16 {'sustained' if sustained else 'burst'} / 2 (tf32) / 3 (3xTF32 passes)"
    else:
        # Not in the driver-written peaks file: cuBLAS DGEMM 4096^3 (torch.matmul, float64, best of 5,
        # CUDA events) on this pool's B200; the FP64 MMA issue rate (64 FMA/clk/SM) gives the same.
        peak_tflops = 35.0
        peak_note = "cuBLAS DGEMM 4096^3 measured on this pool (35.0 TFLOP/s)"
    engine = plan.query(_lib.Q_ENGINE)
    engine_name = {0: "layerwise", 1: "fused (FP32 pipe)", 2: "fused (tensor cores, 3xTF32 mma)",
                   3: "layerwise (tcgen05 3xTF32 GEMMs)"}[engine]
    kernel_name = {0: "layer-wise kernels of the interior point set",
                   1: "fused_step_kernel (interior point set)",
                   2: "fused_mma_kernel (interior point set)",
                   3: "layer-wise kernels of the interior point set (tcgen05 GEMMs)"}[engine]
    # DRAM traffic of the dominant kernel per launch, from the ncu captures summarised under profiles/
    # (dram__bytes read + write); known for the default workload's fused kernel only.
    traffic = None
    if w.name == "poisson2d" and engine == 2 and per_gpu == 65536 and streams == 4:
        traffic = 114.3e6
    extra_peaks = {}
    if dtype_name == "f32":
        # Also measured on this pool (torch.matmul 8192^3, best of 10): TF32 GEMM 756.5, SGEMM 63.9 TFLOP/s.
        extra_peaks = {"frac_of_tf32_gemm_over_3": achieved_tflops / (756.5 / 3.0),
                       "frac_of_sgemm": achieved_tflops / 63.9}
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": dtype_name, "data": "synthetic",
        "config": {"workload": w.name, "description": w.description, "interior_points_per_gpu": per_gpu,
                   "other_sets": w.extra, "optimizer": "adam lr=1e-3", "parameters": w.parameter_count,
                   "engine": engine_name, "streams": streams, "reference_streams": w.streams,
                   "merged_second_order": interior.merge_weights is not None,
                   "l2": "256 MB written between timed steps, outside the per-step event brackets",
                   "allreduce_us_rank0": float(np.mean(allreduce_ns)) * 1e-3 if world > 1 else 0.0},
        "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "gpu_launches": int(launches),
        "clocks": clocks,
        "roofline": {"bound": "tensor", "achieved": achieved_tflops, "peak": peak_tflops, "unit": "TFLOP/s",
                     "frac": achieved_tflops / peak_tflops, "traffic": traffic, **extra_peaks,
                     "kernel": kernel_name, "kernel_us": kernel_s * 1e6, "flops_per_launch": flops,
                     "step_flops": step_flops, "peak_source": peak_note},
    }
    if rank == 0:
        if world == 1 and not args.no_cpu_baseline:
            cpu_value, sample = cpu_sample(args.workload, args.cpu_seconds, 1)
            line["cpu_baseline"] = {"value": cpu_value, "unit": UNIT, "cores": 1, "kind": "port", "sample": sample}
        print(json.dumps(line))
    if world > 1:
        plan.detach_comm()
        torch.distributed.destroy_process_group()


if __name__ == "__main__":
    main()
