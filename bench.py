"""Benchmark of the PINN training step: collocation points per second per full
Adam step (forward, reverse pass, gradient all-reduce, optimizer update).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

Launched under `python -m torch.distributed.run` for N > 1 (one rank per GPU).
Prints ONE JSON line on rank 0.

The default workload is the 3-D heat equation (float32, tanh MLP 4-256x6-1,
1,048,576 collocation points in total).  With N GPUs the points are cut into N
contiguous equal axis-0 shards in rank order, one per rank (strong scaling:
the total is fixed), and the step ends with one all-reduce of the flat
[loss, gradients] buffer; parameters and Adam moments are replicated.  Inputs
are seeded synthetic points and Xavier-normal weights.

  value    device-resident step: points and parameters already in HBM;
  e2e      the same step through `optim.Trainer.step(batch)` with the batch
           copied from pinned host memory every step and the step's loss read
           back, both inside the timed region;
  details.others   the other workloads (2-D Poisson, Burgers, beam), a few
           steps each after the timed region, sharded the same way.

With N > 1 the run first checks one step of the same workload on a few
thousand points against the CPU oracle on the full batch (rank 0; the process
exits non-zero when the 1e-5 / 1e-10 gate fails) and, after the timed loop,
that every rank holds bit-identical parameters.
"""

from __future__ import annotations

import argparse
import hashlib
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
L2_BYTES = 126 << 20
PARITY_POINTS = 2048  # total interior points of the multi-GPU parity step
PARITY_TOLERANCE = {"f32": 1e-5, "f64": 1e-10}


def parse_args():
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=20)
    parser.add_argument("--warmup", type=int, default=5)
    parser.add_argument("--impl", default="ours", choices=["ours", "reference"])
    parser.add_argument("--workload", default="heat3d")
    parser.add_argument("--points", type=int, default=None,
                        help="interior points in total over all GPUs (default: the workload's)")
    parser.add_argument("--cpu-seconds", type=float, default=12.0, help="target CPU time of the bounded CPU sample")
    parser.add_argument("--no-cpu-baseline", action="store_true")
    parser.add_argument("--no-others", action="store_true", help="skip the other workloads after the timed region")
    parser.add_argument("--no-parity", action="store_true", help="skip the multi-GPU parity step")
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


def workload_config(name: str, total_points: int | None, world: int) -> dict:
    """The `config` object, identical in both arms: what is computed, on how many points, cut how."""
    from quabla_b200 import workloads

    w = workloads.make(name, total_points if total_points is not None else None)
    return {"workload": w.name, "description": w.description, "interior_points": w.interior_points,
            "other_sets": [list(e) for e in w.extra], "parameters": w.parameter_count, "optimizer": "adam lr=1e-3",
            "sharding": f"{world} contiguous equal axis-0 shard(s) of every point set, parameters replicated"}


def cpu_sample(workload_name: str, seconds: float, threads: int, total_points: int | None = None):
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
    full = workloads.make(workload_name, total_points).interior_points
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

    threads = contracted.max_threads()
    per_step = max(1.0, min(8.0, 120.0 / max(1, args.steps + args.warmup)))
    values = []
    sample = ""
    for step in range(args.warmup + args.steps):
        value, sample = cpu_sample(args.workload, per_step, threads, args.points)
        if step >= args.warmup:
            values.append(value)
    value = float(np.median(values))
    config = workload_config(args.workload, args.points, args.gpus)
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * config["interior_points"] / value,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f64", "data": "synthetic",
        "config": config,
        "details": {"note": "CPU oracle port of the reference plan interpreter (contracted form, float64), every "
                            "host thread; the optimizer update is not included; each step is a bounded sample of "
                            "the workload"},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


class Rig:
    """One rank's view of a run: device, process group, and the helpers every measured
    workload uses (sharding, communicator attachment, event-bracketed loops)."""

    def __init__(self, args) -> None:
        import torch

        self.torch = torch
        self.rank = int(os.environ.get("RANK", "0"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        if self.world != args.gpus:
            raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={self.world}: launch with torch.distributed.run")
        if not torch.cuda.is_available():
            raise SystemExit("bench.py needs a CUDA device: the qb200 backend has no CPU fallback")
        torch.cuda.set_device(self.local_rank)
        self.device = f"cuda:{self.local_rank}"
        if self.world > 1:
            torch.distributed.init_process_group("nccl", device_id=torch.device(self.device))
        self.flush = torch.empty(256 << 20, dtype=torch.uint8, device=self.device)  # larger than the 126 MB L2
        self.token = torch.zeros(1, device=self.device)

    def barrier(self) -> None:
        if self.world > 1:
            self.torch.distributed.barrier()
        self.torch.cuda.synchronize()

    def shard(self, w):
        """This rank's rows of every point set: contiguous equal axis-0 shards in rank order
        (python/quabla/distributed.py:101-106); sets too small to cut (two boundary points) are replicated,
        which a mean over ranks leaves unchanged."""
        if self.world == 1:
            return w.data
        out = []
        for a in w.data:
            rows = a.shape[0]
            if rows >= 64 and rows % self.world == 0:
                n = rows // self.world
                out.append(np.ascontiguousarray(a[self.rank * n:(self.rank + 1) * n]))
            else:
                out.append(a)
        return tuple(out)

    def trainer(self, w, data):
        import quabla_b200 as qb
        from quabla_b200._plan import nccl_unique_id

        optimizer = qb.optim.Adam(learning_rate=1e-3)
        trainer = qb.optim.Trainer(w.loss, w.params, optimizer, *data, device=self.device,
                                   batch_argnums=tuple(range(len(data))))
        plan = trainer._executor.plan
        if self.world > 1:
            ids = [nccl_unique_id() if self.rank == 0 else None]
            self.torch.distributed.broadcast_object_list(ids, src=0)
            plan.attach_comm(ids[0], self.rank, self.world, "mean")
        return trainer, plan

    def max_over_ranks(self, values):
        t = self.torch.tensor(values, dtype=self.torch.float64, device=self.device)
        if self.world > 1:
            self.torch.distributed.all_reduce(t, op=self.torch.distributed.ReduceOp.MAX)
        return [float(v) for v in t.cpu()]

    def timed_loop(self, plan, step_fn, count: int, flush_between: bool) -> float:
        """Device milliseconds of `count` steps on the plan's stream.  Working sets larger than L2: ONE
        bracket around all steps, back to back as a training loop runs them (rank skew and launch gaps
        included).  Otherwise per-step brackets with 256 MB written between steps to flush L2, ranks
        aligned before each step."""
        from quabla_b200 import _lib

        torch = self.torch
        stream = torch.cuda.ExternalStream(plan.query(_lib.Q_STREAM), device=self.device)
        if not flush_between:
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            self.barrier()
            start.record(stream)
            for _ in range(count):
                step_fn()
            stop.record(stream)
            stop.synchronize()
            self.barrier()
            return start.elapsed_time(stop)
        starts = [torch.cuda.Event(enable_timing=True) for _ in range(count)]
        stops = [torch.cuda.Event(enable_timing=True) for _ in range(count)]
        for i in range(count):
            self.flush.fill_(i & 0xFF)
            self.barrier()
            if self.world > 1:
                # A one-element all-reduce on the plan's stream releases every rank's stream together.
                with torch.cuda.stream(stream):
                    torch.distributed.all_reduce(self.token)
            starts[i].record(stream)
            step_fn()
            stops[i].record(stream)
            stops[i].synchronize()
        self.barrier()
        return sum(a.elapsed_time(b) for a, b in zip(starts, stops))


ENGINES = {0: "layer-wise (FP64 tensor-core / SIMT GEMMs)", 1: "fused (FP32/FP64 pipe)",
           2: "fused (tensor cores, 3xTF32 mma)", 3: "layer-wise (tcgen05 split-float32 GEMMs)"}


def measure(rig: Rig, name: str, total_points: int | None, steps: int, warmup: int, peaks: dict, live: dict,
            with_e2e: bool) -> dict:
    """One workload on this rig: device-resident steps, optionally the end-to-end loop, and the
    dominant kernel's device time from the last timed step."""
    from quabla_b200 import _lib, workloads

    torch = rig.torch
    w = workloads.make(name, total_points)
    data = rig.shard(w)
    trainer, plan = rig.trainer(w, data)
    plan.set_option(_lib.OPT_KERNEL_TIMERS, 1)
    dtype_name = "f32" if np.dtype(w.dtype) == np.float32 else "f64"
    scratch = plan.query(_lib.Q_SCRATCH_BYTES)
    flush_between = scratch + sum(a.nbytes for a in data) <= 2 * L2_BYTES
    for _ in range(max(warmup, 3)):
        trainer.step()
    plan.synchronize()
    launches0 = plan.query(_lib.Q_KERNEL_LAUNCHES)
    device_ms = rig.timed_loop(plan, trainer.step, steps, flush_between)
    launches = plan.query(_lib.Q_KERNEL_LAUNCHES) - launches0
    engine = plan.query(_lib.Q_ENGINE)
    interior = plan.spec.sets[0]
    local_points = interior.n_points
    # Dominant kernel, from the last timed step: the layer GEMM launches of the layer-wise engines
    # (an event pair around each), the interior set's one fused launch on the fused engines.
    lanes = plan.query(_lib.Q_LANES)
    if engine in (0, 3):
        if lanes > 1:
            # Chunks overlap on two streams in the timed loop, so an event pair there spans more than its kernel:
            # time the GEMM launches in two more steps with every chunk on one stream (outside the timed loop).
            plan.set_option(_lib.OPT_SINGLE_LANE, 1)
            for _ in range(2):
                trainer.step()
            plan.synchronize()
        gemm_ns = plan.query(_lib.Q_GEMM_NANOSECONDS)
        gemm_launches = max(1, plan.query(_lib.Q_GEMM_LAUNCHES))
        gemm_flops = float(plan.query(_lib.Q_GEMM_FLOPS))
        # Tensor-pipe work of the same launches at the bf16 rate: 6 passes per FLOP for a product made of three
        # tf32 instructions, 4 where the two correction products are bf16 instructions (0 off the tensor pipe).
        pipe_flops = float(plan.query(_lib.Q_GEMM_PIPE_FLOPS))
        kernel = {"name": "tc_tma_gemm_kernel (tcgen05: tf32 product + two correction products)" if engine == 3 else
                  "dmma_gemm_kernel (FP64 MMA) / gemm_kernel" if dtype_name == "f64" else "gemm_kernel",
                  "launches_per_step": int(gemm_launches), "us_per_launch": gemm_ns * 1e-3 / gemm_launches,
                  "flops_per_launch": gemm_flops / gemm_launches, "us_per_step": gemm_ns * 1e-3,
                  "bf16_rate_passes_per_flop": pipe_flops / gemm_flops if gemm_flops else 0.0}
        achieved = gemm_flops / max(gemm_ns, 1) * 1e-3  # FLOP / ns = GFLOP/s; / 1e3 = TFLOP/s
        if lanes > 1:
            kernel["timed"] = "two extra steps with the chunks serialised on one stream"
            plan.set_option(_lib.OPT_SINGLE_LANE, 0)
    else:
        set0_ns = plan.query(_lib.Q_SET0_NANOSECONDS)
        flops = w.flops_per_point(interior.streams) * local_points
        kernel = {"name": "fused_mma_kernel" if engine == 2 else "fused_step_kernel", "launches_per_step": 1,
                  "us_per_launch": set0_ns * 1e-3, "flops_per_launch": flops, "us_per_step": set0_ns * 1e-3,
                  "bf16_rate_passes_per_flop": 6.0 if dtype_name == "f32" else 0.0}
        achieved = flops / max(set0_ns, 1) * 1e-3
    allreduce_us = plan.query(_lib.Q_ALLREDUCE_NANOSECONDS) * 1e-3 if rig.world > 1 else 0.0

    e2e_ms = None
    h2d = int(sum(a.nbytes for a in data))
    if with_e2e:
        pinned = [torch.from_numpy(np.ascontiguousarray(a)).pin_memory() for a in data]
        pinned_np = [p.numpy() for p in pinned]

        def e2e_step():
            trainer.step(*pinned_np)  # host -> device copy of this rank's batch, the step, ...
            _ = trainer.value         # ... and the step's loss read back

        for _ in range(3):
            e2e_step()
        rig.barrier()
        t0 = time.perf_counter()
        for i in range(steps):
            if flush_between:
                rig.flush.fill_(i & 0xFF)
                torch.cuda.synchronize()
            e2e_step()
        plan.synchronize()
        e2e_ms = 1e3 * (time.perf_counter() - t0)
        rig.barrier()

    # Every rank must hold the same parameters after the same number of updates.
    digest = hashlib.sha256()
    for index in range(len(plan.spec.parameters)):
        digest.update(plan.read_parameter(index).tobytes())
    word = int.from_bytes(digest.digest()[:6], "little")  # 48 bits: exact in float64
    lo_hi = rig.max_over_ranks([float(word), -float(word)])
    identical = lo_hi[0] == -lo_hi[1]

    device_ms, = rig.max_over_ranks([device_ms])
    total_points_run = w.interior_points
    ms_per_step = device_ms / steps
    streams = interior.streams
    step_flops = (w.flops_per_point(streams) * w.interior_points
                  + sum(w.flops_per_point(s) * n for n, s in w.extra))
    if dtype_name == "f32":
        # Split float32 on the tensor pipe: a tf32 instruction runs at half the bf16 rate, so three tf32 products
        # cost 6 bf16-rate passes per FLOP and a tf32 product with two bf16 correction products costs 4; the
        # denominator is the bf16 rate over the passes the timed launches actually execute.  The burst figure
        # for kernels timed alone in a short step, the sustained one (seconds-long loop under the power cap)
        # when the timed kernels keep the GPU busy for tens of milliseconds per step.
        sustained = kernel["us_per_step"] > 2e4 and "bf16_tflops_sustained" in peaks
        passes = kernel["bf16_rate_passes_per_flop"] or 6.0
        peak = peaks["bf16_tflops_sustained" if sustained else "bf16_tflops"] / passes
        peak_source = f"bf16 {'sustained' if sustained else 'burst'} / {passes:.2f} (tensor-pipe passes per FLOP at the bf16 rate)"
    else:
        peak = live.get("dgemm_tflops")
        peak_source = "torch.matmul float64 4096^3, best of 5, timed at start-up of this run"
    out = {
        "workload": w.name, "dtype": dtype_name, "interior_points": total_points_run, "ms_per_step": ms_per_step,
        "points_per_s": total_points_run / (ms_per_step * 1e-3), "engine": ENGINES[engine], "streams": streams,
        "reference_streams": w.streams, "merged_second_order": interior.merge_weights is not None,
        "step_tflops": step_flops / (ms_per_step * 1e-3) / 1e12 / 1.0,
        "kernel": kernel, "kernel_tflops": achieved, "peak_tflops": peak, "peak_source": peak_source,
        "kernel_frac": achieved / peak if peak else None,
        "step_frac": step_flops / (ms_per_step * 1e-3) / 1e12 / rig.world / peak if peak else None,
        "gpu_launches": int(launches), "allreduce_us_rank0": allreduce_us, "replicas_identical": bool(identical),
        "lanes": int(lanes),
        "l2": ("256 MB written between timed steps, per-step event brackets" if flush_between else
               f"one event bracket around {steps} back-to-back steps; per-rank working set "
               f"{(scratch + h2d) / 2**30:.1f} GiB > L2"),
        "h2d_bytes_per_step": h2d * rig.world, "d2h_bytes_per_step": int(np.dtype(w.dtype).itemsize) * rig.world,
    }
    if e2e_ms is not None:
        e2e_ms, = rig.max_over_ranks([e2e_ms])
        out["e2e_points_per_s"] = total_points_run / (e2e_ms / steps * 1e-3)
    if rig.world > 1:
        plan.detach_comm()
    plan.close()
    return out


def parity_step(rig: Rig, name: str) -> dict:
    """One value-and-gradient step of `name` on PARITY_POINTS points cut over the ranks; rank 0 compares
    the all-reduced [loss, gradients] with the CPU oracle on the full batch (mean of shard means, gradients
    summed in shard order: crates/quabla-core/src/tensor_ir.rs:11622-11724)."""
    from oracle import contracted
    from quabla_b200 import workloads
    from quabla_b200._transforms import CompiledLoss

    w = workloads.make(name, PARITY_POINTS)
    # The timed step's tcgen05 GEMMs run the scheme the library picks for large launches (bfloat16 correction
    # products); a launch of this size would get the other one, so the parity step asks for the timed one.
    forced = "QB200_TC_COR" not in os.environ
    if forced:
        os.environ["QB200_TC_COR"] = "bf16"
    try:
        trainer, plan = rig.trainer(w, rig.shard(w))
        plan.execute()
        outputs = plan.outputs()
    finally:
        if forced:
            del os.environ["QB200_TC_COR"]
    dtype_name = "f32" if np.dtype(w.dtype) == np.float32 else "f64"
    tolerance = PARITY_TOLERANCE[dtype_name]
    worst = 0.0
    if rig.rank == 0:
        args = (w.params, *w.data)
        full = CompiledLoss(w.loss, args, (0,), 0, build_plan=False)
        expected_loss, expected_grads = contracted.value_and_grad(full.spec, full.named_inputs(args),
                                                                  threads=contracted.max_threads())
        worst = abs(float(outputs[0]) - expected_loss) / max(abs(expected_loss), 1e-300)
        for got, expected in zip(outputs[1:], expected_grads):
            scale = max(float(np.max(np.abs(expected))), 1e-300)
            worst = max(worst, float(np.max(np.abs(got.reshape(expected.shape).astype(np.float64) - expected))) / scale)
    worst, = rig.max_over_ranks([worst])
    if rig.world > 1:
        plan.detach_comm()
    plan.close()
    return {"points": w.interior_points, "max_rel_err": worst, "tol": tolerance, "passed": bool(worst <= tolerance)}


def live_peaks(rig: Rig) -> dict:
    """Library GEMM rates of this GPU, timed at start-up outside every timed region (torch.matmul, CUDA
    events, best of 5): the denominators of the float64 fractions and a cross-check of the float32 one."""
    torch = rig.torch
    out = {}
    for key, dtype, n, tf32 in (("dgemm_tflops", torch.float64, 4096, False), ("tf32_gemm_tflops", torch.float32, 8192, True)):
        previous = torch.backends.cuda.matmul.allow_tf32
        torch.backends.cuda.matmul.allow_tf32 = tf32
        try:
            a = torch.randn(n, n, dtype=dtype, device=rig.device)
            b = torch.randn(n, n, dtype=dtype, device=rig.device)
            torch.matmul(a, b)
            best = float("inf")
            for _ in range(5):
                start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                start.record()
                torch.matmul(a, b)
                stop.record()
                stop.synchronize()
                best = min(best, start.elapsed_time(stop))
            out[key] = 2.0 * n**3 / (best * 1e-3) / 1e12
            del a, b
        finally:
            torch.backends.cuda.matmul.allow_tf32 = previous
    torch.cuda.empty_cache()
    return out


# DRAM bytes (read + write) per row of one forward/data-gradient launch of tc_tma_gemm_kernel at width 256, from
# the ncu capture summarised in profiles/tc_tma_gemm_kernel_heat3d.md (2.50-2.54 TB/s x 299-305 us = 760 MB over
# the 393,216 rows of a launch; the algorithmic bytes are 2,048 per row: one row of A read, one row of C written).
TC_GEMM_DRAM_BYTES_PER_ROW = 760e6 / 393216


def main() -> None:
    args = parse_args()
    if args.impl == "reference":
        run_reference(args)
        return

    rig = Rig(args)
    torch = rig.torch
    peaks, peak_kind = measured_peaks()
    live = live_peaks(rig)

    parity = None
    if rig.world > 1 and not args.no_parity:
        parity = parity_step(rig, args.workload)
        if not parity["passed"]:
            if rig.rank == 0:
                print(json.dumps({"error": "multi-GPU parity failed", "parity": parity}))
            torch.distributed.destroy_process_group()
            raise SystemExit(3)

    try:
        gpu_uuid = str(torch.cuda.get_device_properties(rig.local_rank).uuid)
    except Exception:
        gpu_uuid = None
    sampler = ClockSampler(rig.local_rank, gpu_uuid)
    sampler.start()
    main_result = measure(rig, args.workload, args.points, args.steps, args.warmup, peaks, live, with_e2e=True)
    clocks = sampler.stop()
    if not main_result["replicas_identical"]:
        if rig.rank == 0:
            print(json.dumps({"error": "replicas diverged", "result": main_result}))
        raise SystemExit(4)

    others = {}
    if not args.no_others and args.points is None:
        for name in ("poisson2d", "burgers", "beam"):
            if name == args.workload:
                continue
            r = measure(rig, name, None, 5, 3, peaks, live, with_e2e=False)
            others[name] = {k: r[k] for k in ("dtype", "interior_points", "ms_per_step", "points_per_s", "engine",
                                              "streams", "step_tflops", "kernel", "kernel_tflops", "peak_tflops",
                                              "kernel_frac", "replicas_identical", "allreduce_us_rank0", "lanes")}

    kernel = main_result["kernel"]
    traffic = None
    if main_result["engine"] == ENGINES[3] and args.workload == "heat3d":
        rows = kernel["flops_per_launch"] / (2.0 * 256 * 256)
        traffic = TC_GEMM_DRAM_BYTES_PER_ROW * rows
    line = {
        "metric": METRIC, "value": main_result["points_per_s"], "unit": UNIT, "n_gpus": rig.world,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": main_result["ms_per_step"],
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": main_result["dtype"],
        "data": "synthetic",
        "config": workload_config(args.workload, args.points, rig.world),
        "details": {"engine": main_result["engine"], "streams": main_result["streams"],
                    "reference_streams": main_result["reference_streams"],
                    "merged_second_order": main_result["merged_second_order"], "l2": main_result["l2"],
                    "allreduce_us_rank0": main_result["allreduce_us_rank0"],
                    "step_tflops_all_gpus": main_result["step_tflops"], "step_frac_per_gpu": main_result["step_frac"],
                    "parity": None if parity is None else {**parity, "replicas_identical": main_result["replicas_identical"]},
                    "replicas_identical": main_result["replicas_identical"],
                    "library_gemm_tflops_this_run": live, "others": others},
        "e2e": {"value": main_result["e2e_points_per_s"], "unit": UNIT,
                "h2d_bytes_per_step": main_result["h2d_bytes_per_step"],
                "d2h_bytes_per_step": main_result["d2h_bytes_per_step"]},
        "gpu_launches": main_result["gpu_launches"],
        "clocks": clocks,
        "roofline": {"bound": "tensor", "achieved": main_result["kernel_tflops"], "peak": main_result["peak_tflops"],
                     "unit": "TFLOP/s", "frac": main_result["kernel_frac"], "traffic": traffic,
                     "kernel": kernel["name"], "launches_per_step": kernel["launches_per_step"],
                     "kernel_us": kernel["us_per_launch"], "flops_per_launch": kernel["flops_per_launch"],
                     "kernel_us_per_step": kernel["us_per_step"],
                     "peak_source": f"{peak_kind}: {main_result['peak_source']}",
                     # the fraction against the plain 3xTF32 denominator (6 passes per FLOP), comparable across schemes
                     "frac_at_six_passes": (main_result["kernel_tflops"] * 6.0 / (main_result["peak_tflops"] * kernel["bf16_rate_passes_per_flop"])
                                            if main_result["dtype"] == "f32" and kernel["bf16_rate_passes_per_flop"] else None),
                     # the same fraction against the library's TF32 GEMM timed in this run (tf32 = 2 bf16-rate passes)
                     "frac_of_library_tf32_gemm": (main_result["kernel_tflops"] * kernel["bf16_rate_passes_per_flop"] / 2.0
                                                   / live["tf32_gemm_tflops"] if main_result["dtype"] == "f32" else None)},
    }
    if rig.rank == 0:
        if rig.world == 1 and not args.no_cpu_baseline:
            cpu_value, sample = cpu_sample(args.workload, args.cpu_seconds, 1, args.points)
            line["cpu_baseline"] = {"value": cpu_value, "unit": UNIT, "cores": 1, "kind": "port", "sample": sample}
        print(json.dumps(line))
    if rig.world > 1:
        torch.distributed.destroy_process_group()


if __name__ == "__main__":
    main()
