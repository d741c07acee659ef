#!/usr/bin/env python
"""Benchmark of the numba-mlir offload path on B200.

    python bench.py --gpus N --steps K --warmup W [--impl reference]
                    [--workload NAME]

One "step" is one pass of the hot path over one batch of synthetic input.  The
headline workload is the Black-Scholes fused ufunc chain over 2^24 float32
options per GPU (20 algorithmic bytes per option); the metric is effective HBM
GB/s = algorithmic bytes / device time, whole job over all N GPUs.  Inputs and
outputs (320 MB per GPU) exceed the 126 MB L2, so no flush is needed between
iterations.  Rank 0 prints ONE JSON line.

`--impl reference` times the CPU implementation of the same workload (upstream
Numba njit(parallel=True), which is what the reference's njit is with its MLIR
pipeline off) on the host cores.
"""

import argparse
import json
import os
import statistics
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "effective_hbm_bandwidth"
UNIT = "GB/s"
NOMINAL_HBM_GBS = 8000.0


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return json.load(f).get("hbm_gbs"), "measured"
    return 6650.0, "fallback"


# dram__bytes_read.sum + dram__bytes_write.sum per launch from the ncu capture
# summarised under profiles/ (None until captured).
NCU_TRAFFIC_BYTES = {"black_scholes": None}


# ------------------------------------------------------------- workloads ----
class BlackScholes:
    """Config: N = 2^24 float32 options per GPU; spot, strike ~ U[10,50],
    expiry ~ U[1,2], rate 0.1, volatility 0.2; outputs call and put."""

    name = "black_scholes_f32_n2^24"
    key = "black_scholes"
    n = 1 << 24
    bytes_per_step = 20 * n  # 3 float32 reads + 2 float32 writes per option
    units_per_step = n
    dtype = "f32"

    def host_inputs(self, seed):
        rng = np.random.default_rng(seed)
        f32 = np.float32
        return (
            rng.uniform(10, 50, self.n).astype(f32),
            rng.uniform(10, 50, self.n).astype(f32),
            rng.uniform(1, 2, self.n).astype(f32),
            f32(0.1),
            f32(0.2),
        )

    def setup_device(self, queue, seed):
        import numba_mlir_b200 as nm

        price, strike, t, self.rate, self.vol = self.host_inputs(seed)
        self.queue = queue
        # pinned staging for the end-to-end leg
        self.h_in = [nm.pinned_empty(self.n, np.float32, queue) for _ in range(3)]
        for dst, src in zip(self.h_in, (price, strike, t)):
            dst[:] = src
        self.h_out = [nm.pinned_empty(self.n, np.float32, queue) for _ in range(2)]
        self.d_in = [nm.from_host(x, queue) for x in (price, strike, t)]
        self.d_out = [nm.empty(self.n, np.float32, queue) for _ in range(2)]
        self.h2d_bytes = 3 * 4 * self.n
        self.d2h_bytes = 2 * 4 * self.n

    def step_device(self):
        from numba_mlir_b200 import builtin_ops

        builtin_ops.black_scholes_f32(*self.d_in, self.rate, self.vol, *self.d_out)
        return 1  # kernels launched

    def step_e2e(self):
        """Host buffers in, host buffers out, through the public API."""
        for d, h in zip(self.d_in, self.h_in):
            d.copy_from_host(h, wait=False)
        launches = self.step_device()
        for d, h in zip(self.d_out, self.h_out):
            d.copy_to_host(h, wait=False)
        self.queue.synchronize()
        return launches

    def check(self):
        """Cheap sanity check of the last result (not the parity test)."""
        call = self.d_out[0][:1024].copy_to_host()
        assert np.isfinite(call).all()

    # CPU side ---------------------------------------------------------------
    def cpu_setup(self, seed, fraction=1.0):
        from oracle import configs as O

        m = max(1, int(self.n * fraction))
        price, strike, t, rate, vol = self.host_inputs(seed)
        self.cpu_args = (price[:m].copy(), strike[:m].copy(), t[:m].copy(), rate, vol)
        self.cpu_out = (np.zeros(m, np.float32), np.zeros(m, np.float32))
        self.cpu_units = m
        self.cpu_bytes = 20 * m
        self._cpu_fn = O.black_scholes
        self._cpu_fn(*self.cpu_args, *self.cpu_out)  # compile, excluded

    def cpu_step(self):
        self._cpu_fn(*self.cpu_args, *self.cpu_out)


WORKLOADS = {"black_scholes": BlackScholes}


# ---------------------------------------------------------------- clocks ----
class ClockSampler:
    """Samples SM clock and throttle reasons through NVML (read-only) while the
    timed regions run."""

    def __init__(self, device_index):
        self.samples = []
        self.reasons = set()
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None
        self._active = threading.Event()
        try:
            import pynvml

            pynvml.nvmlInit()
            self.nv = pynvml
            visible = os.environ.get("CUDA_VISIBLE_DEVICES")
            idx = device_index
            if visible:
                ids = [v for v in visible.split(",") if v.strip()]
                if device_index < len(ids) and ids[device_index].strip().isdigit():
                    idx = int(ids[device_index])
            self.handle = pynvml.nvmlDeviceGetHandleByIndex(idx)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _loop(self):
        nv = self.nv
        names = {
            "hw_slowdown": getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8),
            "hw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40),
            "sw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20),
            "sw_power_cap": getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4),
        }
        while not self._stop.is_set():
            if self._active.is_set():
                try:
                    mhz = nv.nvmlDeviceGetClockInfo(self.handle, nv.NVML_CLOCK_SM)
                    self.samples.append(mhz)
                    try:
                        mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self.handle)
                    except Exception:
                        mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.handle)
                    for k, bit in names.items():
                        if mask & bit:
                            self.reasons.add(k)
                except Exception:
                    pass
            time.sleep(0.01)

    def start(self):
        if self.nv is not None:
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()

    def active(self, on):
        (self._active.set if on else self._active.clear)()

    def stop(self):
        self._stop.set()
        if self._thread:
            self._thread.join(timeout=2)
        return {
            "sm_mhz": statistics.median(self.samples) if self.samples else None,
            "sm_max_mhz": self.max_mhz,
            "reasons": sorted(self.reasons),
            "samples": len(self.samples),
        }


# ------------------------------------------------------------ CPU timing ----
def time_cpu(workload, seed, budget_s, max_steps):
    """Best-of timing of the CPU oracle on the full workload within a budget."""
    import numba

    workload.cpu_setup(seed)
    times = []
    t_end = time.perf_counter() + budget_s
    while len(times) < max_steps and (len(times) < 3 or time.perf_counter() < t_end):
        t0 = time.perf_counter()
        workload.cpu_step()
        times.append(time.perf_counter() - t0)
    return times, numba.get_num_threads()


def run_reference(args):
    """CPU arm: the oracle on the host cores, rank 0 only.  Each step is a
    bounded sample of the workload, sized so the whole run stays near two
    minutes whatever --steps is."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    w = WORKLOADS[args.workload]()
    import numba

    steps = args.steps if args.steps is not None else 20
    w.cpu_setup(0)
    t0 = time.perf_counter()
    w.cpu_step()
    t_full = time.perf_counter() - t0
    fraction = 1.0
    while fraction > 1 / 1024 and (steps + args.warmup) * t_full * fraction > 120.0:
        fraction /= 2
    if fraction < 1.0:
        w.cpu_setup(0, fraction)
    for _ in range(max(args.warmup, 1)):
        w.cpu_step()
    t0 = time.perf_counter()
    for _ in range(steps):
        w.cpu_step()
    dt = (time.perf_counter() - t0) / max(steps, 1)
    value = w.cpu_bytes / dt / 1e9
    line = {
        "impl": "reference",
        "metric": METRIC,
        "value": value,
        "unit": UNIT,
        "n_gpus": args.gpus,
        "steps": steps,
        "warmup": args.warmup,
        "ms_per_step": dt * 1e3,
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": None,
        "dtype": w.dtype,
        "data": "synthetic",
        "config": {"workload": w.name, "elements_per_step": w.cpu_units},
        "elements_per_s": w.cpu_units / dt,
        "cpu_baseline": {
            "value": value,
            "unit": UNIT,
            "cores": numba.get_num_threads(),
            "kind": "port",
            "sample": f"{w.cpu_units} of {w.units_per_step} elements per step; upstream "
            f"numba.njit(parallel=True), threading layer {numba.threading_layer()}",
        },
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------- GPU timing ---
def run_gpu(args):
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))

    import torch

    from numba_mlir_b200 import build as _build

    if rank == 0:
        _build.build()
    from numba_mlir_b200 import runtime

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: there is no CPU fallback")
    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
        dist.barrier()
        if rank != 0:
            _build.build()  # no-op: picks up rank 0's library

    queue = runtime.get_queue(f"cuda:{local_rank}")
    w = WORKLOADS[args.workload]()
    w.setup_device(queue, seed=rank)

    def barrier():
        queue.synchronize()
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
            torch.cuda.synchronize()

    sampler = ClockSampler(local_rank)
    sampler.start()

    # -- device-resident leg ---------------------------------------------------
    for _ in range(max(args.warmup, 3)):
        w.step_device()
    barrier()
    sampler.active(True)
    launches = 0
    count0 = runtime.launch_count()
    e0 = queue.record()
    for _ in range(args.steps):
        launches += w.step_device()
    e1 = queue.record()
    queue.wait(e1)
    barrier()
    sampler.active(False)
    dev_ms = queue.elapsed_ms(e0, e1)
    counted = runtime.launch_count() - count0
    queue.destroy_event(e0)
    queue.destroy_event(e1)
    w.check()

    # -- end-to-end leg (host buffers, copies inside the timed region) ---------
    e2e_steps = max(1, min(args.steps, 50))
    for _ in range(2):
        w.step_e2e()
    barrier()
    sampler.active(True)
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        w.step_e2e()
    barrier()
    e2e_s = time.perf_counter() - t0
    sampler.active(False)
    clocks = sampler.stop()

    if dist is not None:
        t = torch.tensor([dev_ms, e2e_s], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dev_ms, e2e_s = t.tolist()

    if rank == 0:
        ms_per_step = dev_ms / args.steps
        total_bytes = w.bytes_per_step * world
        value = total_bytes / (ms_per_step * 1e-3) / 1e9
        e2e_value = total_bytes / (e2e_s / e2e_steps) / 1e9
        peak, peak_kind = measured_peaks()
        achieved = w.bytes_per_step / (ms_per_step * 1e-3) / 1e9  # per GPU, per launch
        line = {
            "metric": METRIC,
            "value": value,
            "unit": UNIT,
            "n_gpus": world,
            "steps": args.steps,
            "warmup": max(args.warmup, 3),
            "ms_per_step": ms_per_step,
            "higher_is_better": True,
            "scaling": "weak",
            "vs_baseline": None,
            "dtype": w.dtype,
            "data": "synthetic",
            "config": {
                "workload": w.name,
                "elements_per_step_per_gpu": w.units_per_step,
                "sharding": "independent contiguous ranges per GPU, no collective",
                "l2": "inputs+outputs (320 MB/GPU) exceed the 126 MB L2; no flush",
            },
            "elements_per_s": w.units_per_step * world / (ms_per_step * 1e-3),
            "frac_of_nominal_8TBs": achieved / NOMINAL_HBM_GBS,
            "roofline": {
                "bound": "hbm",
                "achieved": achieved,
                "peak": peak,
                "peak_kind": peak_kind,
                "unit": "GB/s",
                "frac": achieved / peak,
                "traffic": NCU_TRAFFIC_BYTES.get(w.key),
            },
            "e2e": {
                "value": e2e_value,
                "unit": UNIT,
                "h2d_bytes_per_step": w.h2d_bytes,
                "d2h_bytes_per_step": w.d2h_bytes,
                "steps": e2e_steps,
            },
            "gpu_launches": counted,
            "clocks": clocks,
        }
        if world == 1 and not args.no_cpu:
            times, threads = time_cpu(w, 0, budget_s=12.0, max_steps=100)
            best = min(times)
            line["cpu_baseline"] = {
                "value": w.cpu_bytes / best / 1e9,
                "unit": UNIT,
                "cores": threads,
                "kind": "port",
                "sample": f"the full workload ({w.cpu_units} elements) per step, best of "
                f"{len(times)}; upstream numba.njit(parallel=True)",
                "ms_per_step": best * 1e3,
            }
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=None)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="black_scholes", choices=sorted(WORKLOADS))
    ap.add_argument("--no-cpu", action="store_true", help="skip the cpu_baseline leg")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        if args.steps is None:
            args.steps = 2000
        run_gpu(args)


if __name__ == "__main__":
    main()
