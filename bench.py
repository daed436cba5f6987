#!/usr/bin/env python
"""Benchmark of the compiled-graph hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c1|c2|c2g|c3|c3b|c4|c5] [--impl reference]

One step = one pass of a `torch.compile(fn, backend='gcu')` graph over one batch of seeded
synthetic input.  Default workload: c2, `mean(relu(x*w + b), dim=-1)` with x bf16 [16384, 4096]
-- the configuration the samples/s metric is quoted on.  With N > 1 (launched under
torch.distributed.run, one process per GPU) every rank runs the same graph on its own batch:
rows are independent, so the path shards with no collective (weak scaling).

Prints ONE JSON line on rank 0:
  value     samples/s over all ranks, inputs resident in HBM, plan replayed from a CUDA graph
  e2e       the same metric through the public API with HOST tensors: pinned host -> device copy
            of the step's inputs, kernel(s), device -> host read of the result, every step
  roofline  the dominant kernel's achieved HBM GB/s (or TFLOP/s) against the measured peak
  cpu_baseline  the reference's executed path (PyTorch eager on the host cores) on the same batch
`--impl reference` times only that CPU path and prints it with "impl": "reference".
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

L2_BYTES = 126 * 1024 * 1024
POOL_BYTES_MIN = 4 * L2_BYTES          # rotating input pool is at least this large
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


# ---------------------------------------------------------------- workloads
class Workload:
    """name, graph, per-rank inputs, algorithmic bytes/flops of the dominant kernel."""

    def __init__(self, key):
        from examples import workloads as rp

        self.key = key
        self.rp = rp
        self.module = None
        if key == "c1":
            self.name = "c1 mul_add a*b+c fp32 [4096,4096]"
            self.fn, self.dtype, self.samples = rp.mul_add, "f32", 4096
            self.make = lambda seed: rp.inputs_mul_add(seed=seed)
            self.batch_inputs = [0, 1, 2]
            self.bytes, self.flops, self.bound = 4 * 4096 * 4096 * 4, None, "hbm"
        elif key == "c2":
            self.name = "c2 mean(relu(x*w+b),-1) x bf16 [16384,4096], w,b bf16 [4096] -> fp32 [16384]"
            self.fn, self.dtype, self.samples = rp.reduce_mean_fusion, "bf16", 16384
            self.make = lambda seed: rp.inputs_reduce_mean(seed=seed)
            self.batch_inputs = [0]
            self.bytes, self.flops, self.bound = 16384 * 4096 * 2 + 2 * 4096 * 2 + 16384 * 4, None, "hbm"
        elif key == "c2g":
            self.name = "c2g mean(relu(x*w-b),-1) bf16 [16384,4096]: config 2's traffic through a run-time kernel instance"
            self.fn, self.dtype, self.samples = rp.reduce_mean_variant, "bf16", 16384
            self.make = lambda seed: rp.inputs_reduce_mean(seed=seed)
            self.batch_inputs = [0]
            self.bytes, self.flops, self.bound = 16384 * 4096 * 2 + 2 * 4096 * 2 + 16384 * 4, None, "hbm"
        elif key == "c3":
            self.name = "c3 row softmax forward fp32 [32768,8192]"
            self.fn, self.dtype, self.samples = rp.softmax_forward, "f32", 32768
            self.make = lambda seed: rp.inputs_softmax(seed=seed)[:1]
            self.batch_inputs = [0]
            self.bytes, self.flops, self.bound = 2 * 32768 * 8192 * 4, None, "hbm"
        elif key == "c3b":
            self.name = "c3 row softmax backward fp32 [32768,8192]"
            self.fn, self.dtype, self.samples = rp.softmax_backward, "f32", 32768

            def make(seed):
                logits, grad = rp.inputs_softmax(seed=seed)
                return [grad, torch.softmax(logits, -1)]

            self.make = make
            self.batch_inputs = [0, 1]
            self.bytes, self.flops, self.bound = 3 * 32768 * 8192 * 4, None, "hbm"
        elif key == "c4":
            self.name = "c4 MLP Linear(1024,4096)+ReLU+Linear(4096,1024) bf16, x [8192,1024]"
            self.module = rp.make_mlp()
            self.fn, self.dtype, self.samples = self.module, "bf16", 8192
            self.make = lambda seed: rp.inputs_mlp(seed=seed)
            self.batch_inputs = [0]
            self.bytes, self.flops, self.bound = None, 2 * 2 * 8192 * 1024 * 4096, "tensor"
        elif key == "c5":
            self.name = "c5 causal SDPA bf16 [8,16,2048,128]"
            self.fn, self.dtype, self.samples = rp.causal_attention, "bf16", 8
            self.make = lambda seed: rp.inputs_attention(seed=seed)
            self.batch_inputs = [0, 1, 2]
            self.bytes, self.flops, self.bound = None, 4 * 8 * 16 * 2048 * 2048 * 128 // 2, "tensor"
        else:
            raise SystemExit(f"unknown workload {key}")


# ---------------------------------------------------------------- helpers
def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            d = json.load(f)
        return d, "measured"
    except Exception:
        return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed regions run."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.samples: list[list[str]] = []
        self.proc = None
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except Exception:
            self.proc = None
            return

        def pump():
            for line in self.proc.stdout:
                parts = [p.strip() for p in line.split(",")]
                if len(parts) >= 6:
                    self.samples.append(parts)

        self.thread = threading.Thread(target=pump, daemon=True)
        self.thread.start()

    def stop(self) -> dict:
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except Exception:
                self.proc.kill()
        if self.thread is not None:
            self.thread.join(timeout=5)
        sm, mx, reasons = [], [], set()
        for s in self.samples:
            try:
                sm.append(float(s[0]))
                mx.append(float(s[1]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), s[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        busy = [c for c in sm if c >= 0.5 * max(sm)] if sm else []
        return {"sm_mhz": statistics.median(busy) if busy else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def dist_setup(n_gpus: int):
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        import torch.distributed as dist

        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    return rank, world, local


def barrier(world: int):
    if world > 1:
        import torch.distributed as dist

        dist.barrier()
    torch.cuda.synchronize()


def max_over_ranks(value: float, world: int, device) -> float:
    if world == 1:
        return value
    import torch.distributed as dist

    t = torch.tensor([value], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


# ---------------------------------------------------------------- CPU arm
def time_reference(wl: Workload, steps: int, warmup: int):
    """The reference's executed path: the graph traced by Dynamo and run as eager ops on CPU
    tensors with every host thread (conductor/compiler/gcu_backend.py:89)."""
    from oracle import reference_path as rp

    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    inputs = wl.make(0)
    fn = wl.fn
    if wl.module is not None:
        import copy

        fn = copy.deepcopy(wl.module).cpu()
    torch._dynamo.reset()
    compiled = torch.compile(fn, backend=rp.reference_backend)
    with torch.no_grad():
        for _ in range(max(warmup, 1)):
            compiled(*inputs)
        t0 = time.perf_counter()
        for _ in range(steps):
            compiled(*inputs)
        dt = time.perf_counter() - t0
    torch._dynamo.reset()
    ms = dt / steps * 1e3
    return wl.samples / (dt / steps), ms, torch.get_num_threads()


def reference_arm(args, wl: Workload):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    steps = max(1, min(args.steps, 50))
    value, ms, threads = time_reference(wl, steps, max(args.warmup, 3))
    line = {
        "impl": "reference", "metric": "compiled-graph samples/s", "value": value, "unit": "samples/s",
        "n_gpus": args.gpus, "steps": steps, "warmup": max(args.warmup, 3), "ms_per_step": ms,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": wl.dtype, "data": "synthetic",
        "config": {"workload": wl.name, "path": "reference backend falls back to PyTorch eager on CPU tensors",
                   "torch": torch.__version__},
        "cpu_baseline": {"value": value, "unit": "samples/s", "cores": threads, "kind": "port",
                         "sample": f"full batch, {steps} steps"},
        "e2e": {"value": value, "unit": "samples/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------- GPU arm
def gpu_arm(args, wl: Workload):
    import conductor  # noqa: F401  -- registers 'gcu'
    from conductor_b200.compiler.gcu_backend import get_gcu_backend
    from conductor_b200.compiler.loader import load_library

    load_library()
    rank, world, local = dist_setup(args.gpus)
    if world != args.gpus and world > 1:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    peaks, peak_kind = load_peaks()

    # ---- inputs: a rotating pool of distinct batches, larger than L2 in total
    host0 = wl.make(0)
    batch_bytes = sum(host0[i].numel() * host0[i].element_size() for i in wl.batch_inputs)
    pool_n = max(2, -(-POOL_BYTES_MIN // batch_bytes))
    pool_n = min(pool_n, 8)
    host_pool = [host0] + [wl.make(1000 * rank + s) for s in range(1, pool_n)]
    if wl.module is not None:
        wl.module.to(dev)
    dev_pool = [[t.to(dev) for t in h] for h in host_pool]
    pinned_pool = [[t.pin_memory() for t in h] for h in host_pool[:2]]

    torch._dynamo.reset()
    compiled = torch.compile(wl.fn, backend="gcu")
    with torch.no_grad():
        first = compiled(*dev_pool[0])
    torch.cuda.synchronize()
    backend = get_gcu_backend()
    plan = list(backend._compiled_functions.values())[-1]
    kernels_per_step = sum(1 for l in plan.launches if l.template)
    # the graph's placeholders include lifted module parameters: run every pool entry once
    # through the public API and keep the placeholder tuples the plan actually received
    plan.record_inputs = True
    placeholder_pool = []
    with torch.no_grad():
        for inp in dev_pool:
            compiled(*inp)
            placeholder_pool.append(plan.last_inputs)
    plan.record_inputs = False
    torch.cuda.synchronize()
    dev_pool = placeholder_pool

    # One CUDA graph per pool slot (one step each) and one "sequence" graph holding SEQ steps
    # that walk the pool: K timed steps = K // SEQ sequence replays + K % SEQ single replays.
    class _Direct:
        def __init__(self, sets):
            self.sets, self.runs = sets, len(sets)

        def replay(self):
            for inp in self.sets:
                plan(*inp)

    seq_len = pool_n * max(1, 32 // pool_n)
    seq_sets = [dev_pool[i % pool_n] for i in range(seq_len)]
    if args.no_graphs:
        singles = [_Direct([inp]) for inp in dev_pool]
        sequence = _Direct(seq_sets)
    else:
        singles = [plan.capture(*inp) for inp in dev_pool]
        sequence = plan.capture_sequence(seq_sets)

    def run_steps(k: int):
        for _ in range(k // seq_len):
            sequence.replay()
        for i in range(k % seq_len):
            singles[i % pool_n].replay()

    clocks = ClockSampler(local)
    if rank == 0:
        clocks.start()

    # ---- value: K steps, inputs resident
    run_steps(max(args.warmup, 3))
    barrier(world)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    run_steps(args.steps)
    e1.record()
    torch.cuda.synchronize()
    dev_ms = max_over_ranks(e0.elapsed_time(e1), world, dev)
    barrier(world)
    ms_per_step = dev_ms / args.steps
    value = wl.samples * world / (ms_per_step * 1e-3)

    if args.quick:          # profiling runs: the timed steps only
        if rank == 0:
            clocks.stop()
            print(json.dumps({"metric": "compiled-graph samples/s", "value": value, "ms_per_step": ms_per_step,
                              "quick": True, "config": {"workload": wl.name}}), flush=True)
        return

    # ---- roofline: the dominant kernel, many launches inside one timed region (about 1.5 s)
    reps = max(4, min(2000, int(1500 / max(ms_per_step * seq_len, 1e-3))))
    sequence.replay()
    torch.cuda.synchronize()
    e0.record()
    for _ in range(reps):
        sequence.replay()
    e1.record()
    torch.cuda.synchronize()
    reps *= seq_len
    kern_ms = e0.elapsed_time(e1) / reps / max(kernels_per_step, 1)
    if wl.bound == "hbm":
        achieved = wl.bytes / (kern_ms * 1e-3) / 1e9
        peak, unit = float(peaks["hbm_gbs"]), "GB/s"
    else:
        achieved = wl.flops / max(kernels_per_step, 1) / (kern_ms * 1e-3) / 1e12
        peak, unit = float(peaks.get("bf16_tflops_sustained", peaks["bf16_tflops"])), "TFLOP/s"
    roofline = {"bound": wl.bound, "achieved": achieved, "peak": peak, "unit": unit, "frac": achieved / peak,
                "traffic": TRAFFIC_BYTES.get(wl.key), "peak_source": f"MEASURED_PEAKS.json ({peak_kind})",
                "kernel_ms": kern_ms, "launches_timed": reps * kernels_per_step,
                "vs_nominal_8TBs": achieved / 8000.0 if wl.bound == "hbm" else None}

    # ---- e2e: public API, host tensors in pinned memory, H2D + kernels + D2H every step
    e2e_steps = max(3, min(args.steps, 200 if batch_bytes < (1 << 28) else 20))
    if wl.module is not None:
        # the reference's convention: model and inputs live on the host; the callable keeps
        # device copies of the parameters and stages the activations every call
        import copy

        host_module = copy.deepcopy(wl.module).cpu()
        torch._dynamo.reset()
        compiled = torch.compile(host_module, backend="gcu")
    with torch.no_grad():
        for i in range(3):
            out = compiled(*pinned_pool[i % 2])
        barrier(world)
        t0 = time.perf_counter()
        for i in range(e2e_steps):
            out = compiled(*pinned_pool[i % 2])
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
    dt = max_over_ranks(dt, world, dev)
    out0 = out[0] if isinstance(out, (tuple, list)) else out
    assert out0.device.type == "cpu"
    h2d = sum(t.numel() * t.element_size() for t in pinned_pool[0])
    d2h = out0.numel() * out0.element_size()
    e2e = {"value": wl.samples * world / (dt / e2e_steps), "unit": "samples/s", "h2d_bytes_per_step": h2d,
           "d2h_bytes_per_step": d2h, "steps": e2e_steps, "ms_per_step": dt / e2e_steps * 1e3}

    clock_info = clocks.stop() if rank == 0 else None

    cpu_baseline = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        cpu_steps = 20 if wl.key in ("c1", "c2", "c2g", "c4", "c5") else 8
        v, ms, threads = time_reference(wl, cpu_steps, 3)
        cpu_baseline = {"value": v, "unit": "samples/s", "cores": threads, "kind": "port",
                        "sample": f"full batch, {cpu_steps} steps, {ms:.2f} ms/step"}

    if rank == 0:
        line = {
            "metric": "compiled-graph samples/s", "value": value, "unit": "samples/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": wl.dtype, "data": "synthetic",
            "config": {"workload": wl.name, "samples_per_step_per_gpu": wl.samples, "sharding": f"rows x{world}",
                       "l2": f"{pool_n} distinct input batches rotate ({pool_n * batch_bytes >> 20} MiB > 126 MB L2)",
                       "launch": f"CUDA graph replay of the compiled plan, {seq_len} steps per graph"},
            "roofline": roofline, "cpu_baseline": cpu_baseline, "e2e": e2e,
            "gpu_launches": args.steps * kernels_per_step, "clocks": clock_info,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        import torch.distributed as dist

        dist.destroy_process_group()


# dram__bytes_read.sum + dram__bytes_write.sum per launch of the dominant kernel, from the ncu
# captures summarised under profiles/ (None until a capture exists for the workload)
TRAFFIC_BYTES: dict = {"c1": 235.0e6, "c2": 137.98e6, "c2g": 138.2e6, "c3": 2097.4e6, "c3b": 3180.9e6, "c4": 81.0e6, "c5": 552.2e6}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--workload", default="c2")
    ap.add_argument("--impl", default="conductor_b200", choices=["conductor_b200", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--quick", action="store_true", help="timed steps only (for profiler runs)")
    ap.add_argument("--no-graphs", action="store_true", help="launch the plan directly instead of replaying a CUDA graph")
    args = ap.parse_args()
    wl = Workload(args.workload)
    if args.impl == "reference":
        reference_arm(args, wl)
    else:
        gpu_arm(args, wl)


if __name__ == "__main__":
    main()
