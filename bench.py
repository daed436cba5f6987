#!/usr/bin/env python
"""Benchmark of the compiled-graph hot path: all five benchmark configurations in one run.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload all|c1|c2|c3|c3b|c4|c5] [--impl reference]

A *pass* is one run of a `torch.compile(fn, backend='gcu')` graph over one batch of seeded
synthetic input.  A *step* is `passes_per_step` back-to-back passes that walk a rotating pool of
distinct input batches (larger than L2 in total); the count is chosen per configuration so that
the K timed steps last at least half a second, and is reported.  Six graphs are timed: c1 mul_add,
c2 mean(relu(x*w+b)), c3 softmax forward, c3b softmax backward, c4 MLP, c5 causal attention.

With N > 1 (launched under torch.distributed.run, one process per GPU) the FIXED configuration is
partitioned by rows / tokens / sequences: rank r runs block r of `row_partition(rows, N)` through
the row-count-polymorphic plan (`Callable(batch_size=...)`), with no collective on the data path
(strong scaling).  Each rank additionally runs the whole configuration (`weak`, replicas), and one
NCCL all-gather of the outputs is timed separately.

Prints ONE JSON line on rank 0.  Headline keys (`value`, `ms_per_step`, `roofline`, `e2e`,
`cpu_baseline`) are configuration c2; `per_config` carries the same keys for all six.
  value     samples/s over all ranks, inputs resident in HBM, plan replayed from a CUDA graph
  e2e       the same metric through the public API with HOST tensors: pinned host -> device copy
            of the step's inputs, kernel(s), device -> host read of the result, every pass
  roofline  achieved HBM GB/s (or TFLOP/s) of the configuration's kernel(s) over the timed region,
            against the measured peak
  cpu_baseline  the reference package itself (its `gcu` backend ends in PyTorch eager on the host
            cores) on the same batch, timed in a child process
`--impl reference` times only that CPU path and prints it with "impl": "reference".
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
REF_DIR = os.path.join(ROOT, "baseline", "_ref")

import torch  # noqa: E402

L2_BYTES = 126 * 1024 * 1024
POOL_BYTES_MIN = 4 * L2_BYTES          # rotating pool (inputs + outputs) is at least this large
MAX_POOL = 64
LANES = 3            # passes in flight in the timed sequences: one pass's ramp-up and tail overlap the steady state of the others
MAX_SEQ = 1024                         # passes captured in one CUDA graph
REGION_S = 0.6                         # every timed region lasts at least this long
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}
ALL = ["c1", "c2", "c3", "c3b", "c4", "c5"]
HEADLINE = "c2"
METRIC = "compiled-graph samples/s"

# dram__bytes_read.sum + dram__bytes_write.sum per launch of the dominant kernel at the full
# configuration, from the ncu captures summarised under profiles/
TRAFFIC_BYTES: dict = {"c1": 235.0e6, "c2": 137.98e6, "c2g": 138.2e6, "c3": 2097.4e6, "c3b": 3180.9e6, "c4": 81.0e6, "c5": 252.2e6}


# ---------------------------------------------------------------- workloads
class Workload:
    """One benchmark configuration: graph, seeded inputs, rows, algorithmic bytes / flops."""

    def __init__(self, key):
        from examples import workloads as rp

        self.key = key
        self.rp = rp
        self.module = None
        if key == "c1":
            self.name = "c1 mul_add a*b+c fp32 [4096,4096]"
            self.fn, self.dtype, self.rows = rp.mul_add, "f32", 4096
            self.make = lambda seed: rp.inputs_mul_add(seed=seed)
            self.user_batch = [0, 1, 2]
            self.bytes_per_row, self.flops_per_row, self.bound = 4 * 4096 * 4, None, "hbm"
            self.fixed_bytes = 0
        elif key == "c2":
            self.name = "c2 mean(relu(x*w+b),-1) x bf16 [16384,4096], w,b bf16 [4096] -> fp32 [16384]"
            self.fn, self.dtype, self.rows = rp.reduce_mean_fusion, "bf16", 16384
            self.make = lambda seed: rp.inputs_reduce_mean(seed=seed)
            self.user_batch = [0]
            self.bytes_per_row, self.flops_per_row, self.bound = 4096 * 2 + 4, None, "hbm"
            self.fixed_bytes = 2 * 4096 * 2
        elif key == "c2g":      # not part of the default run: config 2's traffic through a run-time kernel instance
            self.name = "c2g mean(relu(x*w-b),-1) bf16 [16384,4096]: a chain without an ahead-of-time kernel instance"
            self.fn, self.dtype, self.rows = rp.reduce_mean_variant, "bf16", 16384
            self.make = lambda seed: rp.inputs_reduce_mean(seed=seed)
            self.user_batch = [0]
            self.bytes_per_row, self.flops_per_row, self.bound = 4096 * 2 + 4, None, "hbm"
            self.fixed_bytes = 2 * 4096 * 2
        elif key == "c3":
            self.name = "c3 row softmax forward fp32 [32768,8192]"
            self.fn, self.dtype, self.rows = rp.softmax_forward, "f32", 32768
            self.make = lambda seed: rp.inputs_softmax(seed=seed)[:1]
            self.user_batch = [0]
            self.bytes_per_row, self.flops_per_row, self.bound = 2 * 8192 * 4, None, "hbm"
            self.fixed_bytes = 0
        elif key == "c3b":
            self.name = "c3b row softmax backward fp32 [32768,8192]"
            self.fn, self.dtype, self.rows = rp.softmax_backward, "f32", 32768
            self.make = lambda seed: list(reversed(rp.inputs_softmax(seed=seed)))   # [grad, logits]: y is made on the device
            self.user_batch = [0, 1]
            self.bytes_per_row, self.flops_per_row, self.bound = 3 * 8192 * 4, None, "hbm"
            self.fixed_bytes = 0
        elif key == "c4":
            self.name = "c4 MLP Linear(1024,4096)+ReLU+Linear(4096,1024) bf16, x [8192,1024]"
            self.module = rp.make_mlp()
            self.fn, self.dtype, self.rows = self.module, "bf16", 8192
            self.make = lambda seed: rp.inputs_mlp(seed=seed)
            self.user_batch = [0]
            self.bytes_per_row, self.flops_per_row, self.bound = None, 2 * 2 * 1024 * 4096, "tensor"
            self.fixed_bytes = 0
        elif key == "c5":
            self.name = "c5 causal SDPA bf16 [8,16,2048,128]"
            self.fn, self.dtype, self.rows = rp.causal_attention, "bf16", 8
            self.make = lambda seed: rp.inputs_attention(seed=seed)
            self.user_batch = [0, 1, 2]
            self.bytes_per_row, self.flops_per_row, self.bound = None, 4 * 16 * 2048 * 2048 * 128 // 2, "tensor"
            self.fixed_bytes = 0
        else:
            raise SystemExit(f"unknown workload {key}")

    # seeded host inputs of the whole configuration, as the graph's user arguments
    def host_inputs(self, seed=0):
        ins = self.make(seed)
        if self.key == "c3b":
            grad, logits = ins
            return [grad, torch.softmax(logits, -1)]
        return ins

    def device_batch(self, rows: int, dev, gen):
        """Fresh batch-carrying inputs drawn on the device with the configuration's distributions
        (pool slots other than the seeded one)."""
        k = self.key
        if k == "c1":
            return [torch.randn(rows, 4096, device=dev, generator=gen) for _ in range(3)]
        if k in ("c2", "c2g"):
            return [torch.randn(rows, 4096, device=dev, generator=gen).bfloat16()]
        if k in ("c3", "c3b"):
            logits = 3 * torch.randn(rows, 8192, device=dev, generator=gen)
            logits += 40 * torch.rand(rows, 1, device=dev, generator=gen) - 20
            if k == "c3":
                return [logits]
            return [torch.randn(rows, 8192, device=dev, generator=gen), torch.softmax(logits, -1)]
        if k == "c4":
            return [torch.randn(rows, 1024, device=dev, generator=gen).bfloat16()]
        if k == "c5":
            return [torch.randn(rows, 16, 2048, 128, device=dev, generator=gen).bfloat16() for _ in range(3)]
        raise AssertionError(k)


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
        self.samples: list[tuple[float, list[str]]] = []
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
                    self.samples.append((time.monotonic(), parts))

        self.thread = threading.Thread(target=pump, daemon=True)
        self.thread.start()

    @staticmethod
    def _summary(samples) -> dict:
        sm, mx, reasons = [], [], set()
        for _, s in samples:
            try:
                sm.append(float(s[0]))
                mx.append(float(s[1]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), s[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}

    def window(self, t0: float, t1: float) -> dict:
        """Clock summary of the samples taken inside [t0, t1] (monotonic seconds)."""
        return self._summary([s for s in self.samples if t0 <= s[0] <= t1])

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except Exception:
                self.proc.kill()
        if self.thread is not None:
            self.thread.join(timeout=5)


def dist_setup():
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


def sum_over_ranks(value: float, world: int, device) -> float:
    if world == 1:
        return value
    import torch.distributed as dist

    t = torch.tensor([value], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.SUM)
    return float(t.item())


def nbytes(tensors) -> int:
    return sum(t.numel() * t.element_size() for t in tensors if isinstance(t, torch.Tensor))


# ---------------------------------------------------------------- CPU arm
def reference_available() -> bool:
    return os.path.isfile(os.path.join(REF_DIR, "conductor", "__init__.py"))


def _import_reference():
    """Import the UNMODIFIED reference package installed under baseline/_ref (this process must
    not have imported the new package of the same name).  Returns the `kind` of the arm."""
    if not reference_available():
        return "port"
    os.environ.setdefault("PYTHONDONTWRITEBYTECODE", "1")
    os.environ.setdefault("CONDUCTOR_LOG_LEVEL", "ERROR")
    os.environ.setdefault("CONDUCTOR_DEBUG", "0")
    sys.path.insert(0, REF_DIR)
    import logging

    logging.disable(logging.CRITICAL)
    import conductor  # noqa: F401  -- the reference: registers its 'gcu' backend

    if not os.path.realpath(conductor.__file__).startswith(os.path.realpath(REF_DIR)):
        raise SystemExit(f"expected the reference under {REF_DIR}, imported {conductor.__file__}")
    try:
        from conductor.utils.config import get_config

        get_config().debug.enabled = False          # the shipped configuration dumps tensors
    except Exception:
        pass
    return "reference"


def time_reference(wl: Workload, steps: int, warmup: int, kind: str):
    """The reference's execution of the graph: `torch.compile(fn, backend='gcu')` of the reference
    package on CPU tensors, every host thread (its compile step fails without the Choreo
    toolchain and it runs the traced graph as eager ops, conductor/compiler/gcu_backend.py:70-89).
    Without an installed reference, the port of that path under oracle/ stands in."""
    inputs = wl.host_inputs(0)
    fn = wl.fn
    if wl.module is not None:
        import copy

        fn = copy.deepcopy(wl.module).cpu()
    torch._dynamo.reset()
    if kind == "reference":
        compiled = torch.compile(fn, backend="gcu")
    else:
        from oracle import reference_path as rp

        compiled = torch.compile(fn, backend=rp.reference_backend)
    with torch.no_grad():
        t0 = time.perf_counter()
        compiled(*inputs)
        first = time.perf_counter() - t0
        for _ in range(max(warmup - 1, 1)):
            t0 = time.perf_counter()
            compiled(*inputs)
            est = time.perf_counter() - t0
        steps = max(3, min(steps, int(8.0 / max(est, 1e-4))))       # bounded: about 8 s per configuration
        times = []
        for _ in range(steps):
            t0 = time.perf_counter()
            compiled(*inputs)
            times.append(time.perf_counter() - t0)
    torch._dynamo.reset()
    dt = sum(times) / steps
    return {"value": wl.rows / dt, "unit": "samples/s", "ms_per_step": dt * 1e3, "median_ms": statistics.median(times) * 1e3,
            "best_ms": min(times) * 1e3, "steps": steps, "first_call_s": first, "dtype": wl.dtype, "workload": wl.name}


def reference_arm(args, keys):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    kind = _import_reference()
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    per = {}
    for k in keys:
        wl = Workload(k)
        r = time_reference(wl, args.steps, max(args.warmup, 3), kind)
        r["cpu_baseline"] = {"value": r["value"], "unit": "samples/s", "cores": torch.get_num_threads(), "kind": kind,
                             "sample": f"whole batch, {r['steps']} steps"}
        r["e2e"] = {"value": r["value"], "unit": "samples/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
        per[k] = r
    head = per[HEADLINE if HEADLINE in per else keys[0]]
    line = {
        "impl": "reference", "metric": METRIC, "value": head["value"], "unit": "samples/s",
        "n_gpus": args.gpus, "steps": head["steps"], "warmup": max(args.warmup, 3), "ms_per_step": head["ms_per_step"],
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": head["dtype"], "data": "synthetic",
        "config": bench_config(head["workload"], keys),
        "cpu_baseline": head["cpu_baseline"], "e2e": head["e2e"], "gpu_launches": 0,
        "path": ("the reference package from baseline/_ref, torch.compile(backend='gcu') on CPU tensors" if kind == "reference"
                 else "port of the reference's executed path (oracle/reference_path.py): baseline/_ref is not installed"),
        "torch": torch.__version__, "host_threads": torch.get_num_threads(), "per_config": per,
    }
    print(json.dumps(line), flush=True)


def bench_config(workload_name: str, keys) -> dict:
    """The `config` object: identical in both arms."""
    return {"workload": workload_name, "configs": list(keys),
            "inputs": "seeded synthetic tensors of the benchmark shapes (no dataset)"}


def cpu_baseline_child(keys) -> dict:
    """Time the reference arm in a child process (the reference package shares this package's
    import name, so it cannot live in this process) and return its per-configuration results."""
    cmd = [sys.executable, os.path.abspath(__file__), "--impl", "reference", "--steps", "10", "--warmup", "3",
           "--workload", ",".join(keys)]
    env = {k: v for k, v in os.environ.items() if k not in ("RANK", "WORLD_SIZE", "LOCAL_RANK", "OMP_NUM_THREADS")}
    try:
        res = subprocess.run(cmd, capture_output=True, text=True, timeout=900, env=env, cwd=ROOT)
        for ln in reversed(res.stdout.strip().splitlines()):
            if ln.startswith("{"):
                return json.loads(ln)["per_config"]
        return {"error": (res.stderr or res.stdout)[-400:]}
    except Exception as exc:        # the baseline is reported, never required
        return {"error": repr(exc)}


# ---------------------------------------------------------------- GPU arm
class Measurement:
    """Compiles one configuration and times this rank's block of it."""

    def __init__(self, wl: Workload, rank: int, world: int, dev, peaks, args):
        self.wl, self.rank, self.world, self.dev, self.peaks, self.args = wl, rank, world, dev, peaks, args
        import conductor  # noqa: F401  -- registers 'gcu'
        from conductor_b200.compiler.callable import Callable
        from conductor_b200.compiler.gcu_backend import get_gcu_backend
        from conductor_b200.compiler.sharding import batch_inputs

        if wl.module is not None:
            wl.module.to(dev)
        # compile for the WHOLE configuration (what a user of the backend does), on tensors of the
        # full shape whose batch-carrying members hold no data yet
        self.host_full = wl.host_inputs(0)
        example = [torch.empty(t.shape, dtype=t.dtype, device=dev) if i in wl.user_batch else t.to(dev)
                   for i, t in enumerate(self.host_full)]
        torch._dynamo.reset()
        backend = get_gcu_backend()
        backend.clear_cache()                              # the only entry afterwards is this graph's plan
        self.compiled = torch.compile(wl.fn, backend="gcu")
        with torch.no_grad():
            self.compiled(*example)
        torch.cuda.synchronize()
        plan = list(backend._compiled_functions.values())[-1]
        plan.record_inputs = True
        with torch.no_grad():
            self.compiled(*example)
        plan.record_inputs = False
        self.template = list(plan.last_inputs)            # the graph's placeholders (module parameters lifted in)
        del example
        self.full_plan = plan
        self.batch, self.batch_idx = batch_inputs(plan.dag)
        if self.batch != wl.rows or len(self.batch_idx) != len(wl.user_batch):
            raise SystemExit(f"{wl.key}: batch inputs {self.batch_idx} of batch {self.batch} do not match the configuration")
        self.plan = Callable(plan.artifact, batch_size=self.batch)
        self.kernels_per_pass = sum(1 for l in plan.launches if l.template)

    def placeholders(self, batch_tensors):
        ph = list(self.template)
        for i, t in zip(self.batch_idx, batch_tensors):
            ph[i] = t
        return tuple(ph)

    # ------------------------------------------------------------ device-resident timing
    def run(self, start: int, stop: int, clocks) -> dict:
        wl, dev, args, world = self.wl, self.dev, self.args, self.world
        rows = stop - start
        seeded = [self.host_full[i][start:stop].to(dev) for i in wl.user_batch]
        with torch.no_grad():
            out0 = self.plan(*self.placeholders(seeded))
        slot_bytes = nbytes(seeded) + nbytes(out0)
        pool_n = int(min(MAX_POOL, max(2, -(-POOL_BYTES_MIN // max(slot_bytes, 1)))))
        gen = torch.Generator(device=dev).manual_seed(1000 * self.rank + 17)
        pool = [self.placeholders(seeded)] + [self.placeholders(wl.device_batch(rows, dev, gen)) for _ in range(pool_n - 1)]
        del out0
        torch.cuda.synchronize()

        # size the captured sequence from a direct run of a few passes
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with torch.no_grad():
            self.plan(*pool[0])
            e0.record()
            for i in range(4):
                self.plan(*pool[i % pool_n])
            e1.record()
        torch.cuda.synchronize()
        est_ms = max(e0.elapsed_time(e1) / 4, 1e-3)
        seq_len = int(min(MAX_SEQ, max(pool_n, 4.0 / est_ms)))
        seq_len = -(-seq_len // pool_n) * pool_n if seq_len > pool_n else pool_n
        class _Direct:
            def __init__(s, plan, sets):
                s.plan, s.sets = plan, sets

            def replay(s):
                with torch.no_grad():
                    for inp in s.sets:
                        s.plan(*inp)

        def build(n, lanes):
            sets = [pool[i % pool_n] for i in range(n)]
            seq = _Direct(self.plan, sets) if args.no_graphs else self.plan.capture_sequence(sets, keep_outputs="first", lanes=lanes)
            seq.replay()
            torch.cuda.synchronize()
            e0.record()
            seq.replay()
            seq.replay()
            e1.record()
            torch.cuda.synchronize()
            return seq, max(e0.elapsed_time(e1) / 2, 1e-3)

        def timed(lanes, n0, with_clocks):
            """One timed region: `steps` steps of back-to-back replays of a captured sequence with `lanes`
            independent passes in flight."""
            n = n0
            sequence, replay_ms = build(n, lanes)
            # the first estimate came from direct launches, which are launch-bound for microsecond kernels:
            # one graph replay should last a few milliseconds, so that the host's replay calls stay far ahead
            grown = n
            if not args.no_graphs and replay_ms < 3.0 and n < MAX_SEQ:
                grown = int(min(MAX_SEQ, n * math.ceil(4.0 / replay_ms)))
                grown = max(pool_n, grown // pool_n * pool_n)
            if grown > n:
                del sequence
                n = grown
                sequence, replay_ms = build(n, lanes)
            region = 0.05 if args.quick else REGION_S
            replays_per_step = max(1, math.ceil(region * 1e3 / (args.steps * replay_ms)))
            for _ in range(max(args.warmup, 3) * replays_per_step if not args.quick else 1):
                sequence.replay()
            barrier(world)
            t_wall0 = time.monotonic()
            e0.record()
            for _ in range(args.steps * replays_per_step):
                sequence.replay()
            e1.record()
            torch.cuda.synchronize()
            t_wall1 = time.monotonic()
            own = e0.elapsed_time(e1)
            barrier(world)
            del sequence
            return {"own_ms": own, "passes_per_step": replays_per_step * n, "seq_len": n,
                    "clocks": clocks.window(t_wall0, t_wall1) if (clocks is not None and with_clocks) else None}

        def roofline_of(own_ms, passes):
            pass_ms = own_ms / passes
            kern_ms = pass_ms / max(self.kernels_per_pass, 1)
            if wl.bound == "hbm":
                alg = wl.bytes_per_row * rows + wl.fixed_bytes
                achieved = alg / (kern_ms * 1e-3) / 1e9
                peak, unit = float(self.peaks["hbm_gbs"]), "GB/s"
            else:
                alg = wl.flops_per_row * rows
                achieved = alg / max(self.kernels_per_pass, 1) / (kern_ms * 1e-3) / 1e12
                peak, unit = float(self.peaks.get("bf16_tflops_sustained", self.peaks["bf16_tflops"])), "TFLOP/s"
            return {"bound": wl.bound, "achieved": achieved, "peak": peak, "unit": unit, "frac": achieved / peak,
                    "algorithmic": alg, "kernel_ms": kern_ms, "kernels_per_pass": self.kernels_per_pass,
                    "launches_timed": passes * self.kernels_per_pass, "region_ms": own_ms,
                    "vs_nominal": achieved / 8000.0 if wl.bound == "hbm" else achieved / 2250.0}

        lanes = 1 if args.no_graphs else max(1, args.lanes)
        main = timed(lanes, seq_len, True)
        own_ms = main["own_ms"]
        passes_per_step = main["passes_per_step"]      # per rank: the aggregate counts every rank's own rows x passes
        dev_ms = max_over_ranks(own_ms, world, dev)
        rows_done = sum_over_ranks(float(rows) * args.steps * passes_per_step, world, dev)   # samples of all ranks
        passes = args.steps * passes_per_step
        roofline = roofline_of(own_ms, passes)
        traffic = TRAFFIC_BYTES.get(wl.key)
        roofline["traffic"] = traffic * rows / wl.rows if traffic else None
        roofline["passes_in_flight"] = lanes
        if lanes > 1:
            # the same launches one at a time (every launch waits for the one before it): what one launch takes by itself
            alone = timed(1, seq_len, False)
            r1 = roofline_of(alone["own_ms"], args.steps * alone["passes_per_step"])
            roofline["one_at_a_time"] = {k: r1[k] for k in ("achieved", "frac", "kernel_ms", "launches_timed", "region_ms", "vs_nominal")}
        result = {
            "rows_per_gpu": rows, "rows_done_all_ranks": rows_done, "passes_per_step": passes_per_step, "ms_per_step": dev_ms / args.steps,
            "ms_per_pass": dev_ms / passes, "timed_region_ms": dev_ms, "pool_slots": pool_n,
            "pool_mib": pool_n * slot_bytes >> 20, "passes_per_graph": main["seq_len"], "passes_in_flight": lanes,
            "gpu_launches": passes * self.kernels_per_pass, "roofline": roofline,
            "clocks": main["clocks"],
        }
        region = 0.05 if args.quick else REGION_S
        if args.with_library and world == 1:
            result["library"] = self.library(pool, pool_n, region, own_ms / passes)
        del pool
        return result

    # ------------------------------------------------------------ the same passes through PyTorch's own kernels
    def library(self, pool, pool_n: int, region: float, own_pass_ms: float) -> dict:
        """Eager PyTorch (cuBLAS, its fused attention, ATen kernels) over the same rotating pool,
        replayed from a CUDA graph and timed the same way: a comparison beside the product path, not part of it."""
        wl = self.wl
        fn = wl.module if wl.module is not None else wl.fn
        pick = (lambda ph: [ph[i] for i in self.batch_idx]) if wl.module is not None else (lambda ph: list(ph))
        side = torch.cuda.Stream()
        with torch.no_grad():
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                for i in range(3):
                    fn(*pick(pool[i % pool_n]))
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            keep = []
            lanes = max(1, min(self.args.lanes, pool_n))
            with torch.cuda.graph(graph):
                main = torch.cuda.current_stream()
                branches = [main] + [torch.cuda.Stream() for _ in range(lanes - 1)]
                for b in branches[1:]:
                    b.wait_stream(main)
                for i in range(pool_n):
                    with torch.cuda.stream(branches[i % lanes]):
                        out = fn(*pick(pool[i]))
                        if i == 0:
                            keep.append(out)
                        del out
                for b in branches[1:]:
                    main.wait_stream(b)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        graph.replay()
        torch.cuda.synchronize()
        e0.record()
        graph.replay()
        e1.record()
        torch.cuda.synchronize()
        replays = max(3, math.ceil(region * 1e3 / max(e0.elapsed_time(e1), 1e-3)))
        for _ in range(3):
            graph.replay()
        e0.record()
        for _ in range(replays):
            graph.replay()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / (replays * pool_n)
        del graph, keep
        return {"what": f"eager PyTorch on the same pool, CUDA-graph replays, {lanes} passes in flight", "ms_per_pass": ms,
                "conductor_b200_ms_per_pass": own_pass_ms, "library_over_conductor_b200": ms / own_pass_ms}

    # ------------------------------------------------------------ all-gather of the outputs
    def allgather(self, start: int, stop: int) -> dict:
        """One NCCL all-gather of this configuration's output blocks (outside every roofline
        figure), and a check that `ShardedCallable` on the whole input reproduces this rank's block."""
        import torch.distributed as dist

        from conductor_b200.compiler.sharding import ShardedCallable

        wl, dev = self.wl, self.dev
        gen = torch.Generator(device=dev).manual_seed(4242)           # the same full input on every rank
        full = self.placeholders(wl.device_batch(wl.rows, dev, gen))
        sc = ShardedCallable.for_rank(self.full_plan.artifact, self.rank, self.world, device=dev, gather_outputs=True)
        with torch.no_grad():
            gathered = sc(*full)
            local = self.plan(*self.placeholders([full[i][start:stop] for i in self.batch_idx]))
        ok = bool(torch.equal(gathered[0][start:stop], local[0])) and gathered[0].shape[0] == wl.rows
        mine = local[0].contiguous()
        out = mine.new_empty((wl.rows,) + tuple(mine.shape[1:]))
        even = mine.shape[0] * self.world == wl.rows
        ms = None
        if even:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            for _ in range(3):
                dist.all_gather_into_tensor(out, mine)
            barrier(self.world)
            e0.record()
            for _ in range(10):
                dist.all_gather_into_tensor(out, mine)
            e1.record()
            torch.cuda.synchronize()
            ms = max_over_ranks(e0.elapsed_time(e1) / 10, self.world, dev)
        total = out.numel() * out.element_size()
        return {"ms": ms, "bytes": total, "algbw_gbs": total / (ms * 1e-3) / 1e9 if ms else None,
                "sharded_callable_matches_local_block": ok}

    # ------------------------------------------------------------ end to end, host tensors
    def e2e(self, start: int, stop: int) -> dict:
        """The public call with HOST tensors: every pass copies its inputs from pinned host memory
        to the device, runs the plan and copies the result back to the host.  One GPU: the callable
        `torch.compile(fn, backend='gcu')` returns (a module lives on the host, as in the reference;
        the callable keeps device copies of its parameters).  Several GPUs: this rank's block through
        the row-count-polymorphic `Callable` that `ShardedCallable` drives."""
        wl, dev, world = self.wl, self.dev, self.world

        def pinned_block(pos, shift):
            t = self.host_full[pos][start:stop]
            return (t.roll(shift, 0) if shift else t).contiguous().pin_memory()

        slots = []
        if world == 1:
            if wl.module is not None:
                import copy

                torch._dynamo.reset()
                fn = torch.compile(copy.deepcopy(wl.module).cpu(), backend="gcu")
            else:
                fn = self.compiled
            for shift in (0, 1):
                slots.append(tuple(pinned_block(pos, shift) if pos in wl.user_batch else t.pin_memory()
                                   for pos, t in enumerate(self.host_full)))
        else:
            fn = self.plan
            for shift in (0, 1):
                ph = list(self.template)                   # module parameters stay resident on the device
                if wl.module is None:
                    assert len(ph) == len(self.host_full)
                    ph = [t.pin_memory() if pos not in wl.user_batch else None for pos, t in enumerate(self.host_full)]
                for pos, idx in enumerate(self.batch_idx):
                    ph[idx] = pinned_block(wl.user_batch[pos], shift)
                slots.append(tuple(ph))
        with torch.no_grad():
            for i in range(2):
                out = fn(*slots[i % 2])
            t0 = time.perf_counter()
            out = fn(*slots[0])
            est = time.perf_counter() - t0
            steps = int(max(5, min(2000, math.ceil(REGION_S / max(est, 1e-5)))))
            if world > 1:
                steps = int(max_over_ranks(float(steps), world, dev))
            barrier(world)
            t0 = time.perf_counter()
            for i in range(steps):
                out = fn(*slots[i % 2])
            torch.cuda.synchronize()
            dt = time.perf_counter() - t0
        dt = max_over_ranks(dt, world, dev)
        out0 = out[0] if isinstance(out, (tuple, list)) else out
        assert out0.device.type == "cpu"
        h2d = nbytes([t for t in slots[0] if t.device.type == "cpu"])
        d2h = nbytes([out0])
        return {"value": wl.rows / (dt / steps), "unit": "samples/s",
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "steps": steps, "ms_per_step": dt / steps * 1e3,
                "timed_region_ms": dt * 1e3, "pcie_gbs_per_gpu": (h2d + d2h) / (dt / steps) / 1e9}


def h2d_bandwidth(dev, world: int) -> dict:
    """Pinned host -> device copy rate of this rank while every rank copies at once: the ceiling of
    the end-to-end figures."""
    n = 256 << 20
    host = torch.empty(n, dtype=torch.uint8, pin_memory=True)
    dst = torch.empty(n, dtype=torch.uint8, device=dev)
    dst.copy_(host, non_blocking=True)
    barrier(world)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(8):
        dst.copy_(host, non_blocking=True)
    e1.record()
    torch.cuda.synchronize()
    ms = max_over_ranks(e0.elapsed_time(e1) / 8, world, dev)
    return {"h2d_gbs_per_gpu_all_ranks_copying": n / (ms * 1e-3) / 1e9, "bytes": n}


def gpu_arm(args, keys):
    import conductor  # noqa: F401  -- registers 'gcu'
    from conductor_b200.compiler.loader import load_library
    from conductor_b200.compiler.sharding import row_partition

    load_library()          # fails loudly when the CUDA library is missing
    rank, world, local = dist_setup()
    if world != args.gpus and world > 1:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    peaks, peak_kind = load_peaks()
    clocks = ClockSampler(local) if rank == 0 else None
    if clocks is not None:
        clocks.start()

    per = {}
    t_begin = time.monotonic()
    for k in keys:
        wl = Workload(k)
        m = Measurement(wl, rank, world, dev, peaks, args)
        start, stop = row_partition(wl.rows, world)[rank]
        if args.shard_of > 1 and world == 1:       # one GPU standing in for rank 0 of a larger world
            start, stop = row_partition(wl.rows, args.shard_of)[0]
        r = m.run(start, stop, clocks)
        # strong scaling: the fixed configuration over all ranks; every rank's rows x passes, over the slowest rank's time
        r["value"] = r["rows_done_all_ranks"] / (r["timed_region_ms"] * 1e-3)
        r["unit"], r["dtype"], r["workload"], r["scaling"] = "samples/s", wl.dtype, wl.name, "strong"
        r["roofline"]["peak_source"] = f"MEASURED_PEAKS.json ({peak_kind})"
        if not args.quick:
            r["e2e"] = m.e2e(start, stop)
            if world > 1:
                r["allgather"] = m.allgather(start, stop)
                torch.cuda.empty_cache()
                w = m.run(0, wl.rows, None)      # replicas: every rank the whole configuration
                r["weak"] = {"value": w["rows_done_all_ranks"] / (w["timed_region_ms"] * 1e-3),
                             "unit": "samples/s", "ms_per_pass": w["ms_per_pass"], "roofline_frac": w["roofline"]["frac"],
                             "timed_region_ms": w["timed_region_ms"]}
        per[k] = r
        del m
        torch._dynamo.reset()
        torch.cuda.empty_cache()

    pcie = None if args.quick else h2d_bandwidth(dev, world)
    if clocks is not None:
        clocks.stop()
        clock_info = clocks.window(t_begin, time.monotonic())
    if rank == 0 and world == 1 and not args.no_cpu_baseline and not args.quick:
        base = cpu_baseline_child(keys)
        for k in keys:
            b = base.get(k)
            per[k]["cpu_baseline"] = b["cpu_baseline"] | {"ms_per_step": b["ms_per_step"]} if isinstance(b, dict) else {"error": base.get("error")}

    if rank == 0:
        head = per[HEADLINE if HEADLINE in per else keys[0]]
        line = {
            "metric": METRIC, "value": head["value"], "unit": "samples/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": head["ms_per_step"],
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": head["dtype"], "data": "synthetic",
            "config": bench_config(head["workload"], keys),
            "roofline": head["roofline"], "cpu_baseline": head.get("cpu_baseline"), "e2e": head.get("e2e"),
            "gpu_launches": head["gpu_launches"], "clocks": clock_info,
            "passes_per_step": head["passes_per_step"],
            "run": {"sharding": f"fixed configuration, rows partitioned over {world} GPU(s), no data-path collective",
                    "step": "passes_per_step passes of the compiled plan over distinct batches, replayed from CUDA graphs with "
                            f"{head.get('passes_in_flight', 1)} independent passes in flight (roofline.one_at_a_time: the same launches serialised)",
                    "l2": "a rotating pool of distinct batches larger than 4x L2 (pool_mib per configuration)",
                    "timing": "CUDA events on the launching stream, max over ranks"},
            "host_link": pcie, "per_config": per,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        import torch.distributed as dist

        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default="all", help="all, or a comma-separated subset of " + ",".join(ALL))
    ap.add_argument("--impl", default="conductor_b200", choices=["conductor_b200", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--quick", action="store_true", help="short device-resident regions only (for profiler runs)")
    ap.add_argument("--no-graphs", action="store_true", help="launch the plan directly instead of replaying a CUDA graph")
    ap.add_argument("--lanes", type=int, default=LANES,
                    help="independent passes in flight inside a captured sequence (Callable.capture_sequence(lanes=...)); "
                         "1 = every launch waits for the one before it")
    ap.add_argument("--with-library", action="store_true",
                    help="one GPU: also time eager PyTorch's own kernels on the same batches (per_config[*].library)")
    ap.add_argument("--shard-of", type=int, default=1,
                    help="with one GPU: time the row block rank 0 of a world of this size would run (value then counts "
                         "the whole configuration per pass, i.e. what that world would reach if every rank kept this pace)")
    args = ap.parse_args()
    keys = ALL if args.workload == "all" else [k.strip() for k in args.workload.split(",") if k.strip()]
    for k in keys:
        if k not in ALL + ["c2g"]:
            raise SystemExit(f"unknown workload {k}")
    if args.impl == "reference":
        reference_arm(args, keys)
    else:
        gpu_arm(args, keys)


if __name__ == "__main__":
    main()
