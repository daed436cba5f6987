"""The object ``torch.compile`` calls at run time (reference: ``conductor/compiler/callable.py:42-94``).

Contract kept from the reference: called with the graph's placeholders positionally, returns a
**tuple**; a failing kernel raises :class:`ExecutionError`.  Input handling:

* CUDA tensors: the plan runs on their device and stream, asynchronously; outputs are CUDA tensors.
* CPU tensors (the reference's only mode, ``host_wrapper.py:374-396``): inputs are staged to the
  GPU through pinned buffers, the plan runs, outputs are copied back; the call is synchronous.
  A graph whose rows are independent (the same test that batch sharding uses) is run in row
  chunks on three streams, so that the copy in of chunk i+1, the kernels of chunk i and the copy
  out of chunk i-1 overlap inside the one call; PCIe is full duplex, so a graph with as much output
  as input finishes in about half the time of copy-in + kernels + copy-out.

There is no eager fallback: everything in the plan is a hand-written kernel template.
"""
from __future__ import annotations

import time
from typing import Optional

import torch

from ..codegen.kernel_templates import KernelLaunch
from ..utils.exceptions import DeviceError, ExecutionError
from ..utils.logging import get_logger
from ..utils.tracer import get_tracer
from .executor import get_executor
from .jit_compiler import CompiledArtifact

logger = get_logger(__name__)


class Callable:
    def __init__(self, artifact: CompiledArtifact, graph_module: Optional[torch.fx.GraphModule] = None,
                 device: Optional[torch.device] = None, batch_size: Optional[int] = None):
        self.artifact = artifact
        self.graph_module = graph_module      # kept for introspection only; never executed
        self.dag = artifact.dag
        self.launches: list[KernelLaunch] = artifact.launches
        self.default_device = device
        # when set, tensors whose leading extent equals it may arrive with fewer rows (one shard
        # of the batch); outputs with that leading extent are sized to the rows actually given
        self.batch_size = batch_size
        self._executor = None
        self._const_cache: dict[tuple, tuple] = {}
        self._pinned: dict[int, torch.Tensor] = {}
        self._param_cache: dict[tuple, tuple] = {}
        self.calls = 0
        self._grad_kind: Optional[str] = None
        self._grad_layers = None
        self.chunked_calls = 0                # host calls that ran in overlapped row chunks
        self._chunk_plan = None               # (batch, batch input indices) or False, decided on first host call
        self._batch_override: Optional[int] = None   # the batch size while a host call runs in row chunks
        # (a Callable is driven by one thread at a time: the override and the launches' marshalled
        # descriptors are per-object state)
        self._copy_streams: dict = {}
        # when set, every call stores the placeholder tensors it ran on (graph capture needs the
        # full list, including module parameters Dynamo lifted into placeholders)
        self.record_inputs = False
        self.last_inputs: Optional[tuple] = None

    # ------------------------------------------------------------------ helpers
    def _exec(self):
        if self._executor is None:
            self._executor = get_executor()
        return self._executor

    def _pick_device(self, tensors) -> torch.device:
        for t in tensors:
            if t.device.type == "cuda":
                return t.device
        if self.default_device is not None:
            return self.default_device
        if not torch.cuda.is_available():
            raise DeviceError("no CUDA device available; this backend has no CPU execution path")
        return torch.device("cuda", torch.cuda.current_device())

    def _constant_on(self, buf, device) -> torch.Tensor:
        """Device copy of a constant the plan captured (a module parameter, a ``get_attr`` tensor),
        refreshed when the source was modified in place since the copy was made."""
        key = (id(buf), device)
        src = buf.constant_value
        hit = self._const_cache.get(key)
        if hit is not None and hit[0] == src._version:
            return hit[1]
        if src.device == device and src.is_contiguous():
            t = src.detach()                  # already where it is needed: no copy, always current
        else:
            t = src.detach().to(device).contiguous()
        self._const_cache[key] = (src._version, t)
        return t

    def _stage_in(self, idx: int, t: torch.Tensor, device) -> torch.Tensor:
        """Host -> device through a reusable pinned buffer (pageable tensors) or directly
        (already pinned)."""
        if isinstance(t, torch.nn.Parameter):
            # module parameters Dynamo lifted into placeholders: keep a device copy until the
            # parameter is modified in place (its version counter moves) or replaced
            key = (idx, device)
            hit = self._param_cache.get(key)
            if hit is not None and hit[0] is t and hit[1] == t._version:
                return hit[2]
            dev_t = t.detach().to(device).contiguous()
            self._param_cache[key] = (t, t._version, dev_t)
            return dev_t
        if t.is_pinned():
            return t.to(device, non_blocking=True)
        t = t.contiguous()
        pin = self._pinned.get(idx)
        if pin is None or pin.shape != t.shape or pin.dtype != t.dtype:
            pin = torch.empty(t.shape, dtype=t.dtype, pin_memory=True)
            self._pinned[idx] = pin
        pin.copy_(t)
        return pin.to(device, non_blocking=True)

    # ------------------------------------------------------------------ call
    def __call__(self, *args):
        tracer = get_tracer()
        t_start = time.perf_counter() if tracer.should_trace_execution() else None
        tensors = [a for a in args if isinstance(a, torch.Tensor)]
        dag = self.dag
        if len(tensors) != len(dag.inputs):
            raise ExecutionError(f"compiled graph takes {len(dag.inputs)} tensors, got {len(tensors)}",
                                 kernel_name=self.artifact.entry_point)
        device = self._pick_device(tensors)
        host_mode = any(t.device.type == "cpu" for t in tensors)
        if host_mode and not (torch.is_grad_enabled() and any(t.requires_grad for t in tensors)):
            chunks = self._host_chunks(tensors)
            if chunks is not None:
                outputs = self._call_host_chunked(tensors, device, chunks)
                self.calls += 1
                self.chunked_calls += 1
                if t_start is not None:
                    tracer.trace_execution(self.artifact.entry_point, tensors, list(outputs), (time.perf_counter() - t_start) * 1e3)
                return tuple(outputs)
        env: dict = {}
        with torch.cuda.device(device):
            for i, (buf, t) in enumerate(zip(dag.inputs, tensors)):
                if buf.shape is not None and tuple(t.shape) != buf.shape and not self._is_shard(t, buf):
                    raise ExecutionError(
                        f"input {i} has shape {tuple(t.shape)}, compiled for {buf.shape}",
                        kernel_name=self.artifact.entry_point)
                env[buf] = self._stage_in(i, t, device) if t.device.type == "cpu" else t
            rows = self._rows_given(tensors)
            outputs = None
            if torch.is_grad_enabled() and any(t.requires_grad for t in tensors):
                from .autograd import LinearChainFunction, SoftmaxFunction, differentiable_kind, linear_chain_layers

                if self._grad_kind is None:           # decided once per plan
                    self._grad_kind = differentiable_kind(self.launches, dag.inputs)
                    self._grad_layers = linear_chain_layers(self.launches, dag.inputs) if self._grad_kind == "linear_chain" else None
                kind = self._grad_kind if not host_mode and rows is None else ""
                if kind == "softmax":
                    # forward through an autograd.Function whose backward is the softmax-backward template
                    outputs = [SoftmaxFunction.apply(env[dag.inputs[0]], self._exec(), self.launches[0])]
                elif kind == "linear_chain" and len(dag.output_spec) == 1 and dag.output_spec[0] is self.launches[-1].outputs[0]:
                    layers = self._grad_layers
                    operands = [env[self.launches[0].inputs[0]]]
                    for l, _ in layers:
                        operands += [env[b] for b in l.inputs[1:]]
                    outputs = [LinearChainFunction.apply(self._exec(), layers, *operands)]
                else:
                    # the reference would run such a graph eagerly and keep autograd working; there is
                    # no eager path here, and detaching silently would lose the caller's gradients
                    raise ExecutionError(
                        "inputs require grad but this compiled graph has no backward (differentiable plans: a row "
                        "softmax, a chain of linear(+relu) layers); call it under torch.no_grad() or detach the inputs",
                        kernel_name=self.artifact.entry_point)
            if outputs is None:
                outputs = self._run_plan(env, device, rows)
            if host_mode:
                # device -> pinned host (blocks come from torch's caching host allocator, so a
                # steady-state call allocates nothing), then one wait for the whole plan
                host = []
                for o in outputs:
                    if isinstance(o, torch.Tensor) and o.device.type == "cuda":
                        h = torch.empty(o.shape, dtype=o.dtype, pin_memory=True)
                        h.copy_(o, non_blocking=True)
                        host.append(h)
                    else:
                        host.append(o)
                torch.cuda.current_stream(device).synchronize()
                outputs = host
        self.calls += 1
        if self.record_inputs:
            self.last_inputs = tuple(env[b] for b in dag.inputs)
        if t_start is not None:
            tracer.trace_execution(self.artifact.entry_point, tensors, list(outputs), (time.perf_counter() - t_start) * 1e3)
        return tuple(outputs)

    def _rows_given(self, tensors) -> Optional[int]:
        """Row count of the block this call runs on, or None when it is the whole batch."""
        if self.batch_size is None:
            return None
        for buf, t in zip(self.dag.inputs, tensors):
            if buf.shape and buf.shape[0] == self.batch_size and t.dim() > 0 and t.shape[0] != self.batch_size:
                return t.shape[0]
        return None

    def _is_shard(self, t: torch.Tensor, buf) -> bool:
        return (self.batch_size is not None and buf.shape and buf.shape[0] == self.batch_size and t.dim() == len(buf.shape)
                and tuple(t.shape[1:]) == buf.shape[1:] and 0 < t.shape[0] <= self.batch_size)

    def _shard_shape(self, shape, rows):
        batch = self._batch_override if self._batch_override is not None else self.batch_size
        if rows is None or not shape or shape[0] != batch:
            return tuple(shape)
        return (rows,) + tuple(shape[1:])

    # ------------------------------------------------------------------ chunked host calls
    def _host_chunks(self, tensors) -> Optional[list]:
        """Row ranges to run a host-tensor call in, or None when the call runs in one piece: the
        graph must be row-parallel with every batch input on the host, free of layout-change
        launches (their views are tied to the full shapes), and large enough to be worth it."""
        from ..utils.config import get_config

        cfg = get_config().runtime
        if cfg.host_chunk_bytes <= 0 or self.batch_size is not None:
            return None
        if self._chunk_plan is None:
            from .sharding import batch_inputs

            from ..codegen.operator_registry import Template

            batch, idx = batch_inputs(self.dag)
            carried = {self.dag.inputs[i] for i in idx}
            row_local = (0, Template.ELEMENTWISE, Template.ROW_REDUCE, Template.SOFTMAX_FWD, Template.SOFTMAX_BWD,
                         Template.LAYER_NORM, Template.GEMM_EPILOGUE, Template.ATTENTION)
            ok = bool(idx) and batch > 1 and all(l.view_strides is None and l.out_view is None and l.template in row_local
                                                 for l in self.launches)
            # a product's weight must be whole on every chunk
            ok = ok and not any(l.template == Template.GEMM_EPILOGUE and any(b in carried for b in l.inputs[1:])
                                for l in self.launches)
            ok = ok and all(hasattr(o, "shape") and o.shape and o.shape[0] == batch for o in self.dag.output_spec)
            self._chunk_plan = (batch, idx) if ok else False
        if not self._chunk_plan:
            return None
        batch, idx = self._chunk_plan
        if any(tensors[i].device.type != "cpu" or tensors[i].shape[0] != batch for i in idx):
            return None
        in_bytes = sum(tensors[i].numel() * tensors[i].element_size() for i in idx)
        n = min(cfg.host_max_chunks, in_bytes // cfg.host_chunk_bytes, batch)
        if n < 2:
            return None
        per = -(-batch // n)
        return [(s, min(s + per, batch)) for s in range(0, batch, per)]

    def _streams_for(self, device):
        st = self._copy_streams.get(device)
        if st is None:
            st = self._copy_streams[device] = (torch.cuda.Stream(device=device), torch.cuda.Stream(device=device))
        return st

    def _call_host_chunked(self, tensors, device, chunks) -> list:
        batch, idx = self._chunk_plan
        dag = self.dag
        with torch.cuda.device(device):
            compute = torch.cuda.current_stream(device)
            h2d, d2h = self._streams_for(device)
            h2d.wait_stream(compute)
            d2h.wait_stream(compute)
            shared = {}
            for i, (buf, t) in enumerate(zip(dag.inputs, tensors)):
                if i not in idx:                       # weights, row vectors, scalars: staged once
                    shared[buf] = self._stage_in(i, t, device) if t.device.type == "cpu" else t
            sources = {}
            for i in idx:                              # pageable inputs go through a pinned copy, chunk by chunk
                t = tensors[i].contiguous()
                sources[i] = t
            host_out = None
            self._batch_override = batch
            try:
                for (s, e) in chunks:
                    env = dict(shared)
                    with torch.cuda.stream(h2d):
                        for i in idx:
                            src = sources[i][s:e]
                            if not src.is_pinned():
                                pin = torch.empty(src.shape, dtype=src.dtype, pin_memory=True)
                                pin.copy_(src)
                                src = pin
                            d = src.to(device, non_blocking=True)
                            d.record_stream(compute)
                            env[dag.inputs[i]] = d
                    compute.wait_stream(h2d)
                    outs = self._run_plan(env, device, e - s)
                    if host_out is None:
                        host_out = [torch.empty((batch,) + tuple(o.shape[1:]), dtype=o.dtype, pin_memory=True) for o in outs]
                    d2h.wait_stream(compute)
                    with torch.cuda.stream(d2h):
                        for h, o in zip(host_out, outs):
                            o.record_stream(d2h)
                            h[s:e].copy_(o, non_blocking=True)
            finally:
                self._batch_override = None
            d2h.synchronize()
        return host_out

    def _run_plan(self, env: dict, device, rows: Optional[int] = None) -> list:
        """Bind every launch's tensors (outputs are allocated here, views and aliases resolved),
        then hand the whole list to the library in one call."""
        ex = self._exec()
        steps = []
        for launch in self.launches:
            ins = []
            for b in launch.inputs:
                t = env.get(b)
                if t is None:
                    if b.constant_value is None:
                        raise ExecutionError(f"value {b.name} is not available", kernel_name=launch.name)
                    t = env[b] = self._constant_on(b, device)
                ins.append(t)
            if launch.template == 0:                       # alias: reshape, no kernel
                src = ins[0]
                if not src.is_contiguous():                # a caller's strided tensor: gather it with the copy template
                    src = env[launch.inputs[0]] = ex.make_contiguous(src)
                env[launch.outputs[0]] = src.reshape(self._shard_shape(launch.out_shapes[0], rows))
                continue
            if launch.view_strides is not None:            # transpose / permute / slice: gather the strided view
                if rows is not None:
                    raise ExecutionError("a plan with layout changes cannot run on a block of its rows", kernel_name=launch.name)
                src = ins[0]
                if not src.is_contiguous():
                    # the view's strides were derived for a contiguous source (every buffer of a plan
                    # is): a caller's strided tensor is gathered first, once, and reused by later launches
                    src = env[launch.inputs[0]] = ex.make_contiguous(src)
                ins = [torch.as_strided(src, launch.out_shapes[0], launch.view_strides, src.storage_offset() + launch.view_offset)]
            if launch.out_view is not None:                # cat: this launch fills one slice of the result
                if rows is not None:
                    raise ExecutionError("a plan with a concatenation cannot run on a block of its rows", kernel_name=launch.name)
                whole = env.get(launch.outputs[0])
                if whole is None:
                    whole = env[launch.outputs[0]] = torch.empty(launch.out_shapes[0], dtype=launch.out_dtypes[0], device=device)
                shape, strides, offset = launch.out_view
                steps.append((launch, ins, [torch.as_strided(whole, shape, strides, whole.storage_offset() + offset)]))
                continue
            outs = [torch.empty(self._shard_shape(sh, rows), dtype=dt, device=device)
                    for sh, dt in zip(launch.out_shapes, launch.out_dtypes)]
            steps.append((launch, ins, outs))
            for b, t in zip(launch.outputs, outs):
                env[b] = t
        if len(steps) == 1:
            ex.execute(*steps[0])
        elif steps:
            ex.execute_many(steps)
        result = []
        for item in self.dag.output_spec:
            if hasattr(item, "name") and item in env:
                result.append(env[item])
            elif hasattr(item, "constant_value") and item.constant_value is not None:
                result.append(self._constant_on(item, device))
            elif hasattr(item, "producer"):
                raise ExecutionError(f"output {item.name} was not produced", kernel_name=self.artifact.entry_point)
            else:
                result.append(item)
        return result

    # ------------------------------------------------------------------ CUDA graphs
    def capture(self, *device_tensors) -> "GraphedCall":
        """Record one run of the plan on `device_tensors` into a CUDA graph.  Replaying it
        re-runs every kernel of the plan on the same buffers with one driver call, which is
        what keeps microsecond-scale plans from being launch-bound."""
        return GraphedCall(self, [tuple(device_tensors)])

    def capture_sequence(self, input_sets, keep_outputs: str = "all", lanes: int = 1) -> "GraphedCall":
        """Record one run of the plan per entry of `input_sets` (tuples of device tensors)
        in a single CUDA graph: one driver call replays the whole sequence.
        ``keep_outputs="first"`` keeps only the first run's output tensors; the later runs'
        outputs are released inside the capture, so the graph's memory pool holds two runs'
        worth of outputs instead of one per run (long sequences of large graphs).
        ``lanes`` > 1 records run i on branch ``i % lanes`` of the graph: the runs are independent
        of one another (each has its own inputs and outputs), so up to `lanes` of them are in flight
        at a time and one run's ramp-up and tail overlap another's steady state.  Runs on one
        branch stay in order; every branch has its own scratch buffers."""
        return GraphedCall(self, [tuple(t) for t in input_sets], keep_outputs=keep_outputs, lanes=lanes)

    # reference API (callable.py:96-152)
    def get_artifact(self) -> CompiledArtifact:
        return self.artifact

    def plan_text(self) -> str:
        return self.artifact.metadata.get("plan", "")

    def __repr__(self) -> str:
        return f"Callable({self.artifact.entry_point}, kernels={sum(1 for l in self.launches if l.template)})"


class GraphedCall:
    """One or more runs of a plan captured in a CUDA graph for fixed input buffers (see
    :meth:`Callable.capture`, :meth:`Callable.capture_sequence`).

    ``replay()`` enqueues the recorded runs on the current stream.  ``outputs`` holds the
    output tuple of the first run, ``all_outputs`` one tuple per run; the tensors are reused by
    every replay."""

    def __init__(self, fn: Callable, input_sets, keep_outputs: str = "all", lanes: int = 1):
        if keep_outputs not in ("all", "first"):
            raise ValueError("keep_outputs is 'all' or 'first'")
        if lanes < 1:
            raise ValueError("lanes must be at least 1")
        if not input_sets or any(not ts or any(t.device.type != "cuda" for t in ts) for ts in input_sets):
            raise DeviceError("CUDA graphs capture device-resident inputs only")
        self.fn = fn
        self.input_sets = input_sets
        device = input_sets[0][0].device
        envs = [dict(zip(fn.dag.inputs, ts)) for ts in input_sets]
        rows = [fn._rows_given(ts) for ts in input_sets]
        side = torch.cuda.Stream(device=device)
        side.wait_stream(torch.cuda.current_stream(device))
        with torch.cuda.device(device), torch.cuda.stream(side):
            fn._run_plan(dict(envs[0]), device, rows[0])        # warm-up: lazy initialisation, constants
        torch.cuda.current_stream(device).wait_stream(side)
        torch.cuda.synchronize(device)
        self.lanes = lanes = min(lanes, len(input_sets))
        ex = fn._exec()
        if lanes > 1:
            # every lane's scratch exists before the capture (allocations inside it would come from the graph's pool)
            for lane in range(1, lanes):
                ex.workspace_lane = lane
                with torch.cuda.device(device), torch.cuda.stream(side):
                    fn._run_plan(dict(envs[0]), device, rows[0])
            ex.workspace_lane = 0
            torch.cuda.current_stream(device).wait_stream(side)
            torch.cuda.synchronize(device)
        self.graph = torch.cuda.CUDAGraph()
        self.all_outputs = []
        try:
            with torch.cuda.device(device), torch.cuda.graph(self.graph):
                main = torch.cuda.current_stream(device)
                branches = [main] + [torch.cuda.Stream(device=device) for _ in range(lanes - 1)]
                for b in branches[1:]:
                    b.wait_stream(main)                       # fork
                for i, (env, r) in enumerate(zip(envs, rows)):
                    ex.workspace_lane = i % lanes
                    with torch.cuda.stream(branches[i % lanes]):
                        out = fn._run_plan(dict(env), device, r)
                        if keep_outputs == "all" or i == 0:
                            self.all_outputs.append(tuple(out))
                        del out                               # dropped outputs: their blocks are reused by the branch's next run
                for b in branches[1:]:
                    main.wait_stream(b)                       # join
        finally:
            ex.workspace_lane = 0
        self.outputs = self.all_outputs[0]
        self.runs = len(input_sets)
        self.n_kernels = self.runs * sum(1 for l in fn.launches if l.template)

    def replay(self):
        self.graph.replay()
        return self.outputs
