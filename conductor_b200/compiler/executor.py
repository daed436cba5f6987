"""Marshal tensors across the C ABI and launch kernel templates
(reference: ``conductor/compiler/executor.py:47-62,577-628`` ``GCUKernelExecutor`` and
``conductor/compiler/host_wrapper.py:360-403`` ``execute_kernel_with_library``).

What is kept: tensors are made contiguous, passed as (pointer, shape) descriptors, the call
returns an ``int`` status and a non-zero status raises :class:`ExecutionError`.  What changed:
no per-call DSL parsing or dummy-tensor allocation (``executor.py:466-469``), outputs are
allocated from the plan's recorded shapes instead of ``empty_like(inputs[0])``
(``executor.py:611``), and launches are asynchronous on the current CUDA stream.
"""
from __future__ import annotations

import ctypes
import threading
from typing import Optional, Sequence

import torch

from ..codegen.operator_registry import Template
from ..codegen.kernel_templates import CdrLaunchItem, CdrTensor, KernelLaunch
from ..utils.exceptions import DeviceError, ExecutionError, UnsupportedOperationError
from ..utils.type_mapping import to_cdr_dtype
from .loader import load_library

CDR_ERR_UNSUPPORTED = -2
CDR_ERR_CUDA = -4


def fill_descriptor(desc: CdrTensor, t: torch.Tensor) -> None:
    desc.data = t.data_ptr()
    desc.dtype = to_cdr_dtype(t.dtype)
    desc.rank = t.dim()
    for i, (s, st) in enumerate(zip(t.shape, t.stride())):
        desc.shape[i] = s
        desc.stride[i] = st


def make_descriptors(tensors: Sequence[torch.Tensor]):
    arr = (CdrTensor * max(len(tensors), 1))()
    for i, t in enumerate(tensors):
        if t.dim() > 8:
            raise UnsupportedOperationError("tensor", f"rank {t.dim()} > 8")
        fill_descriptor(arr[i], t)
    return arr


def raise_for_status(lib, status: int, name: str) -> None:
    if status == 0:
        return
    msg = lib.cdr_last_error().decode(errors="replace")
    what = lib.cdr_status_string(status).decode()
    text = f"kernel '{name}' failed: {what}" + (f" ({msg})" if msg else "")
    if status == CDR_ERR_UNSUPPORTED:
        raise UnsupportedOperationError(name, msg or what)
    if status == CDR_ERR_CUDA:
        raise DeviceError(text)
    raise ExecutionError(text, kernel_name=name, status=status)


class GCUKernelExecutor:
    """Launches one :class:`KernelLaunch` on device tensors.

    The class name is the reference's (``executor.py:33``); the device it drives is a B200.
    """

    def __init__(self):
        self.lib = load_library()
        self._workspaces: dict[tuple, tuple] = {}
        self._item_cache: dict[tuple, tuple] = {}
        # which of several concurrent replays of one plan the launches being bound belong to: runs
        # captured on different streams of one graph must not share scratch (see Callable.capture_sequence).
        # Per thread: another thread's calls keep lane 0 while this one records a sequence.
        self._lane = threading.local()

    @property
    def workspace_lane(self) -> int:
        return getattr(self._lane, "value", 0)

    @workspace_lane.setter
    def workspace_lane(self, lane: int) -> None:
        self._lane.value = int(lane)

    def workspace_for(self, launch: KernelLaunch, ins, outs, in_desc, out_desc, params_ptr, params_size):
        """Scratch of the size the library asks for, one buffer per (device, launch, lane).  Launches
        that share a buffer are ordered by the stream they run on; runs of one plan that are in flight
        at the same time are bound under different `workspace_lane` values."""
        key = (ins[0].device, id(launch), self.workspace_lane)
        hit = self._workspaces.get(key)
        sig = launch._marshal[0] if launch._marshal is not None else None
        if hit is not None and hit[0] == sig and sig is not None:
            return hit[1]
        need = ctypes.c_size_t(0)
        rc = self.lib.cdr_workspace_bytes(launch.template, in_desc, len(ins), out_desc, len(outs), params_ptr,
                                          params_size, ctypes.byref(need))
        raise_for_status(self.lib, rc, launch.name)
        if need.value == 0:
            self._workspaces[key] = (sig, None)
            return None
        ws = hit[1] if hit is not None else None
        if ws is None or ws.numel() < need.value:
            ws = torch.zeros(need.value, dtype=torch.uint8, device=ins[0].device)
        self._workspaces[key] = (sig, ws)
        return ws

    def _prepare(self, launch: KernelLaunch, inputs: Sequence[torch.Tensor], outputs):
        """Marshal one launch: contiguous inputs, allocated outputs, descriptor arrays (built once
        per launch and shape signature, data pointers refreshed per call), parameter block, scratch."""
        if not inputs:
            raise ExecutionError("kernel launch without inputs", kernel_name=launch.name)
        device = inputs[0].device
        if device.type != "cuda":
            raise DeviceError(f"kernel templates run on CUDA tensors, got {device}")
        if launch.template == Template.COPY:
            ins = list(inputs)                      # the view's strides are the point
        else:
            ins = [t if t.is_contiguous() else self.make_contiguous(t) for t in inputs]
        if outputs is None:
            outputs = [torch.empty(shape, dtype=dt, device=device)
                       for shape, dt in zip(launch.out_shapes, launch.out_dtypes)]
        sig = tuple((t.shape, t.stride(), t.dtype) for t in ins) + tuple((t.shape, t.stride(), t.dtype) for t in outputs)
        m = launch._marshal
        if m is None or m[0] != sig:
            in_desc, out_desc = make_descriptors(ins), make_descriptors(outputs)
            if launch.params is not None:
                params_ptr = ctypes.cast(ctypes.byref(launch.params), ctypes.c_void_p)
                params_size = ctypes.sizeof(launch.params)
            else:
                params_ptr, params_size = None, 0
            m = (sig, in_desc, out_desc, params_ptr, params_size)
            launch._marshal = m
        else:
            _, in_desc, out_desc, params_ptr, params_size = m
            for i, t in enumerate(ins):
                in_desc[i].data = t.data_ptr()
            for i, t in enumerate(outputs):
                out_desc[i].data = t.data_ptr()
        ws = None
        if launch.needs_workspace:
            ws = self.workspace_for(launch, ins, outputs, in_desc, out_desc, params_ptr, params_size)
        return device, ins, outputs, in_desc, out_desc, params_ptr, params_size, ws

    def execute(self, launch: KernelLaunch, inputs: Sequence[torch.Tensor],
                outputs: Optional[Sequence[torch.Tensor]] = None) -> list[torch.Tensor]:
        """Run `launch`; allocates the outputs when none are passed.  Asynchronous.  Inputs that are
        not contiguous are first gathered with the strided-copy template (never by torch).

        The descriptor arrays of a launch are built once and kept on the launch object: a repeat
        call with the same shapes, strides and dtypes only refreshes the data pointers, which
        keeps the host cost of one launch to a few microseconds.  A launch object is therefore
        driven by one thread at a time."""
        device, ins, outputs, in_desc, out_desc, params_ptr, params_size, ws = self._prepare(launch, inputs, outputs)
        stream = torch.cuda.current_stream(device).cuda_stream
        args = (launch.template, in_desc, len(ins), out_desc, len(outputs), params_ptr, params_size,
                ws.data_ptr() if ws is not None else None, ws.numel() if ws is not None else 0, stream)
        if torch.cuda.current_device() == device.index:
            rc = self.lib.cdr_launch(*args)
        else:
            with torch.cuda.device(device):
                rc = self.lib.cdr_launch(*args)
        if rc != 0:
            raise_for_status(self.lib, rc, launch.name)
        return list(outputs)

    def execute_many(self, steps) -> list[list[torch.Tensor]]:
        """Run several launches with ONE call into the library (``cdr_launch_many``): the whole
        plan crosses the FFI once, as a compiled graph does in the reference
        (``host_wrapper.py:360-403``).  `steps` is a list of ``(launch, inputs, outputs or None)``;
        later steps may read tensors earlier steps write (stream order).  Returns the outputs of
        every step."""
        results: list = []
        batch: list = []          # (launch, prepared)
        seen: set = set()
        device = None

        def flush():
            nonlocal batch, seen
            if not batch:
                return
            # The item array only holds addresses of per-launch state (descriptor arrays, parameter
            # block, scratch) that is refreshed in place, so it is built once per sequence of launch
            # objects and reused while none of them was re-marshalled.
            key = tuple(id(launch) for launch, _ in batch)
            stamp = tuple((id(p[3]), launch.template, len(p[1]), len(p[2]), p[6], p[7].data_ptr() if p[7] is not None else 0)
                          for launch, p in batch)
            cached = self._item_cache.get(key)
            if cached is not None and cached[0] == stamp:
                items = cached[1]
            else:
                items = (CdrLaunchItem * len(batch))()
                for it, (launch, (dev, ins, outs, in_desc, out_desc, pp, ps, ws)) in zip(items, batch):
                    it.template_id, it.n_inputs, it.n_outputs = launch.template, len(ins), len(outs)
                    it.inputs, it.outputs = ctypes.addressof(in_desc), ctypes.addressof(out_desc)
                    it.params = pp.value if pp is not None else None
                    it.params_bytes = ps
                    it.workspace = ws.data_ptr() if ws is not None else None
                    it.workspace_bytes = ws.numel() if ws is not None else 0
                if len(self._item_cache) > 256:
                    self._item_cache.clear()
                self._item_cache[key] = (stamp, items)
            stream = torch.cuda.current_stream(device).cuda_stream
            failed = ctypes.c_int(-1)
            if torch.cuda.current_device() == device.index:
                rc = self.lib.cdr_launch_many(items, len(batch), stream, ctypes.byref(failed))
            else:
                with torch.cuda.device(device):
                    rc = self.lib.cdr_launch_many(items, len(batch), stream, ctypes.byref(failed))
            if rc != 0:
                name = batch[failed.value][0].name if 0 <= failed.value < len(batch) else "plan"
                raise_for_status(self.lib, rc, name)
            batch, seen = [], set()

        for launch, inputs, outputs in steps:
            # a launch object's descriptors are shared state: the same object twice in one call
            # (two layers of equal shape) would overwrite them, so the first part goes out first
            if id(launch) in seen:
                flush()
            prepared = self._prepare(launch, inputs, outputs)
            if device is not None and prepared[0] != device:
                flush()
            device = prepared[0]
            batch.append((launch, prepared))
            seen.add(id(launch))
            results.append(list(prepared[2]))
        flush()
        return results

    def make_contiguous(self, t: torch.Tensor) -> torch.Tensor:
        """Contiguous copy of a strided view through the strided-copy template."""
        launch = KernelLaunch(Template.COPY, "contiguous", [], [], None, [tuple(t.shape)], [t.dtype])
        return self.execute(launch, [t])[0]

    def execute_host(self, launch: KernelLaunch, inputs: Sequence[torch.Tensor], device: int = 0) -> list[torch.Tensor]:
        """Reference calling convention: CPU tensors in, CPU tensors out, synchronous
        (``cdr_execute_host``; the reference's ``execute_kernel`` does the copies itself,
        ``host_wrapper.py:169-182``)."""
        ins = [t.contiguous() for t in inputs]
        if any(t.device.type != "cpu" for t in ins):
            raise DeviceError("execute_host takes CPU tensors")
        outs = [torch.empty(shape, dtype=dt) for shape, dt in zip(launch.out_shapes, launch.out_dtypes)]
        in_desc, out_desc = make_descriptors(ins), make_descriptors(outs)
        if launch.params is not None:
            params_ptr = ctypes.cast(ctypes.byref(launch.params), ctypes.c_void_p)
            params_size = ctypes.sizeof(launch.params)
        else:
            params_ptr, params_size = None, 0
        rc = self.lib.cdr_execute_host(launch.template, in_desc, len(ins), out_desc, len(outs), params_ptr,
                                       params_size, device)
        raise_for_status(self.lib, rc, launch.name)
        return outs


_executor: Optional[GCUKernelExecutor] = None


def get_executor() -> GCUKernelExecutor:
    global _executor
    if _executor is None:
        _executor = GCUKernelExecutor()
    return _executor
