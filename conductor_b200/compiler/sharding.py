"""Batch sharding of a compiled graph across the GPUs of one node.

Nothing like this exists in the reference (it has no distributed code at all); it is the
multi-GPU form of the same hot path.  Every benchmark graph is independent per row / token /
sequence, so a plan can run on a contiguous block of the leading dimension with no exchange
step: inputs that carry the batch dimension are sliced, everything else (weights, row-broadcast
vectors, scalars) is replicated, and there is NO collective on the data path.  An optional
all-gather (NCCL over NVLink for CUDA tensors, gloo in CPU tests) assembles the full output on
every rank when a caller asks for it.

Two ways to use it:

* one process per GPU (what ``bench.py --gpus N`` does): every rank builds
  ``ShardedCallable.for_rank(...)`` or simply compiles its own shard;
* one process driving several devices: ``GCUBackend`` returns a :class:`ShardedCallable` when
  ``config.runtime.devices > 1``; it walks the devices in turn (launches are asynchronous).
"""
from __future__ import annotations

from typing import Callable as TypingCallable, Optional, Sequence

import torch

from ..utils.exceptions import ExecutionError


def row_partition(n_rows: int, parts: int) -> list[tuple[int, int]]:
    """Contiguous blocks of ``ceil(n_rows / parts)`` rows; trailing parts may be empty."""
    if parts < 1:
        raise ValueError("parts must be >= 1")
    per = -(-n_rows // parts) if n_rows else 0
    out = []
    for p in range(parts):
        start = min(p * per, n_rows)
        out.append((start, min(start + per, n_rows)))
    return out


def batch_inputs(dag) -> tuple[int, list[int]]:
    """(batch size, indices of the graph inputs that carry the batch dimension).

    The batch size is the leading extent of the first graph output.  An input is sharded when
    every node that reads it uses it as a full-size operand: same rank and leading extent as the
    node's output (elementwise, softmax), the reduced operand of a reduction, operand 0 of
    ``linear``, or q/k/v of attention.  Weights, biases, row vectors and scalars are replicated."""
    if not dag.outputs or not dag.outputs[0].shape:
        return 0, []
    batch = dag.outputs[0].shape[0]
    picked = []
    for i, buf in enumerate(dag.inputs):
        if not buf.shape or buf.shape[0] != batch or not buf.consumers:
            continue
        ok = True
        for node in buf.consumers:
            out = node.outputs[0]
            pos = node.inputs.index(buf)
            if node.op_name == "linear":
                ok &= pos == 0
            elif node.op_name == "scaled_dot_product_attention":
                ok &= pos < 3
            elif node.is_reduction():
                ok &= pos == 0 and len(buf.shape) >= 2
            else:
                ok &= out.shape is not None and len(out.shape) == len(buf.shape) and out.shape[0] == batch
        if ok:
            picked.append(i)
    return batch, picked


def _output_spec(dag):
    """[(shape, dtype)] of the graph's tensor outputs, or None when any of them is unknown."""
    spec = []
    for buf in dag.outputs:
        if buf.shape is None or buf.dtype is None:
            return None
        spec.append((tuple(buf.shape), buf.dtype))
    return spec or None


class ShardedCallable:
    """Runs ``run_shard`` on this rank's (or each device's) block of rows.

    ``run_shard(inputs, device_index)`` receives the inputs with the batch inputs already sliced
    and returns a tuple of outputs whose leading dimension is the shard's row count.
    """

    def __init__(self, run_shard: TypingCallable, batch: int, batch_input_idx: Sequence[int], *,
                 devices: Optional[Sequence[int]] = None, rank: Optional[int] = None,
                 world_size: Optional[int] = None, process_group=None, gather_outputs: bool = True,
                 output_spec: Optional[Sequence[tuple]] = None):
        if (devices is None) == (rank is None):
            raise ValueError("give either `devices` (one process, several GPUs) or `rank`/`world_size`")
        self.run_shard = run_shard
        self.batch = batch
        self.batch_input_idx = list(batch_input_idx)
        self.devices = list(devices) if devices is not None else None
        self.rank, self.world_size, self.group = rank, world_size, process_group
        self.gather_outputs = gather_outputs
        # [(shape, dtype)] of the full outputs: lets a rank whose block is empty (batch smaller
        # than the world) still take part in every all-gather with a zero-row contribution
        self.output_spec = [(tuple(s), d) for s, d in output_spec] if output_spec is not None else None

    # ------------------------------------------------------------------ construction
    @classmethod
    def from_artifact(cls, artifact, graph_module=None, n_devices: int = 1, **kw):
        """Single-process form over devices 0..n_devices-1 for a compiled artifact."""
        from .callable import Callable

        batch, idx = batch_inputs(artifact.dag)
        plans = {d: Callable(artifact, graph_module, device=torch.device("cuda", d), batch_size=batch)
                 for d in range(n_devices)}

        def run_shard(inputs, device_index):
            # every device works on its own copy of the block: inputs that live elsewhere
            # (another GPU, or replicated weights on the first one) are moved to it first
            dev = plans[device_index].default_device
            moved = [t.to(dev, non_blocking=True) if t.device.type == "cuda" and t.device != dev else t for t in inputs]
            return plans[device_index](*moved)

        return cls(run_shard, batch, idx, devices=list(range(n_devices)), output_spec=_output_spec(artifact.dag), **kw)

    @classmethod
    def for_rank(cls, artifact, rank: int, world_size: int, graph_module=None, device=None, **kw):
        """One rank of a ``torch.distributed`` world (one process per GPU): this rank runs block
        ``rank`` of ``row_partition(batch, world_size)`` on its own device."""
        from .callable import Callable

        batch, idx = batch_inputs(artifact.dag)
        plan = Callable(artifact, graph_module, device=device, batch_size=batch)

        def run_shard(inputs, _rank):
            return plan(*inputs)

        sc = cls(run_shard, batch, idx, rank=rank, world_size=world_size, output_spec=_output_spec(artifact.dag), **kw)
        sc.plan = plan
        return sc

    # ------------------------------------------------------------------ helpers
    def _slice(self, inputs, start, stop):
        out = list(inputs)
        for i in self.batch_input_idx:
            t = inputs[i]
            if t.shape[0] != self.batch:
                raise ExecutionError(f"input {i} has {t.shape[0]} rows, compiled for a batch of {self.batch}")
            out[i] = t[start:stop]
        return out

    # ------------------------------------------------------------------ call
    def __call__(self, *inputs):
        tensors = [t for t in inputs if isinstance(t, torch.Tensor)]
        if not self.batch_input_idx:
            raise ExecutionError("graph has no batch-carrying input to shard")
        if self.devices is not None:
            return self._call_devices(tensors)
        return self._call_rank(tensors)

    def _call_devices(self, tensors):
        parts = row_partition(self.batch, len(self.devices))
        results = []
        for d, (start, stop) in zip(self.devices, parts):
            if stop > start:
                results.append(self.run_shard(self._slice(tensors, start, stop), d))
        if not self.gather_outputs:
            return tuple(results)
        home = tensors[self.batch_input_idx[0]].device
        n_out = len(results[0])
        return tuple(torch.cat([r[k].to(home, non_blocking=True) for r in results], dim=0) for k in range(n_out))

    def _call_rank(self, tensors):
        import torch.distributed as dist

        parts = row_partition(self.batch, self.world_size)
        start, stop = parts[self.rank]
        if self.gather_outputs and self.output_spec is None and any(e == s for s, e in parts):
            # the partition is the same on every rank, so EVERY rank raises here, before any
            # collective is entered: nobody is left waiting in an all-gather
            raise ExecutionError(f"some ranks have no rows (batch {self.batch} over {self.world_size} ranks) and the "
                                 "output shapes are unknown: build the ShardedCallable with `output_spec`")
        local = self.run_shard(self._slice(tensors, start, stop), self.rank) if stop > start else None
        if not self.gather_outputs:
            return local if local is not None else ()
        per = parts[0][1] - parts[0][0]
        even = per * self.world_size == self.batch
        n_out = len(local) if local is not None else len(self.output_spec)
        device = tensors[self.batch_input_idx[0]].device
        outs = []
        for k in range(n_out):
            if local is not None:
                mine = local[k]
            else:
                shape, dtype = self.output_spec[k]
                mine = torch.empty((0,) + tuple(shape[1:]), dtype=dtype, device=device)
            if even:
                # equal blocks: gather straight into the full tensor, no padding and no concatenation
                full = mine.new_empty((self.batch,) + tuple(mine.shape[1:]))
                dist.all_gather_into_tensor(full, mine.contiguous(), group=self.group)
                outs.append(full)
                continue
            # equal-sized contributions: pad the (possibly shorter or empty) trailing blocks
            padded = mine.new_zeros((per,) + tuple(mine.shape[1:]))
            padded[: mine.shape[0]] = mine
            chunks = [torch.empty_like(padded) for _ in range(self.world_size)]
            dist.all_gather(chunks, padded, group=self.group)
            outs.append(torch.cat([c[: e - s] for c, (s, e) in zip(chunks, parts)], dim=0))
        return tuple(outs)
