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


class ShardedCallable:
    """Runs ``run_shard`` on this rank's (or each device's) block of rows.

    ``run_shard(inputs, device_index)`` receives the inputs with the batch inputs already sliced
    and returns a tuple of outputs whose leading dimension is the shard's row count.
    """

    def __init__(self, run_shard: TypingCallable, batch: int, batch_input_idx: Sequence[int], *,
                 devices: Optional[Sequence[int]] = None, rank: Optional[int] = None,
                 world_size: Optional[int] = None, process_group=None, gather_outputs: bool = True):
        if (devices is None) == (rank is None):
            raise ValueError("give either `devices` (one process, several GPUs) or `rank`/`world_size`")
        self.run_shard = run_shard
        self.batch = batch
        self.batch_input_idx = list(batch_input_idx)
        self.devices = list(devices) if devices is not None else None
        self.rank, self.world_size, self.group = rank, world_size, process_group
        self.gather_outputs = gather_outputs

    # ------------------------------------------------------------------ construction
    @classmethod
    def from_artifact(cls, artifact, graph_module=None, n_devices: int = 1, **kw):
        """Single-process form over devices 0..n_devices-1 for a compiled artifact."""
        from .callable import Callable

        batch, idx = batch_inputs(artifact.dag)
        plans = {d: Callable(artifact, graph_module, device=torch.device("cuda", d), batch_size=batch)
                 for d in range(n_devices)}

        def run_shard(inputs, device_index):
            return plans[device_index](*inputs)

        return cls(run_shard, batch, idx, devices=list(range(n_devices)), **kw)

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
        local = self.run_shard(self._slice(tensors, start, stop), self.rank) if stop > start else None
        if not self.gather_outputs:
            return local
        per = parts[0][1] - parts[0][0]
        outs = []
        n_out = len(local) if local is not None else 1
        for k in range(n_out):
            mine = local[k]
            # equal-sized contributions: pad the (possibly shorter) last block
            padded = mine.new_zeros((per,) + tuple(mine.shape[1:]))
            padded[: mine.shape[0]] = mine
            chunks = [torch.empty_like(padded) for _ in range(self.world_size)]
            dist.all_gather(chunks, padded, group=self.group)
            outs.append(torch.cat([c[: e - s] for c, (s, e) in zip(chunks, parts)], dim=0))
        return tuple(outs)
