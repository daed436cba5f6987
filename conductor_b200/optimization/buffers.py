"""Buffers and their scopes (reference: ``conductor/optimization/buffers.py:22-431``).

A buffer is the value of one FX node.  Its scope says where the value lives when
the graph runs on a B200: LOCAL = registers inside one fused kernel, SHARED =
shared memory / an HBM temporary visible to several kernels of the plan, GLOBAL =
HBM tensors that cross the graph boundary.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple

import torch

from ..utils.constants import BufferScope

_DTYPE_BYTES = {
    torch.float32: 4, torch.float16: 2, torch.bfloat16: 2, torch.float64: 8,
    torch.int32: 4, torch.int64: 8, torch.int16: 2, torch.int8: 1, torch.uint8: 1, torch.bool: 1,
    torch.complex64: 8, torch.complex128: 16,
}
_SCOPE_ORDER = {BufferScope.LOCAL: 0, BufferScope.SHARED: 1, BufferScope.GLOBAL: 2}


@dataclass(eq=False)
class Buffer:
    name: str
    scope: BufferScope
    dtype: torch.dtype
    shape: Optional[tuple[int, ...]] = None
    producer: Optional[Any] = None
    consumers: list = None
    is_temporary: bool = False
    birth_time: int = -1
    death_time: int = -1
    live_range: Tuple[int, int] = field(default_factory=lambda: (-1, -1))
    memory_size: int = 0
    is_input: bool = False
    is_output: bool = False
    constant_value: Optional[Any] = None   # tensor of a get_attr node / module parameter

    def __post_init__(self):
        if self.consumers is None:
            self.consumers = []
        if self.shape is not None:
            self.shape = tuple(int(d) for d in self.shape)
            self.memory_size = self.get_memory_footprint()

    def numel(self) -> int:
        n = 1
        for d in self.shape or ():
            n *= d
        return n

    def get_memory_footprint(self) -> int:
        """Bytes, or -1 when the shape is unknown."""
        if self.shape is None:
            return -1
        return self.numel() * _DTYPE_BYTES.get(self.dtype, 4)

    def set_shape(self, shape, dtype: Optional[torch.dtype] = None) -> None:
        self.shape = tuple(int(d) for d in shape)
        if dtype is not None:
            self.dtype = dtype
        self.memory_size = self.get_memory_footprint()

    def set_lifetime(self, birth_time: int, death_time: int) -> None:
        self.birth_time, self.death_time = birth_time, death_time
        self.live_range = (birth_time, death_time)

    def is_alive_at(self, time: int) -> bool:
        return self.birth_time != -1 and self.death_time != -1 and self.birth_time <= time <= self.death_time

    def overlaps_with(self, other: "Buffer") -> bool:
        if -1 in (self.birth_time, self.death_time, other.birth_time, other.death_time):
            return False
        return not (self.death_time < other.birth_time or other.death_time < self.birth_time)

    def can_reuse_memory_with(self, other: "Buffer") -> bool:
        """True when `other`'s storage may back this buffer: disjoint lifetimes, same scope and
        dtype, neither crossing the graph boundary, and `other` at least as large."""
        if self.overlaps_with(other) or self.scope != other.scope or self.dtype != other.dtype:
            return False
        if self.is_input or self.is_output or other.is_input or other.is_output:
            return False
        return 0 <= self.memory_size <= other.memory_size

    def promote_scope(self, new_scope: BufferScope) -> None:
        """LOCAL < SHARED < GLOBAL; never demotes (reference: ``buffers.py:167-178``)."""
        if _SCOPE_ORDER[new_scope] > _SCOPE_ORDER[self.scope]:
            self.scope = new_scope

    def __hash__(self) -> int:
        return id(self)

    def __repr__(self) -> str:
        return f"Buffer({self.name}, {self.scope.value}, {self.dtype}, {self.shape})"


class BufferManager:
    """Allocation, scope promotion, lifetimes and reuse (reference: ``buffers.py:208-431``)."""

    def __init__(self):
        self.buffers: Dict[str, Buffer] = {}

    def allocate_buffer(self, name: str, dtype: torch.dtype, shape=None,
                        scope: BufferScope = BufferScope.LOCAL) -> Buffer:
        base, n = name, 1
        while name in self.buffers:
            name = f"{base}_{n}"
            n += 1
        buf = Buffer(name=name, scope=scope, dtype=dtype, shape=shape)
        self.buffers[name] = buf
        return buf

    def reset(self) -> None:
        self.buffers.clear()

    def promote_buffer_scope(self, buffer: Buffer, required_scope: BufferScope) -> None:
        buffer.promote_scope(required_scope)

    def get_buffer(self, name: str) -> Optional[Buffer]:
        return self.buffers.get(name)

    def list_buffers(self) -> list[Buffer]:
        return list(self.buffers.values())

    def analyze_buffer_lifetimes(self, dag) -> Dict[str, Tuple[int, int]]:
        """Birth = position of the producer in topological order (0 for graph inputs and
        constants), death = position of the last consumer (end of graph for outputs)."""
        from .dag_naming import DAGTopologicalSorter

        order = DAGTopologicalSorter().sort(dag)
        when = {node: i for i, node in enumerate(order)}
        end = len(order)
        out: Dict[str, Tuple[int, int]] = {}
        for buf in dag.buffers:
            birth = when.get(buf.producer, 0) if buf.producer is not None else 0
            deaths = [when[c] for c in buf.consumers if c in when]
            death = max(deaths) if deaths else birth
            if buf.is_output:
                death = end
            buf.set_lifetime(birth, death)
            out[buf.name] = (birth, death)
        return out

    def optimize_buffer_reuse(self, buffers: List[Buffer]) -> dict[str, str]:
        """Greedy first-fit: map each temporary onto an earlier one whose life has ended."""
        mapping: dict[str, str] = {}
        pool: list[Buffer] = []
        owner_death: dict[str, int] = {}
        for buf in sorted(buffers, key=lambda b: b.birth_time):
            if buf.is_input or buf.is_output or buf.memory_size <= 0:
                continue
            for cand in pool:
                if owner_death[cand.name] < buf.birth_time and buf.can_reuse_memory_with(cand):
                    mapping[buf.name] = cand.name
                    owner_death[cand.name] = buf.death_time
                    break
            else:
                pool.append(buf)
                owner_death[buf.name] = buf.death_time
        return mapping
