"""Operation node of the internal DAG (reference: ``conductor/optimization/graph_nodes.py:16-125``)."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Optional

from ..codegen.operator_registry import get_op_desc


@dataclass(eq=False)
class ConductorNode:
    """One ``call_function`` / ``call_method`` / ``call_module`` of the FX graph.

    ``inputs`` / ``outputs`` hold :class:`Buffer` objects.  ``metadata`` keeps what the
    template selector needs besides tensors: ``arg_spec`` (operand positions: a list of
    ``("buf", index_into_inputs)`` or ``("const", python_value)``), ``kwargs`` and the FX
    node name.  ``fusion_group`` is set once a cluster claims the node.
    """

    op_name: str
    inputs: list[Any] = field(default_factory=list)
    outputs: list[Any] = field(default_factory=list)
    metadata: dict[str, Any] = field(default_factory=dict)
    fusion_group: Optional[Any] = None

    def add_input(self, buf: Any) -> None:
        if buf not in self.inputs:
            self.inputs.append(buf)

    def add_output(self, buf: Any) -> None:
        if buf not in self.outputs:
            self.outputs.append(buf)

    def set_metadata(self, key: str, value: Any) -> None:
        self.metadata[key] = value

    def get_metadata(self, key: str, default: Any = None) -> Any:
        return self.metadata.get(key, default)

    @property
    def name(self) -> str:
        return self.metadata.get("fx_name", self.op_name)

    def op_info(self):
        return get_op_desc(self.op_name)

    def is_elementwise(self) -> bool:
        info = get_op_desc(self.op_name)
        return bool(info and info.is_elementwise())

    def is_reduction(self) -> bool:
        info = get_op_desc(self.op_name)
        return bool(info and info.is_reduction())

    def can_fuse_with(self, other: "ConductorNode") -> bool:
        """Pairwise compatibility used by cluster validation (reference: ``graph_nodes.py:65-93``).

        elementwise/elementwise, elementwise/reduction and reduction/elementwise pairs
        fuse; a matrix op accepts a trailing elementwise op (its epilogue)."""
        from .fusion import FusionHeuristics

        return FusionHeuristics().can_fuse_elementwise(self.op_name, other.op_name)

    def __str__(self) -> str:
        ins = [getattr(b, "name", str(b)) for b in self.inputs]
        outs = [getattr(b, "name", str(b)) for b in self.outputs]
        return f"ConductorNode(op={self.op_name}, inputs={ins}, outputs={outs})"

    __repr__ = __str__

    def __hash__(self) -> int:
        return id(self)
