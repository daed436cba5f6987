"""FX node -> operation name (reference: ``conductor/codegen/operation_factory.py:31-49``)."""
from __future__ import annotations

import torch.fx as fx

_ALIASES = {"mm": "matmul", "bmm": "matmul", "mean": "reduce_mean", "_softmax": "softmax"}


class OperationFactory:
    def extract_operation_name(self, fx_node: fx.Node) -> str:
        """``add`` for ``operator.add``/``torch.add``/``aten.add.Tensor``, ``reduce_mean`` for
        ``mean``, ``matmul`` for ``mm``/``bmm``; ``unknown`` for non-call nodes."""
        if fx_node.op == "call_function":
            target = fx_node.target
            name = getattr(target, "__name__", None)
            if name is None:
                name = str(target).split(".")[-1]
            # aten overloads arrive as "add.Tensor"
            name = name.split(".")[0]
        elif fx_node.op == "call_method":
            name = str(fx_node.target)
        elif fx_node.op == "call_module":
            return "call_module"
        else:
            return "unknown"
        return _ALIASES.get(name, name)


_factory = OperationFactory()


def get_operation_factory() -> OperationFactory:
    return _factory
