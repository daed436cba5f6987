"""Topological ordering of the DAG (reference: ``conductor/optimization/dag_naming.py:66-131``).

The reference's per-node DSL variable naming (``dag_naming.py:150-288``) has no use
without a DSL emitter and is not reproduced."""
from __future__ import annotations

from collections import deque


class CycleError(ValueError):
    pass


class DAGTopologicalSorter:
    """Kahn's algorithm over producer -> consumer edges, stable in insertion order."""

    def sort(self, dag) -> list:
        nodes = list(dag.nodes)
        index = {n: i for i, n in enumerate(nodes)}
        indeg = {n: 0 for n in nodes}
        succ = {n: [] for n in nodes}
        for n in nodes:
            seen = set()
            for buf in n.inputs:
                p = getattr(buf, "producer", None)
                if p is not None and p in indeg and p is not n and p not in seen:
                    seen.add(p)
                    succ[p].append(n)
                    indeg[n] += 1
        ready = deque(sorted((n for n in nodes if indeg[n] == 0), key=index.get))
        order = []
        while ready:
            n = ready.popleft()
            order.append(n)
            for m in succ[n]:
                indeg[m] -= 1
                if indeg[m] == 0:
                    ready.append(m)
        if len(order) != len(nodes):
            raise CycleError("computation graph contains a cycle")
        return order
