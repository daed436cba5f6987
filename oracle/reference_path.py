"""What the reference executes for a compiled graph -- TEST INFRASTRUCTURE ONLY.

``GCUBackend.__call__`` of the reference (conductor/compiler/gcu_backend.py:30-89) tries to
compile the FX graph through Choreo; without the ``choreo`` compiler that always fails and it
returns ``graph_module.forward``, i.e. the graph runs as PyTorch eager ops on the caller's CPU
tensors.  :func:`reference_backend` restates exactly that: a ``torch.compile`` backend that
hands the traced graph back unchanged.  :func:`run_reference` is the convenience the tests
and the benchmark's CPU baseline use.

The benchmark graphs and their seeded inputs (``examples/workloads.py``) are re-exported for
the tests' convenience.
"""
from __future__ import annotations

from typing import Callable, Sequence

import torch
import torch.nn as nn


def reference_backend(graph_module: torch.fx.GraphModule, example_inputs):
    """The reference's effective behaviour: return the graph's own forward (eager)."""
    return graph_module.forward


def run_reference(fn: Callable, inputs: Sequence[torch.Tensor]):
    """Run `fn` the way the reference backend ends up running it: traced by Dynamo, executed
    eagerly on CPU tensors."""
    cpu = [t.detach().cpu() if isinstance(t, torch.Tensor) else t for t in inputs]
    if isinstance(fn, nn.Module):
        fn = fn.cpu()
    torch._dynamo.reset()
    compiled = torch.compile(fn, backend=reference_backend)
    with torch.no_grad():
        out = compiled(*cpu)
    torch._dynamo.reset()
    return out


from examples.workloads import (  # noqa: E402,F401
    causal_attention, inputs_attention, inputs_mlp, inputs_mul_add, inputs_reduce_mean, inputs_softmax,
    make_mlp, mul_add, reduce_mean_fusion, softmax_backward, softmax_backward_written_out, softmax_forward)
