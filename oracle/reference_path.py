"""What the reference executes for a compiled graph -- TEST INFRASTRUCTURE ONLY.

``GCUBackend.__call__`` of the reference (conductor/compiler/gcu_backend.py:30-89) tries to
compile the FX graph through Choreo; without the ``choreo`` compiler that always fails and it
returns ``graph_module.forward``, i.e. the graph runs as PyTorch eager ops on the caller's CPU
tensors.  :func:`reference_backend` restates exactly that: a ``torch.compile`` backend that
hands the traced graph back unchanged.  :func:`run_reference` is the convenience the tests
and the benchmark's CPU baseline use.

Also here: the five benchmark graphs and their seeded synthetic inputs, shared by tests and
bench so that both arms see identical data.
"""
from __future__ import annotations

import math
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


# ---------------------------------------------------------------- the five graphs
def mul_add(a, b, c):
    return a * b + c


def reduce_mean_fusion(x, w, b):
    return torch.mean(torch.relu(x * w + b), dim=-1, dtype=torch.float32)


def softmax_forward(logits):
    return torch.softmax(logits, dim=-1)


def softmax_backward(grad, y):
    return torch._softmax_backward_data(grad, y, -1, torch.float32)


def softmax_backward_written_out(grad, y):
    return y * (grad - (grad * y).sum(-1, keepdim=True))


def make_mlp(d_in=1024, d_hidden=4096, d_out=1024, dtype=torch.bfloat16, seed=0):
    torch.manual_seed(seed)
    m = nn.Sequential(nn.Linear(d_in, d_hidden), nn.ReLU(), nn.Linear(d_hidden, d_out))
    with torch.no_grad():
        m[0].bias.zero_()
        m[2].bias.zero_()
    return m.to(dtype).eval()


def causal_attention(q, k, v):
    return torch.nn.functional.scaled_dot_product_attention(q, k, v, is_causal=True)


# ---------------------------------------------------------------- seeded inputs
def _gen(seed=0):
    return torch.Generator().manual_seed(seed)


def inputs_mul_add(rows=4096, cols=4096, seed=0):
    g = _gen(seed)
    return [torch.randn(rows, cols, generator=g) for _ in range(3)]


def inputs_reduce_mean(rows=16384, cols=4096, seed=0):
    g = _gen(seed)
    x = torch.randn(rows, cols, generator=g).bfloat16()
    w = (torch.rand(cols, generator=g) + 0.5).bfloat16()
    b = (0.1 * torch.randn(cols, generator=g)).bfloat16()
    return [x, w, b]


def inputs_softmax(rows=32768, cols=8192, seed=0):
    g = _gen(seed)
    logits = 3 * torch.randn(rows, cols, generator=g) + (40 * torch.rand(rows, 1, generator=g) - 20)
    grad = torch.randn(rows, cols, generator=g)
    return [logits, grad]


def inputs_mlp(tokens=8192, d_in=1024, seed=0):
    g = _gen(seed)
    return [torch.randn(tokens, d_in, generator=g).bfloat16()]


def inputs_attention(batch=8, heads=16, seq=2048, dim=128, seed=0):
    g = _gen(seed)
    return [torch.randn(batch, heads, seq, dim, generator=g).bfloat16() for _ in range(3)]
