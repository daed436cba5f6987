"""The five benchmark graphs and their seeded synthetic inputs.

Counterpart of the reference's ``examples/`` scripts (``examples/add_mul_fused_example.py:25-58``,
``examples/reduce_mean_fusion_example.py:52-102``), which define a small graph, compile it with
``backend='gcu'`` and compare against eager.  The graphs here are the ones the benchmark names;
inputs come from ``torch.Generator().manual_seed(seed)`` in fp32 on the CPU and are cast
afterwards, so every consumer (tests, benchmark, CPU baseline) sees identical data.  No public
dataset is involved: these synthetic tensors are the benchmark.
"""
from __future__ import annotations

import torch
import torch.nn as nn

def mul_add(a, b, c):
    return a * b + c


def reduce_mean_fusion(x, w, b):
    return torch.mean(torch.relu(x * w + b), dim=-1, dtype=torch.float32)


def reduce_mean_variant(x, w, b):
    """Same traffic as config 2 with a chain that has no ahead-of-time kernel instance (x*w - b): runs
    the run-time instance of the row-reduce skeleton."""
    return torch.mean(torch.relu(x * w - b), dim=-1, dtype=torch.float32)


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
