"""Autograd bridge for compiled plans.

The reference backend is not wrapped in ``aot_autograd`` (``conductor/compiler/gcu_backend.py:30-89``
hands Dynamo's forward graph straight to the compiler), so a ``gcu``-compiled function has no
backward.  Here a plan whose single kernel is the row softmax becomes differentiable: when
gradients are enabled and the input requires them, the forward launch goes through
:class:`SoftmaxFunction`, whose backward launches the softmax-backward template
(``dx = y * (g - sum(g * y))``) on the same C ABI.  Other plans stay forward-only and say so.
"""
from __future__ import annotations

import torch

from ..codegen.kernel_templates import KernelLaunch
from ..codegen.operator_registry import Template
from ..utils.exceptions import UnsupportedOperationError


def _softmax_bwd_launch(shape, dtype) -> KernelLaunch:
    return KernelLaunch(Template.SOFTMAX_BWD, "softmax_bwd[autograd]", [], [], None, [tuple(shape)], [dtype])


class SoftmaxFunction(torch.autograd.Function):
    """y = softmax(x, -1) through the forward template; backward through the backward template."""

    @staticmethod
    def forward(ctx, x, executor, launch):
        (y,) = executor.execute(launch, [x.detach()])
        ctx.executor = executor
        ctx.save_for_backward(y)
        return y

    @staticmethod
    def backward(ctx, grad):
        (y,) = ctx.saved_tensors
        g = grad.contiguous()
        if g.dtype != y.dtype:
            g = g.to(y.dtype)
        (dx,) = ctx.executor.execute(_softmax_bwd_launch(y.shape, y.dtype), [g, y])
        return dx, None, None


def differentiable_kind(launches) -> str:
    """'softmax' when the plan is exactly one softmax-forward kernel, else ''."""
    kernels = [l for l in launches if l.template]
    if len(kernels) == 1 and kernels[0].template == Template.SOFTMAX_FWD and len(launches) == 1:
        return "softmax"
    return ""


def require_differentiable(launches) -> None:
    if not differentiable_kind(launches):
        names = ", ".join(l.name for l in launches if l.template)
        raise UnsupportedOperationError(
            names or "graph", "backward is only available for a plan that is one row-softmax kernel; "
            "run other graphs under torch.no_grad() or detach their inputs")
