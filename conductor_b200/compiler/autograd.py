"""Autograd bridge for compiled plans.

The reference backend is not wrapped in ``aot_autograd`` (``conductor/compiler/gcu_backend.py:30-89``
hands Dynamo's forward graph straight to the compiler), so a ``gcu``-compiled function has no
backward.  Here a plan whose single kernel is the row softmax becomes differentiable: when
gradients are enabled and the input requires them, the forward launch goes through
:class:`SoftmaxFunction`, whose backward launches the softmax-backward template
(``dx = y * (g - sum(g * y))``) on the same C ABI, and a plan that is a chain of linear(+relu)
kernels goes through :class:`LinearChainFunction`, whose backward is again GEMM-template launches.
Other plans stay forward-only and say so.
"""
from __future__ import annotations

import functools

import torch

from ..codegen.kernel_templates import KernelLaunch
from ..codegen.operator_registry import Template
from ..utils.exceptions import UnsupportedOperationError


# Backward launches are built once per (shape, dtype, layout) and reused: the executor keeps the
# marshalled descriptors on the launch object, so a training step pays for them only the first time.
@functools.lru_cache(maxsize=256)
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
        (dx,) = ctx.executor.execute(_softmax_bwd_launch(tuple(y.shape), y.dtype), [g, y])
        return dx, None, None


def differentiable_kind(launches, dag_inputs=None) -> str:
    """'softmax' when the plan is exactly one softmax-forward kernel, 'linear_chain' when it is a
    chain of linear(+relu) kernels whose weights are graph inputs, else ''."""
    kernels = [l for l in launches if l.template]
    if len(kernels) == 1 and kernels[0].template == Template.SOFTMAX_FWD and len(launches) == 1:
        return "softmax"
    if dag_inputs is not None and len(kernels) == len(launches) and linear_chain_layers(launches, dag_inputs):
        return "linear_chain"
    return ""


def require_differentiable(launches) -> None:
    if not differentiable_kind(launches):
        names = ", ".join(l.name for l in launches if l.template)
        raise UnsupportedOperationError(
            names or "graph", "backward is only available for a plan that is one row-softmax kernel; "
            "run other graphs under torch.no_grad() or detach their inputs")


# ---------------------------------------------------------------------------------------------
# Chains of linear layers (C4: Linear -> ReLU -> Linear).  Every gradient is again a launch of the
# GEMM template: the operand-layout switches of `cdr_gemm_params` let it read dY, x and W in place
# as the transposed operands the three products need, so no tensor is ever transposed in memory.
#   dX = dY @ W              x = dY [M, N],            W [N, K] read as [K'=N, N'=K]   (weight_layout KN)
#   dW = dY^T @ x            x = dY read as [K'=M, M'=N] (x_layout KM), W = x [M, K] read as [K'=M, N'=K]
#   dZ = dX * (H > 0)         the ReLU in front of a layer gates that layer's input gradient inside the epilogue of the
#                             product that makes it (gate_input), so the gradient never makes a trip through memory
#   db = sum over rows of dY  the column-sum template (HBM-bound: dY is read once; as a product with a row
#                             of ones the GEMM template ran it on N/256 CTAs and took as long as a full GEMM)
# Only a ReLU on the chain's OUTPUT needs its own launch (dZ = grad * (H > 0), one elementwise kernel).
@functools.lru_cache(maxsize=256)
def _gemm_launch(name, out_shape, dtype, weight_layout=0, x_layout=0, gate=0) -> KernelLaunch:
    from ..codegen.kernel_templates import CdrGemmParams

    return KernelLaunch(Template.GEMM_EPILOGUE, name, [], [], CdrGemmParams(0, 0, weight_layout, x_layout, gate),
                        [tuple(out_shape)], [dtype])


@functools.lru_cache(maxsize=256)
def _relu_mask_launch(shape, dtype) -> KernelLaunch:
    from ..codegen.kernel_templates import CdrEwInstr, CdrEwParams
    from ..codegen.operator_registry import EwOp
    from ..utils.type_mapping import to_cdr_dtype

    p = CdrEwParams()
    p.n_inputs, p.n_instr, p.n_outputs = 2, 3, 1          # r0 = grad, r1 = activation output
    p.instr[0] = CdrEwInstr(EwOp.CONST, 0, 0, 0, 0.0, to_cdr_dtype(torch.float32))
    p.instr[1] = CdrEwInstr(EwOp.GT, 1, 2, 0, 0.0, to_cdr_dtype(torch.float32))
    p.instr[2] = CdrEwInstr(EwOp.MUL, 0, 3, 0, 0.0, to_cdr_dtype(dtype))
    p.out_reg[0] = 4
    return KernelLaunch(Template.ELEMENTWISE, "relu_backward[autograd]", [], [], p, [tuple(shape)], [dtype])


def linear_chain_layers(launches, dag_inputs):
    """[(launch, has_bias)] when the plan is a chain of linear(+relu) kernels fed by graph inputs."""
    if not launches:
        return None
    prev_out = None
    layers = []
    for i, l in enumerate(launches):
        p = l.params
        if l.template != Template.GEMM_EPILOGUE or p is None or p.weight_layout != 0 or p.x_layout != 0:
            return None
        if len(l.inputs) not in (2, 3) or len(l.outputs) != 1:
            return None
        if i == 0:
            if l.inputs[0] not in dag_inputs:
                return None
        elif l.inputs[0] is not prev_out:
            return None
        if any(b not in dag_inputs for b in l.inputs[1:]):
            return None
        layers.append((l, len(l.inputs) == 3))
        prev_out = l.outputs[0]
    return layers


@functools.lru_cache(maxsize=256)
def _col_sum_launch(n: int, dtype) -> KernelLaunch:
    return KernelLaunch(Template.COL_SUM, "bias_grad[autograd]", [], [], None, [(n,)], [dtype], needs_workspace=True)


class LinearChainFunction(torch.autograd.Function):
    """Forward: the plan's GEMM launches.  Backward: GEMM launches with transposed-operand layouts."""

    @staticmethod
    def forward(ctx, executor, layers, x, *params):
        ctx.executor, ctx.layers = executor, layers
        acts = [x.detach()]
        it = iter(params)
        weights, steps = [], []
        for launch, has_bias in layers:
            w = next(it).detach()
            ins = [acts[-1], w] + ([next(it).detach()] if has_bias else [])
            h = torch.empty(launch.out_shapes[0], dtype=launch.out_dtypes[0], device=x.device)
            steps.append((launch, ins, [h]))
            acts.append(h)
            weights.append(w)
        executor.execute_many(steps)          # the whole chain in one call into the library
        ctx.save_for_backward(*acts, *weights)
        ctx.n_layers = len(layers)
        return acts[-1]

    @staticmethod
    def backward(ctx, grad):
        ex, layers, n = ctx.executor, ctx.layers, ctx.n_layers
        saved = ctx.saved_tensors
        acts, weights = saved[:n + 1], saved[n + 1:]
        dt = acts[0].dtype
        dev = acts[0].device
        g = grad if grad.dtype == dt and grad.is_contiguous() else grad.contiguous().to(dt)
        param_grads = []
        steps = []

        def out(shape):
            return torch.empty(shape, dtype=dt, device=dev)

        for i in range(n - 1, -1, -1):
            launch, has_bias = layers[i]
            w, x, h = weights[i], acts[i], acts[i + 1]
            N, K = w.shape
            g2 = g.reshape(-1, N)
            x2 = x.reshape(-1, K)
            M = g2.shape[0]
            if launch.params.activation == 1 and i == n - 1:
                # a ReLU on the chain's output gates the incoming gradient itself
                masked = out((M, N))
                steps.append((_relu_mask_launch((M, N), dt), [g2, h.reshape(-1, N)], [masked]))
                g2 = masked
            db = None
            if has_bias:
                db = out((N,))
                steps.append((_col_sum_launch(N, dt), [g2], [db]))
            dw = out((N, K))
            steps.append((_gemm_launch("weight_grad[autograd]", (N, K), dt, weight_layout=1, x_layout=1), [g2, x2], [dw]))
            param_grads = [dw] + ([db] if has_bias else []) + param_grads
            if i == 0 and not ctx.needs_input_grad[2]:
                g = None                     # nobody asked for d/dx of the chain's input: skip that product
                break
            dx = out((M, K))
            if i > 0 and layers[i - 1][0].params.activation == 1:
                # x is the previous layer's ReLU output: gate this gradient by (x > 0) in the epilogue
                steps.append((_gemm_launch("input_grad_relu[autograd]", (M, K), dt, weight_layout=1, gate=1), [g2, w, x2], [dx]))
            else:
                steps.append((_gemm_launch("input_grad[autograd]", (M, K), dt, weight_layout=1), [g2, w], [dx]))
            g = dx.reshape(x.shape)
        ex.execute_many(steps)                # every gradient launch of the chain in one call into the library
        return (None, None, g, *param_grads)
