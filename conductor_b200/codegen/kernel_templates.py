"""Cluster -> kernel-template instance.

This module takes the place of the reference's Choreo DSL emitter
(``conductor/codegen/dslgen.py:154-217`` ``generate_dsl_file``,
``dslgen.py:524-737`` body generation, ``dma_generator.py:80-268`` tile DMA).  Instead of
printing a ``.co`` program that a compiler turns into a kernel, it *selects* one of the
hand-written sm_100a templates of ``libconductor_b200.so`` for each fused cluster and
fills in that template's parameter block (``include/conductor_b200.h``).

Scope mapping (reference scopes: ``graph_analyzer.py:630-647``): cluster-internal LOCAL
buffers become virtual registers of the elementwise program and never touch memory;
SHARED buffers are HBM temporaries owned by the plan; GLOBAL buffers are the caller's
tensors.
"""
from __future__ import annotations

import ctypes
import math
from dataclasses import dataclass, field
from typing import Any, Optional

import torch

from ..optimization.buffers import Buffer, BufferScope
from ..optimization.fusion import FusionCluster, FusionType, _is_last_dim_reduction
from ..utils.exceptions import UnsupportedOperationError
from ..utils.type_mapping import is_float, is_int, to_cdr_dtype
from .operator_registry import EwOp, ReduceOp, Template, get_op_desc

# ---------------------------------------------------------------- C structs
CDR_MAX_RANK = 8
CDR_EW_MAX_INPUTS = 8
CDR_EW_MAX_INSTR = 24
CDR_EW_MAX_OUTPUTS = 4

IN_FULL, IN_ROW, IN_COL, IN_SCALAR = range(4)


class CdrTensor(ctypes.Structure):
    _fields_ = [("data", ctypes.c_void_p), ("dtype", ctypes.c_int32), ("rank", ctypes.c_int32),
                ("shape", ctypes.c_int64 * CDR_MAX_RANK), ("stride", ctypes.c_int64 * CDR_MAX_RANK)]


class CdrEwInstr(ctypes.Structure):
    _fields_ = [("op", ctypes.c_int32), ("a", ctypes.c_int32), ("b", ctypes.c_int32), ("c", ctypes.c_int32),
                ("imm", ctypes.c_float), ("round_to", ctypes.c_int32)]


class CdrEwParams(ctypes.Structure):
    _fields_ = [("n_inputs", ctypes.c_int32), ("n_instr", ctypes.c_int32), ("n_outputs", ctypes.c_int32),
                ("reserved", ctypes.c_int32), ("input_mode", ctypes.c_int32 * CDR_EW_MAX_INPUTS),
                ("out_reg", ctypes.c_int32 * CDR_EW_MAX_OUTPUTS), ("instr", CdrEwInstr * CDR_EW_MAX_INSTR)]


class CdrReduceParams(ctypes.Structure):
    _fields_ = [("chain", CdrEwParams), ("reduce_op", ctypes.c_int32), ("reserved", ctypes.c_int32)]


class CdrGemmParams(ctypes.Structure):
    _fields_ = [("activation", ctypes.c_int32), ("has_bias", ctypes.c_int32), ("weight_layout", ctypes.c_int32),
                ("x_layout", ctypes.c_int32), ("gate_input", ctypes.c_int32)]


class CdrNormParams(ctypes.Structure):
    _fields_ = [("eps", ctypes.c_float), ("has_weight", ctypes.c_int32), ("has_bias", ctypes.c_int32),
                ("reserved", ctypes.c_int32)]


class CdrAttnParams(ctypes.Structure):
    _fields_ = [("scale", ctypes.c_float), ("causal", ctypes.c_int32)]


class CdrLaunchItem(ctypes.Structure):
    """``cdr_launch_item``: the arguments of one ``cdr_launch`` call, for ``cdr_launch_many``."""

    _fields_ = [("template_id", ctypes.c_int32), ("n_inputs", ctypes.c_int32), ("n_outputs", ctypes.c_int32),
                ("reserved", ctypes.c_int32), ("inputs", ctypes.c_void_p), ("outputs", ctypes.c_void_p),
                ("params", ctypes.c_void_p), ("params_bytes", ctypes.c_size_t), ("workspace", ctypes.c_void_p),
                ("workspace_bytes", ctypes.c_size_t)]


# ---------------------------------------------------------------- launch description
@dataclass
class KernelLaunch:
    """One step of a compiled plan."""

    template: int                       # cdr_template id; 0 = alias (no kernel)
    name: str
    inputs: list[Buffer]
    outputs: list[Buffer]
    params: Any = None                  # ctypes struct or None
    out_shapes: list[tuple] = field(default_factory=list)
    out_dtypes: list[torch.dtype] = field(default_factory=list)
    alias_of: Optional[Buffer] = None   # SHAPE clusters: output is a view of this buffer
    cluster: Optional[FusionCluster] = None
    needs_workspace: bool = False
    view_strides: Optional[tuple] = None  # COPY launches: element strides of the view of inputs[0] that is gathered
    view_offset: int = 0                  # COPY launches: first element of that view, relative to inputs[0]'s own
    out_view: Optional[tuple] = None      # COPY launches that fill one part of outputs[0] (cat): (shape, strides, offset)
    # the executor's marshalled form of this launch (shape signature, descriptor arrays, parameter pointer):
    # built on first use, reused while shapes, strides and dtypes stay the same
    _marshal: Any = field(default=None, repr=False, compare=False)

    def describe(self) -> str:
        ins = ", ".join(b.name for b in self.inputs)
        outs = ", ".join(f"{b.name}:{b.scope.value}" for b in self.outputs)
        tname = {0: "alias", 1: "elementwise", 2: "row_reduce", 3: "softmax_fwd", 4: "softmax_bwd",
                 5: "gemm_epilogue", 6: "attention", 7: "full_reduce", 8: "layer_norm", 9: "copy", 10: "col_sum"}[self.template]
        return f"{outs} = {tname}<{self.name}>({ins})"


# ---------------------------------------------------------------- elementwise lowering
def _strip_ones(shape):
    s = list(shape)
    while s and s[0] == 1:
        s.pop(0)
    return tuple(s)


def classify_broadcast(in_shape, out_shape) -> int:
    """How an input of `in_shape` is indexed against the [rows, cols] view of `out_shape`."""
    n_in = math.prod(in_shape) if in_shape else 1
    n_out = math.prod(out_shape) if out_shape else 1
    if _strip_ones(in_shape) == _strip_ones(out_shape):
        return IN_FULL
    if n_in == 1:
        return IN_SCALAR
    if n_in == n_out:
        raise UnsupportedOperationError("broadcast", f"{in_shape} against {out_shape} needs a reshape")
    cols = out_shape[-1] if out_shape else 1
    if _strip_ones(in_shape) == (cols,):
        return IN_ROW
    aligned = (1,) * (len(out_shape) - len(in_shape)) + tuple(in_shape)
    if len(aligned) == len(out_shape) and aligned[-1] == 1 and aligned[:-1] == tuple(out_shape[:-1]):
        return IN_COL
    raise UnsupportedOperationError("broadcast", f"input {tuple(in_shape)} against output {tuple(out_shape)}")


_CAST_METHODS = {"float": torch.float32, "bfloat16": torch.bfloat16, "half": torch.float16}
_FLOAT_RANK = {torch.bfloat16: 1, torch.float16: 1, torch.float32: 2}


class _ProgramBuilder:
    """Turns the nodes of a cluster into a cdr_ew_params program."""

    def __init__(self, ext_inputs: list[Buffer], iter_shape):
        if len(ext_inputs) > CDR_EW_MAX_INPUTS:
            raise UnsupportedOperationError("elementwise", f"{len(ext_inputs)} inputs (max {CDR_EW_MAX_INPUTS})")
        self.inputs = list(ext_inputs)
        self.iter_shape = tuple(iter_shape)
        self.reg_of: dict[Buffer, int] = {b: i for i, b in enumerate(self.inputs)}
        self.instr: list[tuple] = []
        self.is_int = bool(self.inputs) and all(is_int(b.dtype) for b in self.inputs)
        self.shape_override: dict[Buffer, tuple] = {}   # inputs replaced by an expanded copy

    def _emit(self, op, a=0, b=0, c=0, imm=0.0, dtype=torch.float32) -> int:
        if len(self.instr) >= CDR_EW_MAX_INSTR:
            raise UnsupportedOperationError("elementwise", f"more than {CDR_EW_MAX_INSTR} instructions")
        self.instr.append((op, a, b, c, float(imm), to_cdr_dtype(dtype)))
        return len(self.inputs) + len(self.instr) - 1

    def _operand(self, node, spec, dtype) -> int:
        kind, val = spec
        if kind == "buf":
            return self.reg_of[node.inputs[val]]
        if kind == "const" and isinstance(val, (int, float, bool)):
            return self._emit(EwOp.CONST, imm=val, dtype=dtype)
        raise UnsupportedOperationError(node.op_name, f"operand {val!r} cannot be lowered")

    def _lower_composite(self, node, spec, kw, odt, is_num) -> int:
        """leaky_relu, elu, softplus, hardswish, hardsigmoid, masked_fill, lerp and inference-mode
        dropout as short sequences of existing opcodes.  Intermediates stay fp32 (never rounded to a
        16-bit output type); only the last instruction rounds, as eager's fused kernels do."""
        f32 = torch.float32
        name = node.op_name.rstrip("_")

        def num(pos, key, default):
            if key in kw:
                return kw[key]
            if len(spec) > pos:
                if not is_num(spec[pos]):
                    raise UnsupportedOperationError(node.op_name, f"{key} must be a Python number")
                return spec[pos][1]
            return default

        x = self._operand(node, spec[0], odt)
        const = lambda v: self._emit(EwOp.CONST, imm=v, dtype=f32)  # noqa: E731
        if name == "dropout":
            if num(2, "training", True) and num(1, "p", 0.5) != 0:
                raise UnsupportedOperationError(node.op_name, "training-mode dropout")
            return x
        if name == "leaky_relu":                              # max(x, 0) + slope * min(x, 0)
            slope = num(1, "negative_slope", 0.01)
            zero = const(0.0)
            neg = self._emit(EwOp.MUL_IMM, self._emit(EwOp.MIN, x, zero, dtype=f32), imm=slope, dtype=f32)
            return self._emit(EwOp.ADD, self._emit(EwOp.MAX, x, zero, dtype=f32), neg, dtype=odt)
        if name == "elu":                                     # x > 0 ? x : alpha * (exp(x) - 1)
            alpha = num(1, "alpha", 1.0)
            em1 = self._emit(EwOp.ADD_IMM, self._emit(EwOp.EXP, x, dtype=f32), imm=-1.0, dtype=f32)
            neg = self._emit(EwOp.MUL_IMM, em1, imm=alpha, dtype=f32)
            return self._emit(EwOp.WHERE, self._emit(EwOp.GT, x, const(0.0), dtype=f32), x, neg, dtype=odt)
        if name == "softplus":                                # beta*x > threshold ? x : log(1 + exp(beta*x)) / beta
            beta, threshold = num(1, "beta", 1.0), num(2, "threshold", 20.0)
            bx = self._emit(EwOp.MUL_IMM, x, imm=beta, dtype=f32)
            soft = self._emit(EwOp.LOG, self._emit(EwOp.ADD_IMM, self._emit(EwOp.EXP, bx, dtype=f32), imm=1.0, dtype=f32), dtype=f32)
            soft = self._emit(EwOp.MUL_IMM, soft, imm=1.0 / beta, dtype=f32)
            return self._emit(EwOp.WHERE, self._emit(EwOp.GT, bx, const(threshold), dtype=f32), x, soft, dtype=odt)
        if name in ("hardswish", "hardsigmoid"):              # clamp(x + 3, 0, 6) / 6 [* x]
            t = self._emit(EwOp.ADD_IMM, x, imm=3.0, dtype=f32)
            t = self._emit(EwOp.MIN, self._emit(EwOp.MAX, t, const(0.0), dtype=f32), const(6.0), dtype=f32)
            if name == "hardsigmoid":
                return self._emit(EwOp.MUL_IMM, t, imm=1.0 / 6.0, dtype=odt)
            return self._emit(EwOp.MUL_IMM, self._emit(EwOp.MUL, x, t, dtype=f32), imm=1.0 / 6.0, dtype=odt)
        if name == "masked_fill":                             # mask ? value : x
            if len(spec) < 3 or not is_num(spec[2]):
                raise UnsupportedOperationError(node.op_name, "the fill value must be a Python number")
            mask = self._operand(node, spec[1], odt)
            return self._emit(EwOp.WHERE, mask, self._emit(EwOp.CONST, imm=spec[2][1], dtype=odt), x, dtype=odt)
        if name == "lerp":                                    # x + w * (y - x)
            if len(spec) < 3:
                raise UnsupportedOperationError(node.op_name, "needs start, end and weight")
            y = self._operand(node, spec[1], odt)
            d = self._emit(EwOp.SUB, y, x, dtype=f32)
            if is_num(spec[2]):
                wd = self._emit(EwOp.MUL_IMM, d, imm=spec[2][1], dtype=f32)
            else:
                wd = self._emit(EwOp.MUL, self._operand(node, spec[2], odt), d, dtype=f32)
            return self._emit(EwOp.ADD, x, wd, dtype=odt)
        raise UnsupportedOperationError(node.op_name, "no lowering")

    def lower(self, node) -> None:
        info = get_op_desc(node.op_name)
        out = node.outputs[0]
        odt = out.dtype
        spec = list(node.metadata.get("arg_spec", []))
        kw = node.metadata.get("kwargs", {})
        kws = node.metadata.get("kwarg_spec", {})
        op = info.ew_op

        def is_buf(s):
            return s[0] == "buf"

        def is_num(s):
            return s[0] == "const" and isinstance(s[1], (int, float)) and not isinstance(s[1], bool)

        if op == EwOp.COPY:                                   # dtype cast
            src = self._operand(node, spec[0], odt)
            src_dt = node.inputs[spec[0][1]].dtype if is_buf(spec[0]) else odt
            widening = (src_dt == odt) or (is_float(src_dt) and is_float(odt)
                                          and _FLOAT_RANK[odt] > _FLOAT_RANK[src_dt])
            self.reg_of[out] = src if widening else self._emit(EwOp.COPY, src, dtype=odt)
            return
        canon = info.canonical_name
        if canon == "clamp":                                  # clamp / clip / hardtanh / relu6
            lo, hi = {"relu6": (0.0, 6.0), "hardtanh": (-1.0, 1.0)}.get(node.op_name, (None, None))
            nums = [s[1] if is_num(s) else None for s in spec[1:3]] + [None, None]
            if node.op_name.rstrip("_") == "clamp_max":      # clamp_max(x, hi): the one bound is the upper one
                nums = [None, nums[0]]
            lo = kw.get("min", kw.get("min_val", nums[0] if nums[0] is not None else lo))
            hi = kw.get("max", kw.get("max_val", nums[1] if nums[1] is not None else hi))
            if any(is_buf(s) for s in spec[1:]) or any(k[0] == "buf" for k in kws.values()):
                raise UnsupportedOperationError(node.op_name, "tensor bounds")
            r = self._operand(node, spec[0], odt)
            if lo is not None:
                r = self._emit(EwOp.MAX, r, self._emit(EwOp.CONST, imm=lo, dtype=odt), dtype=odt)
            if hi is not None:
                r = self._emit(EwOp.MIN, r, self._emit(EwOp.CONST, imm=hi, dtype=odt), dtype=odt)
            self.reg_of[out] = r
            return
        if canon == "composite":                              # activations written out over the opcode set
            self.reg_of[out] = self._lower_composite(node, spec, kw, odt, is_num)
            return
        if canon == "pow":                                    # pow / square / reciprocal
            x = self._operand(node, spec[0], odt)
            e = {"square": 2, "reciprocal": -1}.get(node.op_name)
            if e is None:
                if len(spec) < 2 or not is_num(spec[1]):
                    raise UnsupportedOperationError(node.op_name, "only constant exponents 2, 3, 0.5, -1, 1")
                e = spec[1][1]
            if e == 2:
                r = self._emit(EwOp.MUL, x, x, dtype=odt)
            elif e == 3:                                      # eager: (x*x)*x
                r = self._emit(EwOp.MUL, self._emit(EwOp.MUL, x, x, dtype=odt), x, dtype=odt)
            elif e == 0.5:
                r = self._emit(EwOp.SQRT, x, dtype=odt)
            elif e == -1:
                r = self._emit(EwOp.RDIV_IMM, x, imm=1.0, dtype=odt)
            elif e == 1:
                r = x
            else:
                raise UnsupportedOperationError(node.op_name, f"exponent {e!r}")
            self.reg_of[out] = r
            return
        if op in (EwOp.ADD, EwOp.SUB, EwOp.MUL, EwOp.DIV, EwOp.MAX, EwOp.MIN):
            if len(spec) < 2:
                raise UnsupportedOperationError(node.op_name, "needs two operands")
            alpha = kw.get("alpha", 1)
            if alpha != 1:
                raise UnsupportedOperationError(node.op_name, "alpha != 1")
            if kw.get("rounding_mode") is not None:
                raise UnsupportedOperationError(node.op_name, "rounding_mode")
            a, b = spec[0], spec[1]
            if is_buf(a) and is_num(b):
                ra = self._operand(node, a, odt)
                if op == EwOp.ADD:
                    r = self._emit(EwOp.ADD_IMM, ra, imm=b[1], dtype=odt)
                elif op == EwOp.SUB:
                    r = self._emit(EwOp.ADD_IMM, ra, imm=-b[1], dtype=odt)
                elif op == EwOp.MUL:
                    r = self._emit(EwOp.MUL_IMM, ra, imm=b[1], dtype=odt)
                else:
                    r = self._emit(op, ra, self._operand(node, b, odt), dtype=odt)
            elif is_num(a) and is_buf(b):
                rb = self._operand(node, b, odt)
                if op == EwOp.ADD:
                    r = self._emit(EwOp.ADD_IMM, rb, imm=a[1], dtype=odt)
                elif op == EwOp.MUL:
                    r = self._emit(EwOp.MUL_IMM, rb, imm=a[1], dtype=odt)
                elif op == EwOp.SUB:
                    r = self._emit(EwOp.RSUB_IMM, rb, imm=a[1], dtype=odt)
                elif op == EwOp.DIV:
                    r = self._emit(EwOp.RDIV_IMM, rb, imm=a[1], dtype=odt)
                else:
                    r = self._emit(op, self._operand(node, a, odt), rb, dtype=odt)
            else:
                r = self._emit(op, self._operand(node, a, odt), self._operand(node, b, odt), dtype=odt)
            self.reg_of[out] = r
            return
        if op in (EwOp.GT, EwOp.GE, EwOp.LT, EwOp.LE, EwOp.EQ, EwOp.NE):
            if len(spec) < 2:
                raise UnsupportedOperationError(node.op_name, "needs two operands")
            cdt = torch.float32                               # the 1.0 / 0.0 result is never rounded
            regs = [self._operand(node, s, cdt) for s in spec[:2]]
            self.reg_of[out] = self._emit(op, regs[0], regs[1], dtype=cdt)
            return
        if op == EwOp.WHERE:
            if len(spec) < 3:
                raise UnsupportedOperationError(node.op_name, "needs condition and two values")
            regs = [self._operand(node, s, odt) for s in spec[:3]]
            self.reg_of[out] = self._emit(op, regs[0], regs[1], regs[2], dtype=odt)
            return
        if op == EwOp.GELU and kw.get("approximate", "none") != "none":
            raise UnsupportedOperationError(node.op_name, "only the erf form of gelu")
        if op in (EwOp.ADDCDIV, EwOp.ADDCMUL):
            value = kw.get("value", 1)
            if len(spec) > 3 and spec[3][0] == "const":
                value = spec[3][1]
            regs = [self._operand(node, s, odt) for s in spec[:3]]
            self.reg_of[out] = self._emit(op, regs[0], regs[1], regs[2], imm=value, dtype=odt)
            return
        if info.arity == 1:                                   # unary math / relu
            self.reg_of[out] = self._emit(op, self._operand(node, spec[0], odt), dtype=odt)
            return
        raise UnsupportedOperationError(node.op_name, "no elementwise lowering")

    def build(self, out_regs: list[int]) -> CdrEwParams:
        p = CdrEwParams()
        p.n_inputs = len(self.inputs)
        p.n_instr = len(self.instr)
        p.n_outputs = len(out_regs)
        for i, b in enumerate(self.inputs):
            if b.shape is None:
                raise UnsupportedOperationError("elementwise", f"input {b.name} has no static shape")
            p.input_mode[i] = classify_broadcast(self.shape_override.get(b, b.shape), self.iter_shape)
        for i, r in enumerate(out_regs):
            p.out_reg[i] = r
        for i, (op, a, b, c, imm, rt) in enumerate(self.instr):
            p.instr[i] = CdrEwInstr(op, a, b, c, imm, rt)
        return p


def _require_shapes(cluster: FusionCluster) -> None:
    for b in cluster.external_inputs + cluster.external_outputs:
        if b.shape is None:
            raise UnsupportedOperationError(cluster.signature(), f"buffer {b.name} has no static shape")


def _expand_general_broadcasts(inputs, iter_shape, cluster: FusionCluster):
    """The elementwise kernels index an input as full-size, one row, one column or a scalar.  Any
    other broadcast (a middle dimension of 1, a missing leading batch dimension) is materialised
    first: one strided copy of the input's expand() view, whose broadcast dimensions have stride 0.
    Returns the launches to run first and the input list with those inputs replaced."""
    pre, replaced = [], []
    for b in inputs:
        try:
            classify_broadcast(b.shape, iter_shape)
            replaced.append(b)
            continue
        except UnsupportedOperationError as exc:
            try:
                view = torch.empty(b.shape, dtype=b.dtype, device="meta").expand(tuple(iter_shape))
            except Exception:
                raise exc from None
        done = getattr(b, "_expanded", None)
        if done is None:
            done = b._expanded = {}
        if tuple(iter_shape) in done:               # an earlier cluster of this plan already expanded it
            replaced.append(done[tuple(iter_shape)])
            continue
        full = done[tuple(iter_shape)] = Buffer(name=f"{b.name}_expanded", scope=BufferScope.SHARED, dtype=b.dtype,
                                                shape=tuple(iter_shape), is_temporary=True)
        pre.append(KernelLaunch(Template.COPY, f"{cluster.signature()}:expand", [b], [full], None, [full.shape],
                                [full.dtype], cluster=cluster, view_strides=tuple(view.stride())))
        replaced.append(full)
    return pre, replaced


def _lower_elementwise(cluster: FusionCluster):
    _require_shapes(cluster)
    outs = cluster.external_outputs
    if not outs or len(outs) > CDR_EW_MAX_OUTPUTS:
        raise UnsupportedOperationError(cluster.signature(), f"{len(outs)} outputs")
    iter_shape = outs[0].shape
    for b in outs:
        if b.shape != iter_shape:
            raise UnsupportedOperationError(cluster.signature(), "outputs of different shapes")
    pre, launch_inputs = _expand_general_broadcasts(cluster.external_inputs, iter_shape, cluster)
    builder = _ProgramBuilder(cluster.external_inputs, iter_shape)
    builder.shape_override = {b: r.shape for b, r in zip(cluster.external_inputs, launch_inputs) if r is not b}
    for node in cluster._topological_sort():
        if node.outputs[0].shape != iter_shape:
            raise UnsupportedOperationError(cluster.signature(), "intermediate of a different shape")
        builder.lower(node)
    out_regs = [builder.reg_of[b] for b in outs]
    for i, (b, r) in enumerate(zip(outs, out_regs)):
        if r < len(builder.inputs):         # output is a pure alias of an input: materialise a copy
            out_regs[i] = builder._emit(EwOp.COPY, r, dtype=b.dtype)
    params = builder.build(out_regs)
    launch = KernelLaunch(Template.ELEMENTWISE, cluster.signature(), list(launch_inputs), list(outs),
                          params, [b.shape for b in outs], [b.dtype for b in outs], cluster=cluster)
    return pre + [launch] if pre else launch


def _lower_reduction(cluster: FusionCluster) -> KernelLaunch:
    _require_shapes(cluster)
    order = cluster._topological_sort()
    red = [n for n in order if n.is_reduction()]
    if len(red) != 1 or order[-1] is not red[0]:
        raise UnsupportedOperationError(cluster.signature(), "expected a chain ending in one reduction")
    red = red[0]
    last = _is_last_dim_reduction(red)
    if last is False:
        if len(order) != 1:
            raise UnsupportedOperationError(red.op_name, "a fused chain in front of a reduction over inner dimensions")
        return _lower_inner_reduction(cluster, red)
    full_shape = red.inputs[0].shape
    if not full_shape:
        raise UnsupportedOperationError(red.op_name, "rank-0 input")
    builder = _ProgramBuilder(cluster.external_inputs, full_shape)
    for node in order[:-1]:
        builder.lower(node)
    src = builder.reg_of[red.inputs[0]]
    if not any(classify_broadcast(b.shape, full_shape) == IN_FULL for b in cluster.external_inputs):
        raise UnsupportedOperationError(cluster.signature(), "no full-size input")
    out = red.outputs[0]
    if not is_float(out.dtype):
        raise UnsupportedOperationError(red.op_name, f"{out.dtype} reduction")
    p = CdrReduceParams()
    p.chain = builder.build([src])
    p.reduce_op = get_op_desc(red.op_name).reduce_op
    template = Template.FULL_REDUCE if last is None else Template.ROW_REDUCE
    return KernelLaunch(template, cluster.signature(), list(cluster.external_inputs), [out], p, [out.shape],
                        [out.dtype], cluster=cluster, needs_workspace=template == Template.FULL_REDUCE)


def _lower_inner_reduction(cluster: FusionCluster, red) -> list:
    """sum / mean / amax / amin over dimensions other than the last: the reduced dimensions are moved
    behind the kept ones with one strided copy (skipped when they already trail), the result is
    seen as [kept, reduced] and goes through the row-reduce template."""
    src, out = red.inputs[0], red.outputs[0]
    rank = len(src.shape)
    kw = red.metadata.get("kwargs", {})
    consts = _const_args(red)
    dim = kw.get("dim", consts[0] if consts else None)
    dims = [dim] if isinstance(dim, int) else list(dim or [])
    if not dims or not all(isinstance(d, int) and -rank <= d < rank for d in dims):
        raise UnsupportedOperationError(red.op_name, f"dim={dim!r}")
    dims = sorted({d % rank for d in dims})
    if not is_float(out.dtype) or not is_float(src.dtype):
        raise UnsupportedOperationError(red.op_name, f"{src.dtype} reduction")
    keep = [d for d in range(rank) if d not in dims]
    view = torch.empty(src.shape, dtype=src.dtype, device="meta").permute(keep + dims)
    n_keep = math.prod(src.shape[d] for d in keep)
    n_red = math.prod(src.shape[d] for d in dims)
    if n_red == 0 or n_keep == 0:
        raise UnsupportedOperationError(red.op_name, "empty reduction")
    sig = cluster.signature()
    launches, cur = [], src
    if not view.is_contiguous():
        moved = Buffer(name=f"{out.name}_moved", scope=BufferScope.SHARED, dtype=src.dtype, shape=tuple(view.shape),
                       is_temporary=True)
        launches.append(KernelLaunch(Template.COPY, f"{sig}:move", [src], [moved], None, [moved.shape], [moved.dtype],
                                     cluster=cluster, view_strides=tuple(view.stride())))
        cur = moved
    flat = Buffer(name=f"{out.name}_rows", scope=BufferScope.SHARED, dtype=src.dtype, shape=(n_keep, n_red),
                  is_temporary=True)
    launches.append(KernelLaunch(0, f"{sig}:rows", [cur], [flat], None, [flat.shape], [flat.dtype], alias_of=cur,
                                 cluster=cluster))
    p = CdrReduceParams()
    p.chain = _ProgramBuilder([flat], flat.shape).build([0])
    p.reduce_op = get_op_desc(red.op_name).reduce_op
    launches.append(KernelLaunch(Template.ROW_REDUCE, sig, [flat], [out], p, [out.shape], [out.dtype], cluster=cluster))
    return launches


def _const_args(node):
    return [v for k, v in node.metadata.get("arg_spec", []) if k == "const"]


def _lower_softmax(cluster: FusionCluster) -> KernelLaunch:
    _require_shapes(cluster)
    if cluster.pattern == "softmax_bwd_written_out":
        roles = cluster.nodes[0].metadata["softmax_bwd_roles"]
        out = cluster.external_outputs[0]
        return KernelLaunch(Template.SOFTMAX_BWD, cluster.signature(), [roles["grad"], roles["y"]], [out], None,
                            [out.shape], [out.dtype], cluster=cluster)
    node = cluster.nodes[0]
    kw = node.metadata.get("kwargs", {})
    consts = _const_args(node)
    out = node.outputs[0]
    if node.op_name == "softmax":
        x = node.inputs[0]
        dim = kw.get("dim", consts[0] if consts else None)
        dtype = kw.get("dtype", consts[2] if len(consts) > 2 else None)
        if not isinstance(dim, int) or not x.shape:
            raise UnsupportedOperationError("softmax", f"dim={dim!r}")
        if dtype is not None and dtype != x.dtype:
            raise UnsupportedOperationError("softmax", "dtype conversion inside softmax")
        if kw.get("_half_to_float", consts[1] if len(consts) > 1 and isinstance(consts[1], bool) else False):
            raise UnsupportedOperationError("softmax", "half_to_float")
        d, rank = dim % len(x.shape), len(x.shape)
        if d != rank - 1:
            # softmax over an inner dimension: swap it with the last one by a strided copy, run the
            # row kernel, swap back
            sig = cluster.signature()
            fwd = torch.empty(x.shape, dtype=x.dtype, device="meta").transpose(d, -1)
            moved = Buffer(name=f"{out.name}_moved", scope=BufferScope.SHARED, dtype=x.dtype, shape=tuple(fwd.shape),
                           is_temporary=True)
            rows = Buffer(name=f"{out.name}_rows", scope=BufferScope.SHARED, dtype=x.dtype, shape=tuple(fwd.shape),
                          is_temporary=True)
            back = torch.empty(fwd.shape, dtype=x.dtype, device="meta").transpose(d, -1)
            return [KernelLaunch(Template.COPY, f"{sig}:move", [x], [moved], None, [moved.shape], [x.dtype],
                                 cluster=cluster, view_strides=tuple(fwd.stride())),
                    KernelLaunch(Template.SOFTMAX_FWD, sig, [moved], [rows], None, [rows.shape], [x.dtype], cluster=cluster),
                    KernelLaunch(Template.COPY, f"{sig}:restore", [rows], [out], None, [out.shape], [out.dtype],
                                 cluster=cluster, view_strides=tuple(back.stride()))]
        return KernelLaunch(Template.SOFTMAX_FWD, cluster.signature(), [x], [out], None, [out.shape], [out.dtype],
                            cluster=cluster)
    if node.op_name == "_softmax_backward_data":
        g, y = node.inputs[0], node.inputs[1]
        dim = kw.get("dim", consts[0] if consts else None)
        if dim is None or (dim % len(y.shape)) != len(y.shape) - 1:
            raise UnsupportedOperationError("_softmax_backward_data", f"dim={dim}")
        return KernelLaunch(Template.SOFTMAX_BWD, cluster.signature(), [g, y], [out], None, [out.shape], [out.dtype],
                            cluster=cluster)
    raise UnsupportedOperationError(node.op_name, "not a softmax operation")


W_NK, W_KN = 0, 1   # cdr_weight_layout


def _lower_gemm(cluster: FusionCluster) -> KernelLaunch:
    """linear(x, W[N,K][, b]) -> out = x @ W^T (+ b); matmul / mm(x, W[K,N]) -> out = x @ W with the
    weight read in place as an MN-major operand.  A following relu joins as the epilogue."""
    _require_shapes(cluster)
    node = cluster.nodes[0]
    spec = node.metadata.get("arg_spec", [])
    kws = node.metadata.get("kwarg_spec", {})
    ops = [s for s in spec if s[0] == "buf"]
    if node.op_name == "linear":
        if "bias" in kws and kws["bias"][0] == "buf":
            ops.append(kws["bias"])
        bufs = [node.inputs[s[1]] for s in ops]
        if len(bufs) not in (2, 3):
            raise UnsupportedOperationError("linear", "expected (x, weight[, bias])")
        x, w = bufs[0], bufs[1]
        if len(w.shape) != 2 or x.shape[-1] != w.shape[1]:
            raise UnsupportedOperationError("linear", f"shapes {x.shape} x {w.shape}")
        layout = W_NK
    elif get_op_desc(node.op_name).canonical_name == "matmul":
        bufs = [node.inputs[s[1]] for s in ops]
        if len(bufs) != 2:
            raise UnsupportedOperationError(node.op_name, "expected two tensor operands")
        x, w = bufs
        if len(w.shape) != 2 or len(x.shape) < 2 or x.shape[-1] != w.shape[0]:
            raise UnsupportedOperationError(node.op_name, f"shapes {x.shape} x {w.shape}: the right operand must be 2-D")
        layout = W_KN
    elif node.op_name == "addmm":                             # addmm(bias[N], x[M,K], W[K,N]) = bias + x @ W
        kw = node.metadata.get("kwargs", {})
        if len(ops) != 3 or len(spec) != 3 or kw.get("beta", 1) != 1 or kw.get("alpha", 1) != 1:
            raise UnsupportedOperationError("addmm", "expected (bias, x, weight) with beta = alpha = 1")
        bias, x, w = (node.inputs[s[1]] for s in ops)
        if len(w.shape) != 2 or len(x.shape) != 2 or x.shape[-1] != w.shape[0] or _strip_ones(bias.shape) != (w.shape[1],):
            raise UnsupportedOperationError("addmm", f"shapes {bias.shape} + {x.shape} x {w.shape}: the addend must be one row")
        bufs = [x, w, bias]
        layout = W_KN
    else:
        raise UnsupportedOperationError(node.op_name, "no GEMM lowering")
    act = 0
    if len(cluster.nodes) == 2:
        if cluster.nodes[1].op_name != "relu":
            raise UnsupportedOperationError(cluster.signature(), "unsupported epilogue")
        act = 1
    out = cluster.external_outputs[0]
    p = CdrGemmParams(act, 1 if len(bufs) == 3 else 0, layout, 0)
    return KernelLaunch(Template.GEMM_EPILOGUE, cluster.signature(), bufs, [out], p, [out.shape], [out.dtype],
                        cluster=cluster)


def _lower_attention(cluster: FusionCluster) -> KernelLaunch:
    _require_shapes(cluster)
    node = cluster.nodes[0]
    kw = node.metadata.get("kwargs", {})
    kws = node.metadata.get("kwarg_spec", {})
    spec = node.metadata.get("arg_spec", [])
    bufs = [node.inputs[s[1]] for s in spec if s[0] == "buf"]
    if len(bufs) != 3 or any(v[0] == "buf" for v in kws.values()):
        raise UnsupportedOperationError("scaled_dot_product_attention", "attn_mask tensors are not supported")
    consts = _const_args(node)
    if kw.get("attn_mask") is not None or (consts and consts[0] is not None):
        raise UnsupportedOperationError("scaled_dot_product_attention", "attn_mask")
    dropout = kw.get("dropout_p", consts[1] if len(consts) > 1 else 0.0)
    if dropout:
        raise UnsupportedOperationError("scaled_dot_product_attention", "dropout")
    if kw.get("enable_gqa"):
        raise UnsupportedOperationError("scaled_dot_product_attention", "enable_gqa")
    causal = bool(kw.get("is_causal", consts[2] if len(consts) > 2 else False))
    q = bufs[0]
    scale = kw.get("scale", consts[3] if len(consts) > 3 else None)
    if scale is None:
        scale = 1.0 / math.sqrt(q.shape[-1])
    out = node.outputs[0]
    p = CdrAttnParams(float(scale), 1 if causal else 0)
    return KernelLaunch(Template.ATTENTION, cluster.signature(), bufs, [out], p, [out.shape], [out.dtype],
                        cluster=cluster, needs_workspace=True)


def _lower_cat(cluster: FusionCluster) -> list:
    """cat / concat: one strided copy per part, each writing its slice of the result."""
    node = cluster.nodes[0]
    out = node.outputs[0]
    spec = node.metadata.get("arg_spec", [])
    kw = node.metadata.get("kwargs", {})
    if not spec or spec[0][0] != "seq" or any(s[0] != "buf" for s in spec[0][1]):
        raise UnsupportedOperationError(node.op_name, "expected a sequence of tensors")
    parts = [node.inputs[s[1]] for s in spec[0][1]]
    consts = _const_args(node)
    dim = kw.get("dim", consts[0] if consts else 0)
    rank = len(out.shape)
    if not isinstance(dim, int) or any(p.shape is None or len(p.shape) != rank or p.dtype != out.dtype for p in parts):
        raise UnsupportedOperationError(node.op_name, "parts must share rank and dtype")
    dim %= rank
    full = torch.empty(out.shape, dtype=out.dtype, device="meta")
    launches, start = [], 0
    for i, part in enumerate(parts):
        n = part.shape[dim]
        if n == 0:
            continue
        view = full.narrow(dim, start, n)
        if tuple(view.shape) != tuple(part.shape):
            raise UnsupportedOperationError(node.op_name, f"part {i} has shape {part.shape}")
        launches.append(KernelLaunch(Template.COPY, f"{cluster.signature()}:part{i}", [part], [out], None, [out.shape],
                                     [out.dtype], cluster=cluster,
                                     out_view=(tuple(view.shape), tuple(view.stride()), int(view.storage_offset()))))
        start += n
    if start != out.shape[dim] or not launches:
        raise UnsupportedOperationError(node.op_name, "parts do not cover the result")
    return launches


def _lower_shape(cluster: FusionCluster):
    node = cluster.nodes[0]
    out = node.outputs[0]
    if node.op_name in ("cat", "concat", "concatenate"):
        return _lower_cat(cluster)
    if out.shape is None or not node.inputs:
        raise UnsupportedOperationError(node.op_name, "unknown output shape")
    src = node.inputs[0]
    info = get_op_desc(node.op_name)
    canonical = info.canonical_name if info is not None else None
    if canonical != "slice" and src.shape is not None and math.prod(src.shape) != math.prod(out.shape):
        raise UnsupportedOperationError(node.op_name, "element count changes")
    # A value that is itself a view of an earlier buffer (a slice, a transposed view, a reshape of
    # one) carries that view's description; a layout change applied to it is composed with it and
    # gathers straight from the earlier buffer, so slice -> view -> transpose costs one copy.  The
    # intermediate launches stay in the list and are dropped later if nothing else reads them.
    base, base_view = getattr(src, "_view_of", None) or (src, None)

    def meta_of_src():
        m = torch.empty(base.shape, dtype=base.dtype, device="meta")
        return m if base_view is None else m.as_strided(*base_view)

    if canonical in ("permute", "slice"):
        # transpose / permute / t / swapaxes / movedim, and basic slicing (x[a:b, ::2], narrow,
        # select, members of chunk / split / unbind, expand): replay the call on a meta tensor to
        # get the view's strides and first element, then gather that view into a contiguous buffer
        # (every buffer of a plan is contiguous, so the layout change has to move data)
        if src.shape is None:
            raise UnsupportedOperationError(node.op_name, "unknown input shape")
        if len(node.inputs) != 1 and node.op_name != "expand_as":
            raise UnsupportedOperationError(node.op_name, "indexing by a tensor")
        try:
            meta = meta_of_src()
            consts = _const_args(node)
            if node.op_name == "expand_as":      # the second tensor only gives the shape
                view = meta.expand(tuple(out.shape))
            elif "view_call" in node.metadata:     # one member of chunk / split / unbind
                method, m_args, m_kwargs, index = node.metadata["view_call"]
                view = getattr(meta, method)(*m_args, **m_kwargs)[index]
            elif node.op_name in ("getitem", "__getitem__"):
                view = meta[consts[0]]
            else:
                view = getattr(meta, node.op_name)(*consts, **node.metadata.get("kwargs", {}))
        except Exception as exc:
            raise UnsupportedOperationError(node.op_name, f"cannot evaluate the layout change: {exc}") from exc
        if not isinstance(view, torch.Tensor):
            raise UnsupportedOperationError(node.op_name, "the call returns several views")
        if tuple(view.shape) != tuple(out.shape):
            raise UnsupportedOperationError(node.op_name, f"shape {tuple(view.shape)} != {tuple(out.shape)}")
        if view.is_contiguous() and view.storage_offset() == 0 and view.numel() == math.prod(base.shape):
            return KernelLaunch(0, cluster.signature(), [base], [out], None, [out.shape], [out.dtype], alias_of=base,
                                cluster=cluster)
        out._view_of = (base, (tuple(view.shape), tuple(view.stride()), int(view.storage_offset())))
        return KernelLaunch(Template.COPY, cluster.signature(), [base], [out], None, [out.shape], [out.dtype],
                            cluster=cluster, view_strides=tuple(view.stride()), view_offset=int(view.storage_offset()))
    if base_view is not None:                    # reshape of a view: keep the description when it stays a view
        try:
            view = meta_of_src().view(tuple(out.shape))
            out._view_of = (base, (tuple(view.shape), tuple(view.stride()), int(view.storage_offset())))
        except Exception:
            pass
    return KernelLaunch(0, cluster.signature(), [src], [out], None, [out.shape], [out.dtype], alias_of=src,
                        cluster=cluster)


def prune_dead_launches(launches: list) -> list:
    """Drop launches whose outputs nothing reads (left behind when a later layout change was
    composed with the view they materialised).  A launch is kept when one of its outputs is a
    result of the graph or an input of a kept launch."""
    needed: set = set()
    kept = []
    for launch in reversed(launches):
        if any(b.is_output or b in needed for b in launch.outputs):
            kept.append(launch)
            needed.update(launch.inputs)
    return kept[::-1]


def _lower_layer_norm(cluster: FusionCluster) -> list:
    """layer_norm over the last dimension: the fused one-pass template when a row is a whole number
    of 16-byte vectors, fits in registers and everything has one dtype; otherwise three launches of
    existing templates: row mean, row variance (mean of squared deviations, two-pass) and the
    normalising elementwise chain with the two statistics as column-broadcast inputs.  Statistics
    are fp32 either way; the result is rounded once to the output dtype, like eager's kernel."""
    _require_shapes(cluster)
    node = cluster.nodes[0]
    spec = node.metadata.get("arg_spec", [])
    kw = node.metadata.get("kwargs", {})
    kws = node.metadata.get("kwarg_spec", {})
    consts = _const_args(node)
    x = node.inputs[spec[0][1]]
    out = node.outputs[0]
    norm_shape = kw.get("normalized_shape", consts[0] if consts else None)
    if norm_shape is None or len(tuple(norm_shape)) != 1 or tuple(norm_shape)[0] != x.shape[-1]:
        raise UnsupportedOperationError("layer_norm", f"normalized_shape={norm_shape}; only the last dimension")
    if not is_float(x.dtype):
        raise UnsupportedOperationError("layer_norm", f"{x.dtype} input")

    def operand(pos, name):
        if name in kws and kws[name][0] == "buf":
            return node.inputs[kws[name][1]]
        if len(spec) > pos and spec[pos][0] == "buf":
            return node.inputs[spec[pos][1]]
        return None

    w, b = operand(2, "weight"), operand(3, "bias")
    eps = kw.get("eps", next((c for c in consts[1:] if isinstance(c, float)), 1e-5))
    # rows that are whole 16-byte vectors and fit in registers, one dtype throughout: the fused kernel
    cols = x.shape[-1]
    per_vec = 16 // (4 if x.dtype == torch.float32 else 2)
    if (cols % per_vec == 0 and cols <= 16384 and out.dtype == x.dtype
            and all(t is None or (t.dtype == x.dtype and tuple(t.shape) == (cols,)) for t in (w, b))):
        p = CdrNormParams(float(eps), 1 if w is not None else 0, 1 if b is not None else 0, 0)
        return [KernelLaunch(Template.LAYER_NORM, cluster.signature(), [x] + [t for t in (w, b) if t is not None], [out], p,
                             [out.shape], [out.dtype], cluster=cluster)]
    f32 = torch.float32
    stat_shape = tuple(x.shape[:-1]) + (1,)
    mean = Buffer(name=f"{out.name}_mean", scope=BufferScope.SHARED, dtype=f32, shape=stat_shape, is_temporary=True)
    var = Buffer(name=f"{out.name}_var", scope=BufferScope.SHARED, dtype=f32, shape=stat_shape, is_temporary=True)
    sig = cluster.signature()

    p1 = CdrReduceParams()
    p1.chain = _ProgramBuilder([x], x.shape).build([0])
    p1.reduce_op = ReduceOp.MEAN
    l1 = KernelLaunch(Template.ROW_REDUCE, f"{sig}:mean", [x], [mean], p1, [stat_shape], [f32], cluster=cluster)

    b2 = _ProgramBuilder([x, mean], x.shape)
    d = b2._emit(EwOp.SUB, 0, 1, dtype=f32)
    sq = b2._emit(EwOp.MUL, d, d, dtype=f32)
    p2 = CdrReduceParams()
    p2.chain = b2.build([sq])
    p2.reduce_op = ReduceOp.MEAN
    l2 = KernelLaunch(Template.ROW_REDUCE, f"{sig}:var", [x, mean], [var], p2, [stat_shape], [f32], cluster=cluster)

    ins = [x, mean, var] + [t for t in (w, b) if t is not None]
    b3 = _ProgramBuilder(ins, x.shape)
    d = b3._emit(EwOp.SUB, 0, 1, dtype=f32)
    r = b3._emit(EwOp.RSQRT, b3._emit(EwOp.ADD_IMM, 2, imm=eps, dtype=f32), dtype=f32)
    y = b3._emit(EwOp.MUL, d, r, dtype=f32 if (w is not None or b is not None) else out.dtype)
    nxt = 3
    if w is not None:
        y = b3._emit(EwOp.MUL, y, nxt, dtype=f32 if b is not None else out.dtype)
        nxt += 1
    if b is not None:
        y = b3._emit(EwOp.ADD, y, nxt, dtype=out.dtype)
    l3 = KernelLaunch(Template.ELEMENTWISE, f"{sig}:normalize", ins, [out], b3.build([y]), [out.shape], [out.dtype],
                      cluster=cluster)
    return [l1, l2, l3]


def _row_statistic(cluster, tag, inputs, reduce_op, emit_chain):
    """One ROW_REDUCE launch over inputs[0]'s rows into a fresh fp32 [.., 1] buffer; `emit_chain`
    gets the program builder and returns the register to reduce."""
    x = inputs[0]
    stat_shape = tuple(x.shape[:-1]) + (1,)
    out = Buffer(name=f"{cluster.nodes[0].outputs[0].name}_{tag}", scope=BufferScope.SHARED, dtype=torch.float32,
                 shape=stat_shape, is_temporary=True)
    b = _ProgramBuilder(inputs, x.shape)
    p = CdrReduceParams()
    p.chain = b.build([emit_chain(b)])
    p.reduce_op = reduce_op
    return out, KernelLaunch(Template.ROW_REDUCE, f"{cluster.signature()}:{tag}", list(inputs), [out], p, [stat_shape],
                             [torch.float32], cluster=cluster)


def _last_dim_only(node, x, pos=1):
    kw = node.metadata.get("kwargs", {})
    consts = _const_args(node)
    dim = kw.get("dim", consts[pos - 1] if len(consts) >= pos else None)
    if isinstance(dim, (list, tuple)) and len(dim) == 1:
        dim = dim[0]
    if not isinstance(dim, int) or dim % len(x.shape) != len(x.shape) - 1:
        raise UnsupportedOperationError(node.op_name, f"dim={dim!r}; only the last dimension is supported")
    return kw, consts


def _lower_rms_norm(cluster: FusionCluster) -> list:
    """rms_norm over the last dimension: mean(x^2) per row in fp32, then x * rsqrt(ms + eps) [* w]
    with one rounding to the output dtype."""
    _require_shapes(cluster)
    node = cluster.nodes[0]
    spec = node.metadata.get("arg_spec", [])
    kw = node.metadata.get("kwargs", {})
    kws = node.metadata.get("kwarg_spec", {})
    consts = _const_args(node)
    x, out = node.inputs[spec[0][1]], node.outputs[0]
    norm_shape = kw.get("normalized_shape", consts[0] if consts else None)
    if norm_shape is None or tuple(norm_shape) != (x.shape[-1],) or not is_float(x.dtype):
        raise UnsupportedOperationError("rms_norm", f"normalized_shape={norm_shape}; only the last dimension of a float tensor")
    w = None
    if "weight" in kws and kws["weight"][0] == "buf":
        w = node.inputs[kws["weight"][1]]
    elif len(spec) > 2 and spec[2][0] == "buf":
        w = node.inputs[spec[2][1]]
    eps = kw.get("eps", next((c for c in consts[1:] if isinstance(c, float)), None))
    if eps is None:
        eps = torch.finfo(x.dtype).eps
    f32 = torch.float32
    ms, l1 = _row_statistic(cluster, "meansq", [x], ReduceOp.MEAN, lambda b: b._emit(EwOp.MUL, 0, 0, dtype=f32))
    ins = [x, ms] + ([w] if w is not None else [])
    b2 = _ProgramBuilder(ins, x.shape)
    r = b2._emit(EwOp.RSQRT, b2._emit(EwOp.ADD_IMM, 1, imm=eps, dtype=f32), dtype=f32)
    y = b2._emit(EwOp.MUL, 0, r, dtype=f32 if w is not None else out.dtype)
    if w is not None:
        y = b2._emit(EwOp.MUL, y, 2, dtype=out.dtype)
    l2 = KernelLaunch(Template.ELEMENTWISE, f"{cluster.signature()}:normalize", ins, [out], b2.build([y]), [out.shape],
                      [out.dtype], cluster=cluster)
    return [l1, l2]


def _lower_log_softmax(cluster: FusionCluster) -> list:
    """log_softmax / logsumexp over the last dimension in the stable form: row maximum m, then
    s = sum(exp(x - m)), then x - m - log(s) (or m + log(s)); statistics in fp32."""
    _require_shapes(cluster)
    node = cluster.nodes[0]
    spec = node.metadata.get("arg_spec", [])
    x, out = node.inputs[spec[0][1]], node.outputs[0]
    if not is_float(x.dtype) or not x.shape:
        raise UnsupportedOperationError(node.op_name, f"{x.dtype} input")
    _last_dim_only(node, x)
    f32 = torch.float32
    m, l1 = _row_statistic(cluster, "max", [x], ReduceOp.MAX, lambda b: 0)
    ssum, l2 = _row_statistic(cluster, "sumexp", [x, m], ReduceOp.SUM,
                              lambda b: b._emit(EwOp.EXP, b._emit(EwOp.SUB, 0, 1, dtype=f32), dtype=f32))
    if node.op_name == "logsumexp":
        b3 = _ProgramBuilder([m, ssum], m.shape)
        y = b3._emit(EwOp.ADD, 0, b3._emit(EwOp.LOG, 1, dtype=f32), dtype=out.dtype)
        ins = [m, ssum]
    else:
        b3 = _ProgramBuilder([x, m, ssum], x.shape)
        y = b3._emit(EwOp.SUB, b3._emit(EwOp.SUB, 0, 1, dtype=f32), b3._emit(EwOp.LOG, 2, dtype=f32), dtype=out.dtype)
        ins = [x, m, ssum]
    l3 = KernelLaunch(Template.ELEMENTWISE, f"{cluster.signature()}:finish", ins, [out], b3.build([y]), [out.shape],
                      [out.dtype], cluster=cluster)
    return [l1, l2, l3]


def _lower_variance(cluster: FusionCluster) -> list:
    """var / std over the last dimension, two-pass: row mean, then the mean of squared deviations
    scaled by n / (n - correction) (and its square root for std)."""
    _require_shapes(cluster)
    node = cluster.nodes[0]
    spec = node.metadata.get("arg_spec", [])
    x, out = node.inputs[spec[0][1]], node.outputs[0]
    if not is_float(x.dtype) or not x.shape:
        raise UnsupportedOperationError(node.op_name, f"{x.dtype} input")
    kw, consts = _last_dim_only(node, x)
    correction = kw.get("correction", None)
    if correction is None:
        unbiased = kw.get("unbiased", next((c for c in consts[1:] if isinstance(c, bool)), True))
        correction = 1 if unbiased else 0
    n = x.shape[-1]
    if n - correction <= 0:
        raise UnsupportedOperationError(node.op_name, "rows too short for the correction")
    f32 = torch.float32
    mean, l1 = _row_statistic(cluster, "mean", [x], ReduceOp.MEAN, lambda b: 0)

    def sq_dev(b):
        d = b._emit(EwOp.SUB, 0, 1, dtype=f32)
        return b._emit(EwOp.MUL, d, d, dtype=f32)

    ssq, l2 = _row_statistic(cluster, "sumsq", [x, mean], ReduceOp.SUM, sq_dev)
    b3 = _ProgramBuilder([ssq], ssq.shape)
    is_std = node.op_name == "std"
    y = b3._emit(EwOp.MUL_IMM, 0, imm=1.0 / (n - correction), dtype=f32 if is_std else out.dtype)
    if is_std:
        y = b3._emit(EwOp.SQRT, y, dtype=out.dtype)
    l3 = KernelLaunch(Template.ELEMENTWISE, f"{cluster.signature()}:finish", [ssq], [out], b3.build([y]), [out.shape],
                      [out.dtype], cluster=cluster)
    return [l1, l2, l3]


def _lower_pointwise_loss(cluster: FusionCluster) -> list:
    """mse_loss / l1_loss: the chain (x - y)^2 or |x - y| in fp32 in front of a mean or sum over
    everything (one full-reduce launch), or on its own for reduction='none'."""
    _require_shapes(cluster)
    node = cluster.nodes[0]
    spec = node.metadata.get("arg_spec", [])
    kw = node.metadata.get("kwargs", {})
    if len(spec) < 2 or spec[0][0] != "buf" or spec[1][0] != "buf":
        raise UnsupportedOperationError(node.op_name, "expected (input, target)")
    x, y, out = node.inputs[spec[0][1]], node.inputs[spec[1][1]], node.outputs[0]
    consts = _const_args(node)
    reduction = kw.get("reduction", next((c for c in consts if isinstance(c, str)), "mean"))
    if tuple(x.shape) != tuple(y.shape) or not is_float(x.dtype) or reduction not in ("mean", "sum", "none"):
        raise UnsupportedOperationError(node.op_name, f"shapes {x.shape} / {y.shape}, reduction={reduction!r}")
    f32 = torch.float32
    last_dt = out.dtype if reduction == "none" else f32
    b = _ProgramBuilder([x, y], x.shape)
    d = b._emit(EwOp.SUB, 0, 1, dtype=f32)
    r = b._emit(EwOp.MUL, d, d, dtype=last_dt) if node.op_name == "mse_loss" else b._emit(EwOp.ABS, d, dtype=last_dt)
    if reduction == "none":
        return [KernelLaunch(Template.ELEMENTWISE, cluster.signature(), [x, y], [out], b.build([r]), [out.shape],
                             [out.dtype], cluster=cluster)]
    p = CdrReduceParams()
    p.chain = b.build([r])
    p.reduce_op = ReduceOp.MEAN if reduction == "mean" else ReduceOp.SUM
    return [KernelLaunch(Template.FULL_REDUCE, cluster.signature(), [x, y], [out], p, [out.shape], [out.dtype],
                         cluster=cluster, needs_workspace=True)]


def _lower_vector_norm(cluster: FusionCluster) -> list:
    """x.norm(dim=-1) / linalg.vector_norm with p = 2 over the last dimension: fp32 row sum of squares,
    then its square root."""
    _require_shapes(cluster)
    node = cluster.nodes[0]
    spec = node.metadata.get("arg_spec", [])
    kw = node.metadata.get("kwargs", {})
    x, out = node.inputs[spec[0][1]], node.outputs[0]
    consts = _const_args(node)
    p = kw.get("p", kw.get("ord", consts[0] if consts else 2))
    dim = kw.get("dim", consts[1] if len(consts) > 1 else None)
    if isinstance(dim, (list, tuple)) and len(dim) == 1:
        dim = dim[0]
    if p not in (2, 2.0, "fro", None) or not isinstance(dim, int) or dim % len(x.shape) != len(x.shape) - 1 or not is_float(x.dtype):
        raise UnsupportedOperationError(node.op_name, f"p={p!r}, dim={dim!r}; only the 2-norm over the last dimension")
    f32 = torch.float32
    ssq, l1 = _row_statistic(cluster, "sumsq", [x], ReduceOp.SUM, lambda b: b._emit(EwOp.MUL, 0, 0, dtype=f32))
    b2 = _ProgramBuilder([ssq], ssq.shape)
    y = b2._emit(EwOp.SQRT, 0, dtype=out.dtype)
    return [l1, KernelLaunch(Template.ELEMENTWISE, f"{cluster.signature()}:sqrt", [ssq], [out], b2.build([y]), [out.shape],
                             [out.dtype], cluster=cluster)]


def _lower_normalize(cluster: FusionCluster) -> list:
    """F.normalize(x, p=2, dim=last, eps): x / max(||x||_2, eps) with the row norm in fp32."""
    _require_shapes(cluster)
    node = cluster.nodes[0]
    spec = node.metadata.get("arg_spec", [])
    kw = node.metadata.get("kwargs", {})
    x, out = node.inputs[spec[0][1]], node.outputs[0]
    consts = _const_args(node)
    p = kw.get("p", consts[0] if consts else 2.0)
    dim = kw.get("dim", consts[1] if len(consts) > 1 else 1)
    eps = kw.get("eps", consts[2] if len(consts) > 2 else 1e-12)
    if p not in (2, 2.0) or not isinstance(dim, int) or dim % len(x.shape) != len(x.shape) - 1 or not is_float(x.dtype):
        raise UnsupportedOperationError("normalize", f"p={p!r}, dim={dim!r}; only the 2-norm over the last dimension")
    f32 = torch.float32
    ssq, l1 = _row_statistic(cluster, "sumsq", [x], ReduceOp.SUM, lambda b: b._emit(EwOp.MUL, 0, 0, dtype=f32))
    b2 = _ProgramBuilder([x, ssq], x.shape)
    n = b2._emit(EwOp.MAX, b2._emit(EwOp.SQRT, 1, dtype=f32), b2._emit(EwOp.CONST, imm=eps, dtype=f32), dtype=f32)
    y = b2._emit(EwOp.DIV, 0, n, dtype=out.dtype)
    return [l1, KernelLaunch(Template.ELEMENTWISE, f"{cluster.signature()}:divide", [x, ssq], [out], b2.build([y]),
                             [out.shape], [out.dtype], cluster=cluster)]


def _lower_norm(cluster: FusionCluster) -> list:
    name = cluster.nodes[0].op_name
    if name in ("norm", "vector_norm", "linalg_vector_norm"):
        return _lower_vector_norm(cluster)
    if name == "normalize":
        return _lower_normalize(cluster)
    if name in ("mse_loss", "l1_loss"):
        return _lower_pointwise_loss(cluster)
    if name == "rms_norm":
        return _lower_rms_norm(cluster)
    if name in ("log_softmax", "logsumexp"):
        return _lower_log_softmax(cluster)
    if name in ("var", "std"):
        return _lower_variance(cluster)
    return _lower_layer_norm(cluster)


_LOWERING = {
    FusionType.NORM: _lower_norm,
    FusionType.ELEMENTWISE: _lower_elementwise,
    FusionType.REDUCTION: _lower_reduction,
    FusionType.SOFTMAX: _lower_softmax,
    FusionType.GEMM_EPILOGUE: _lower_gemm,
    FusionType.ATTENTION: _lower_attention,
    FusionType.SHAPE: _lower_shape,
}


class KernelTemplateSelector:
    """Public face of this module; plays the role of ``ChoreoDslGen`` in the reference pipeline
    (``jit_compiler.py:150-163`` calls ``generate_dsl_file(dag, function_name)``)."""

    def select(self, cluster: FusionCluster):
        """One KernelLaunch for the cluster, or a list of them when a cluster needs several
        (layer_norm: two reductions and a chain)."""
        fn = _LOWERING.get(cluster.cluster_type)
        if fn is None:
            ops = ",".join(n.op_name for n in cluster.nodes)
            raise UnsupportedOperationError(ops, "no kernel template implements this operation")
        return fn(cluster)

    def generate_plan_text(self, launches: list[KernelLaunch], function_name: str = "kernel") -> str:
        """Readable plan, the analogue of the ``.co`` text the reference dumps for debugging."""
        lines = [f"plan {function_name} {{"]
        lines += [f"  {l.describe()}" for l in launches]
        lines.append("}")
        return "\n".join(lines)
