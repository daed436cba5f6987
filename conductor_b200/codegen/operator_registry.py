"""Operator table: FX op name -> classification and kernel-template binding.

Counterpart of the reference's ``conductor/codegen/operator_registry.py:245-601``,
whose ``OperatorInfo`` carries Choreo DSL snippets.  Here an operator carries the
opcode it contributes to an elementwise program (``cdr_ew_op`` in
``include/conductor_b200.h``) or the template family that implements it.

Differences from the reference table, all needed by the five benchmark graphs:
  * ``relu`` and the unary math ops are ELEMENTWISE and fusable (the reference
    registers relu as ACTIVATION, ``operator_registry.py:365-373``, which blocks every
    chain that contains it);
  * ``softmax``, ``_softmax_backward_data``, ``linear``, ``scaled_dot_product_attention``,
    ``addcdiv``, ``addcmul`` and the dtype casts are registered (absent in the reference,
    ``operator_registry.py:489-500``).
"""
from __future__ import annotations

from dataclasses import dataclass
from enum import Enum
from typing import Dict, Optional

from ..utils.constants import FusionLevel


class OpType(Enum):
    """Operation classes (reference: ``operator_registry.py:72-83``)."""

    ELEMENTWISE = "elementwise"
    REDUCTION = "reduction"
    MATRIX = "matrix"
    ACTIVATION = "activation"
    SHAPE = "shape"
    MATH = "math"
    SOFTMAX = "softmax"
    ATTENTION = "attention"
    NORM = "norm"
    UNKNOWN = "unknown"


# cdr_ew_op codes (include/conductor_b200.h)
class EwOp:
    ADD, SUB, MUL, DIV, RELU, NEG, ABS, EXP, LOG, SQRT, SIGMOID, TANH, SIN, COS = range(1, 15)
    MAX, MIN, ADDCDIV, ADDCMUL, CONST, COPY, ADD_IMM, MUL_IMM, RSUB_IMM, RDIV_IMM = range(15, 25)
    GT, GE, LT, LE, EQ, NE, WHERE, RSQRT, SILU, GELU, ERF = range(25, 36)


class ReduceOp:
    SUM, MEAN, MAX, MIN = 1, 2, 3, 4


class Template:
    """cdr_template ids."""

    ELEMENTWISE, ROW_REDUCE, SOFTMAX_FWD, SOFTMAX_BWD, GEMM_EPILOGUE, ATTENTION, FULL_REDUCE, LAYER_NORM, COPY, COL_SUM = range(1, 11)


@dataclass(frozen=True)
class OperatorInfo:
    """What the analysis and template selection need to know about one operator."""

    name: str
    canonical_name: str
    operation_type: OpType
    fusable: bool = True
    arity: int = 2                      # tensor operands of the elementwise form
    ew_op: Optional[int] = None         # opcode inside an elementwise program
    reduce_op: Optional[int] = None     # reduction kind for REDUCTION operators
    template: Optional[int] = None      # template family for non-elementwise operators
    preferred_fusion_level: FusionLevel = FusionLevel.LOCAL
    requires_device_kernel: bool = True

    def is_elementwise(self) -> bool:
        return self.operation_type is OpType.ELEMENTWISE

    def is_reduction(self) -> bool:
        return self.operation_type is OpType.REDUCTION


def _ew(name, op, arity, canonical=None):
    return OperatorInfo(name, canonical or name, OpType.ELEMENTWISE, True, arity, ew_op=op,
                        template=Template.ELEMENTWISE)


def _red(name, op, canonical=None):
    return OperatorInfo(name, canonical or name, OpType.REDUCTION, True, 1, reduce_op=op,
                        template=Template.ROW_REDUCE, preferred_fusion_level=FusionLevel.GLOBAL)


class OperatorRegistry:
    """Name -> OperatorInfo, with the aliases Dynamo and ``fx.symbolic_trace`` produce."""

    def __init__(self):
        self._ops: Dict[str, OperatorInfo] = {}
        self._register_defaults()

    def register(self, info: OperatorInfo, *aliases: str) -> None:
        self._ops[info.name] = info
        for a in aliases:
            self._ops[a] = info

    def _register_defaults(self) -> None:
        r = self.register
        r(_ew("add", EwOp.ADD, 2), "iadd", "add_")
        r(_ew("sub", EwOp.SUB, 2), "isub", "sub_", "subtract")
        r(_ew("mul", EwOp.MUL, 2), "imul", "mul_", "multiply")
        r(_ew("div", EwOp.DIV, 2), "truediv", "itruediv", "div_", "true_divide", "divide")
        r(_ew("relu", EwOp.RELU, 1), "relu_")
        r(_ew("neg", EwOp.NEG, 1), "negative")
        r(_ew("abs", EwOp.ABS, 1), "absolute")
        r(_ew("exp", EwOp.EXP, 1))
        r(_ew("log", EwOp.LOG, 1))
        r(_ew("sqrt", EwOp.SQRT, 1))
        r(_ew("sigmoid", EwOp.SIGMOID, 1))
        r(_ew("tanh", EwOp.TANH, 1))
        r(_ew("sin", EwOp.SIN, 1))
        r(_ew("cos", EwOp.COS, 1))
        r(_ew("maximum", EwOp.MAX, 2))
        r(_ew("minimum", EwOp.MIN, 2))
        r(_ew("addcdiv", EwOp.ADDCDIV, 3))
        r(_ew("addcmul", EwOp.ADDCMUL, 3))
        # comparisons produce 1.0 / 0.0 inside a fused chain; `where` selects on != 0
        r(_ew("gt", EwOp.GT, 2), "greater", "__gt__")
        r(_ew("ge", EwOp.GE, 2), "greater_equal", "__ge__")
        r(_ew("lt", EwOp.LT, 2), "less", "__lt__")
        r(_ew("le", EwOp.LE, 2), "less_equal", "__le__")
        r(_ew("eq", EwOp.EQ, 2), "__eq__")
        r(_ew("ne", EwOp.NE, 2), "not_equal", "__ne__")
        r(_ew("where", EwOp.WHERE, 3))
        r(_ew("rsqrt", EwOp.RSQRT, 1))
        r(_ew("silu", EwOp.SILU, 1), "silu_")
        r(_ew("gelu", EwOp.GELU, 1))
        r(_ew("erf", EwOp.ERF, 1))
        # lowered to existing instructions: clamp -> max/min with constants, pow -> mul / sqrt / reciprocal
        r(_ew("clamp", EwOp.MAX, 1), "clip", "clamp_", "hardtanh", "relu6", "clamp_min", "clamp_max", "clamp_min_", "clamp_max_")
        r(_ew("pow", EwOp.MUL, 2), "square", "reciprocal")
        # activations and selections written out over the opcode set by the program builder
        r(_ew("composite", EwOp.WHERE, 1), "leaky_relu", "leaky_relu_", "elu", "elu_", "softplus", "hardswish",
          "hardsigmoid", "dropout")
        r(_ew("composite2", EwOp.WHERE, 2, canonical="composite"), "masked_fill", "masked_fill_")
        r(_ew("composite3", EwOp.WHERE, 3, canonical="composite"), "lerp")
        # dtype casts are a rounding-only instruction
        r(_ew("to_dtype", EwOp.COPY, 1), "float", "bfloat16", "half", "to", "type")
        r(_red("sum", ReduceOp.SUM))
        r(_red("reduce_mean", ReduceOp.MEAN), "mean")
        r(_red("amax", ReduceOp.MAX))
        r(_red("amin", ReduceOp.MIN))
        r(OperatorInfo("softmax", "softmax", OpType.SOFTMAX, False, 1, template=Template.SOFTMAX_FWD,
                       preferred_fusion_level=FusionLevel.GLOBAL), "_softmax")
        r(OperatorInfo("_softmax_backward_data", "softmax_backward", OpType.SOFTMAX, False, 2,
                       template=Template.SOFTMAX_BWD, preferred_fusion_level=FusionLevel.GLOBAL))
        r(OperatorInfo("layer_norm", "layer_norm", OpType.NORM, False, 3, preferred_fusion_level=FusionLevel.GLOBAL))
        # row statistics lowered to several launches of the reduce and elementwise templates
        for name, arity in (("rms_norm", 2), ("log_softmax", 1), ("logsumexp", 1), ("var", 1), ("std", 1),
                            ("mse_loss", 2), ("l1_loss", 2), ("norm", 1), ("vector_norm", 1), ("linalg_vector_norm", 1), ("normalize", 1)):
            r(OperatorInfo(name, name, OpType.NORM, False, arity, preferred_fusion_level=FusionLevel.GLOBAL))
        r(OperatorInfo("linear", "linear", OpType.MATRIX, True, 3, template=Template.GEMM_EPILOGUE,
                       preferred_fusion_level=FusionLevel.GLOBAL))
        r(OperatorInfo("matmul", "matmul", OpType.MATRIX, False, 2, template=Template.GEMM_EPILOGUE,
                       preferred_fusion_level=FusionLevel.GLOBAL), "mm", "bmm")
        r(OperatorInfo("addmm", "addmm", OpType.MATRIX, False, 3, template=Template.GEMM_EPILOGUE,
                       preferred_fusion_level=FusionLevel.GLOBAL))
        r(OperatorInfo("scaled_dot_product_attention", "attention", OpType.ATTENTION, False, 3,
                       template=Template.ATTENTION, preferred_fusion_level=FusionLevel.GLOBAL), "attention")
        # metadata-only reshapes of contiguous tensors: no kernel
        # layout changes that move data: one launch of the strided-copy template
        for perm_op in ("transpose", "permute", "t", "swapaxes", "movedim"):
            r(OperatorInfo(perm_op, "permute", OpType.SHAPE, False, 1))
        for slice_op in ("getitem", "__getitem__", "narrow", "select", "view_of", "expand", "broadcast_to", "expand_as"):
            r(OperatorInfo(slice_op, "slice", OpType.SHAPE, False, 1))
        r(OperatorInfo("cat", "cat", OpType.SHAPE, False, 2), "concat", "concatenate")
        for shape_op in ("view", "reshape", "flatten", "unsqueeze", "squeeze", "contiguous", "detach", "clone_view"):
            r(OperatorInfo(shape_op, shape_op, OpType.SHAPE, False, 1, requires_device_kernel=False))

    def get_operation(self, name: str) -> Optional[OperatorInfo]:
        return self._ops.get(name)

    def has_operation(self, name: str) -> bool:
        return name in self._ops

    def list_operations(self) -> list[str]:
        return sorted(self._ops)


_registry: Optional[OperatorRegistry] = None


def get_operator_registry() -> OperatorRegistry:
    global _registry
    if _registry is None:
        _registry = OperatorRegistry()
    return _registry


def get_op_desc(name: str) -> Optional[OperatorInfo]:
    return get_operator_registry().get_operation(name)


def is_elementwise(name: str) -> bool:
    info = get_op_desc(name)
    return bool(info and info.is_elementwise())


def is_reduction(name: str) -> bool:
    info = get_op_desc(name)
    return bool(info and info.is_reduction())
