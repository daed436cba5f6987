"""Operator tables and kernel-template selection (replaces the reference's Choreo DSL
emitter package ``conductor/codegen/``)."""
from .operator_registry import (
    EwOp, OpType, OperatorInfo, OperatorRegistry, ReduceOp, Template,
    get_op_desc, get_operator_registry, is_elementwise, is_reduction,
)
from .operation_factory import OperationFactory, get_operation_factory

__all__ = [
    "EwOp", "OpType", "OperatorInfo", "OperatorRegistry", "ReduceOp", "Template",
    "get_op_desc", "get_operator_registry", "is_elementwise", "is_reduction",
    "OperationFactory", "get_operation_factory",
]
