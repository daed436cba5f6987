"""Enumerations shared by the analysis and template-selection layers.

Counterparts in the reference: ``conductor/utils/constants.py:20-120``
(``MemoryLevel``, ``TensorRank``, ``FusionLevel``, ``BufferScope``).  Only the
members the kernel-template path reads are kept; the Choreo DSL keyword tables
of the reference have no equivalent here.
"""
from __future__ import annotations

from enum import Enum


class BufferScope(Enum):
    """Where a buffer lives (reference: ``constants.py:115-120``).

    On B200 the three scopes map to: LOCAL -> registers of the thread that
    produced the value, SHARED -> shared memory / TMA-staged tiles of one CTA,
    GLOBAL -> HBM.
    """

    LOCAL = "local"
    SHARED = "shared"
    GLOBAL = "global"


class MemoryLevel(Enum):
    """Hardware level a scope is realised in (reference: ``constants.py:20-51``)."""

    GLOBAL = "global"   # HBM3e
    L2 = "l2"           # 126 MB L2
    L1 = "l1"           # shared memory / L1
    REGISTER = "reg"    # register file

    @property
    def priority(self) -> int:
        return {MemoryLevel.REGISTER: 4, MemoryLevel.L1: 3, MemoryLevel.L2: 2, MemoryLevel.GLOBAL: 1}[self]

    @classmethod
    def for_scope(cls, scope: BufferScope) -> "MemoryLevel":
        return {BufferScope.LOCAL: cls.REGISTER, BufferScope.SHARED: cls.L1, BufferScope.GLOBAL: cls.GLOBAL}[scope]


class TensorRank(Enum):
    """Dimensionality class of a tensor (reference: ``constants.py:58-91``)."""

    SCALAR = 0
    VECTOR = 1
    MATRIX = 2
    TENSOR_3D = 3
    TENSOR_ND = 4

    @classmethod
    def from_shape(cls, shape) -> "TensorRank":
        n = len(shape) if shape is not None else 0
        return cls(min(n, 4))


class FusionLevel(Enum):
    """Which phase of the fusion engine produced a cluster (reference: ``constants.py:94-110``)."""

    LOCAL = "local"
    ADJACENT = "adjacent"
    GLOBAL = "global"

    @property
    def priority(self) -> int:
        return {FusionLevel.LOCAL: 3, FusionLevel.ADJACENT: 2, FusionLevel.GLOBAL: 1}[self]
