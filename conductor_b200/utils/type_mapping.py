"""torch dtype <-> C-ABI dtype codes (reference: ``conductor/utils/type_mapping.py:61-273``
maps torch dtypes to Choreo type names f32/f16/bf16/s32...; here the targets are the
``cdr_dtype`` codes of ``include/conductor_b200.h``)."""
from __future__ import annotations

import torch

CDR_F32, CDR_BF16, CDR_F16, CDR_I32, CDR_I64, CDR_BOOL = range(6)

_TORCH_TO_CDR = {
    torch.float32: CDR_F32,
    torch.bfloat16: CDR_BF16,
    torch.float16: CDR_F16,
    torch.int32: CDR_I32,
    torch.int64: CDR_I64,
    torch.bool: CDR_BOOL,
}
_CDR_TO_TORCH = {v: k for k, v in _TORCH_TO_CDR.items()}
_NAMES = {CDR_F32: "f32", CDR_BF16: "bf16", CDR_F16: "f16", CDR_I32: "s32", CDR_I64: "s64", CDR_BOOL: "bool"}


def to_cdr_dtype(dtype: torch.dtype) -> int:
    try:
        return _TORCH_TO_CDR[dtype]
    except KeyError:
        from .exceptions import UnsupportedOperationError

        raise UnsupportedOperationError(str(dtype), "dtype has no kernel-template support") from None


def to_torch_dtype(code: int) -> torch.dtype:
    return _CDR_TO_TORCH[code]


def dtype_name(dtype: torch.dtype) -> str:
    """Short name in the reference's convention (f32, bf16, s32 ...)."""
    return _NAMES[to_cdr_dtype(dtype)]


def is_float(dtype: torch.dtype) -> bool:
    return dtype in (torch.float32, torch.bfloat16, torch.float16)


def is_int(dtype: torch.dtype) -> bool:
    return dtype in (torch.int32, torch.int64, torch.bool)
