"""Locate and load ``libconductor_b200.so`` (reference: ``conductor/compiler/loader.py:1-234`` and
``host_wrapper.py:338-355`` load a freshly compiled per-graph ``.so`` with ``ctypes.CDLL``).

The library is built ahead of time, in-tree, by ``conductor_b200/csrc/build.py``.  A missing
library is a hard error (:class:`DeviceError`): there is no CPU implementation to fall back to.
"""
from __future__ import annotations

import ctypes
import os
from pathlib import Path
from typing import Optional

from ..codegen.kernel_templates import CdrTensor
from ..utils.exceptions import DeviceError

CSRC_DIR = Path(__file__).resolve().parent.parent / "csrc"
LIB_NAME = "libconductor_b200.so"
ABI_VERSION = 1

_lib: Optional[ctypes.CDLL] = None

# name -> (restype, argtypes): every symbol include/conductor_b200.h declares
_c = ctypes
_TENSORS = _c.POINTER(CdrTensor)
SYMBOLS = {
    "cdr_abi_version": (_c.c_int, []),
    "cdr_status_string": (_c.c_char_p, [_c.c_int]),
    "cdr_last_error": (_c.c_char_p, []),
    "cdr_device_count": (_c.c_int, []),
    "cdr_device_status": (_c.c_int, [_c.POINTER(_c.c_int), _c.c_int]),
    "cdr_template_source": (_c.c_int, [_c.c_int, _TENSORS, _c.c_int, _TENSORS, _c.c_int, _c.c_void_p, _c.c_size_t,
                                       _c.c_char_p, _c.c_size_t, _c.c_int]),
    "cdr_workspace_bytes": (_c.c_int, [_c.c_int, _TENSORS, _c.c_int, _TENSORS, _c.c_int, _c.c_void_p, _c.c_size_t,
                                       _c.POINTER(_c.c_size_t)]),
    "cdr_launch": (_c.c_int, [_c.c_int, _TENSORS, _c.c_int, _TENSORS, _c.c_int, _c.c_void_p, _c.c_size_t,
                              _c.c_void_p, _c.c_size_t, _c.c_void_p]),
    "cdr_launch_many": (_c.c_int, [_c.c_void_p, _c.c_int, _c.c_void_p, _c.POINTER(_c.c_int)]),
    "cdr_execute_host": (_c.c_int, [_c.c_int, _TENSORS, _c.c_int, _TENSORS, _c.c_int, _c.c_void_p, _c.c_size_t,
                                    _c.c_int]),
    "cdr_release_host_arena": (_c.c_int, [_c.c_int]),
    "cdr_full_reduce_noalloc": (_c.c_int, [_TENSORS, _c.c_int, _TENSORS, _c.c_int, _c.c_void_p, _c.c_size_t,
                                           _c.c_void_p]),
}


def library_path() -> Path:
    override = os.environ.get("CONDUCTOR_B200_LIB")
    return Path(override) if override else CSRC_DIR / LIB_NAME


def load_library(build_if_missing: bool = False) -> ctypes.CDLL:
    """Load the kernel library once per process and bind every exported symbol."""
    global _lib
    if _lib is not None:
        return _lib
    path = library_path()
    if not path.exists() and build_if_missing:
        from ..csrc.build import build

        build()
    if not path.exists():
        raise DeviceError(f"kernel library {path} is missing; run `python -m conductor_b200.csrc.build`")
    try:
        lib = ctypes.CDLL(str(path))
    except OSError as exc:
        raise DeviceError(f"cannot load {path}: {exc}") from exc
    for name, (restype, argtypes) in SYMBOLS.items():
        try:
            fn = getattr(lib, name)
        except AttributeError as exc:
            raise DeviceError(f"{path} does not export {name}") from exc
        fn.restype = restype
        fn.argtypes = argtypes
    version = lib.cdr_abi_version()
    if version != ABI_VERSION:
        raise DeviceError(f"{path} has ABI version {version}, expected {ABI_VERSION}")
    _lib = lib
    return lib


def unload_library() -> None:
    global _lib
    _lib = None
