"""Exception hierarchy of the backend.

Same class names and constructor arguments as the reference
(``conductor/utils/exceptions.py:16-166``) so that user code catching
``conductor.utils.exceptions.ExecutionError`` keeps working.  The reference's
``FallbackHandler`` (``exceptions.py:169-257``) is intentionally absent: this
backend never falls back to CPU execution; unsupported graphs raise at compile time.
"""
from __future__ import annotations

from typing import Optional


class ConductorError(Exception):
    """Root of all backend errors."""

    def __init__(self, message: str, details: Optional[dict] = None):
        super().__init__(message)
        self.message = message
        self.details = details or {}

    def __str__(self) -> str:
        if self.details:
            extra = ", ".join(f"{k}={v}" for k, v in self.details.items())
            return f"{self.message} ({extra})"
        return self.message


class CompilationError(ConductorError):
    """Graph analysis, clustering or template selection failed.

    ``dsl_code`` / ``compiler_output`` are kept for signature compatibility; here
    they carry the textual kernel plan and the build log of the template library.
    """

    def __init__(self, message: str, dsl_code: str = "", compiler_output: str = ""):
        super().__init__(message, {"has_plan": bool(dsl_code), "has_log": bool(compiler_output)})
        self.dsl_code = dsl_code
        self.compiler_output = compiler_output

    def get_compiler_errors(self) -> list:
        return [ln for ln in self.compiler_output.splitlines() if "error" in ln.lower()]


class UnsupportedOperationError(ConductorError):
    """The graph holds an operation no kernel template covers."""

    def __init__(self, operation: str, reason: str = ""):
        msg = f"Unsupported operation: {operation}"
        if reason:
            msg += f" - {reason}"
        super().__init__(msg, {"operation": operation})
        self.operation = operation
        self.reason = reason


class DeviceError(ConductorError):
    """No usable CUDA device, or the kernel library cannot be loaded."""

    def __init__(self, message: str, device_id: Optional[int] = None):
        super().__init__(message, {"device_id": device_id} if device_id is not None else None)
        self.device_id = device_id


class ExecutionError(ConductorError):
    """A kernel launch returned a non-zero status (reference: ``executor.py:621-622``)."""

    def __init__(self, message: str, kernel_name: str = "", status: Optional[int] = None):
        details = {}
        if kernel_name:
            details["kernel"] = kernel_name
        if status is not None:
            details["status"] = status
        super().__init__(message, details)
        self.kernel_name = kernel_name
        self.status = status
