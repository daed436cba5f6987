"""Cross-cutting helpers (reference: ``conductor/utils/``)."""
from .config import ConductorConfig, get_config, reset_config, set_config
from .constants import BufferScope, FusionLevel, MemoryLevel, TensorRank
from .exceptions import (
    CompilationError,
    ConductorError,
    DeviceError,
    ExecutionError,
    UnsupportedOperationError,
)
from .logging import get_logger, setup_logging

__all__ = [
    "ConductorConfig", "get_config", "set_config", "reset_config",
    "BufferScope", "FusionLevel", "MemoryLevel", "TensorRank",
    "ConductorError", "CompilationError", "DeviceError", "ExecutionError", "UnsupportedOperationError",
    "get_logger", "setup_logging",
]
