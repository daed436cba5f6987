"""Backend object, compile pipeline and runtime (reference: ``conductor/compiler/``)."""
from .backend_registry import is_backend_registered, register_backend
from .gcu_backend import GCUBackend, get_gcu_backend, register_gcu_backend

__all__ = ["GCUBackend", "get_gcu_backend", "register_gcu_backend", "register_backend", "is_backend_registered"]
