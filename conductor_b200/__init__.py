"""conductor_b200: a B200-native ``torch.compile`` backend with the plugin surface of
codes1gn/conductor.

    import torch, conductor            # registers the 'gcu' backend
    fn = torch.compile(model, backend='gcu')

(reference: ``conductor/__init__.py:26-41``).  The FX->DAG analysis, fusion clustering and
buffer scoping are Python; every fused cluster runs as a hand-written sm_100a CUDA kernel
from ``libconductor_b200.so`` reached through a C ABI.
"""
__version__ = "0.1.0"

from .compiler.gcu_backend import GCUBackend, get_gcu_backend, register_gcu_backend
from .utils.config import get_config

__all__ = ["register_gcu_backend", "GCUBackend", "get_gcu_backend", "get_config"]

try:
    register_gcu_backend()
except Exception as exc:  # same policy as the reference: warn, do not break the import
    import warnings

    warnings.warn(f"Failed to register Conductor backend: {exc}", UserWarning)
