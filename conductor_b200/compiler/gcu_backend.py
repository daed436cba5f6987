"""The ``gcu`` backend object (reference: ``conductor/compiler/gcu_backend.py:23-117``).

Same surface: ``GCUBackend()(graph_module, example_inputs) -> callable``, a per-process cache
keyed by a graph hash, ``get_gcu_backend()`` and ``register_gcu_backend()``.  One deliberate
difference: the reference catches every compile failure and returns ``graph_module.forward``
(eager, ``gcu_backend.py:70-89``); this backend has no CPU path and raises instead.
"""
from __future__ import annotations

import hashlib
from typing import Callable as TypingCallable, List, Optional

import torch
import torch.fx as fx

from ..utils.config import get_config
from ..utils.logging import get_logger
from .backend_registry import register_backend
from .callable import Callable as GCUCallable
from .jit_compiler import ChoreoJITCompiler, constants_fingerprint

logger = get_logger(__name__)


class GCUBackend:
    def __init__(self):
        self.jit_compiler = ChoreoJITCompiler()
        self._compiled_functions: dict[str, GCUCallable] = {}

    def __call__(self, graph_module: fx.GraphModule, example_inputs: List[torch.Tensor]) -> TypingCallable:
        graph_hash = self._compute_graph_hash(graph_module, example_inputs)
        cfg = get_config()
        if cfg.cache.enabled and graph_hash in self._compiled_functions:
            return self._compiled_functions[graph_hash]
        artifact = self.jit_compiler.compile_graph(graph_module, example_inputs)
        if cfg.runtime.devices > 1:
            from .sharding import ShardedCallable

            compiled_fn = ShardedCallable.from_artifact(artifact, graph_module, n_devices=cfg.runtime.devices)
        else:
            compiled_fn = GCUCallable(artifact, graph_module)
        if cfg.cache.enabled:
            self._compiled_functions[graph_hash] = compiled_fn
        return compiled_fn

    def _compute_graph_hash(self, graph_module: fx.GraphModule,
                            example_inputs: Optional[List[torch.Tensor]] = None) -> str:
        text = str(graph_module.graph)
        for t in example_inputs or []:
            if isinstance(t, torch.Tensor):
                text += f"|{tuple(t.shape)}:{t.dtype}:{t.stride()}:{t.device.type}"
        # the plan holds module parameters and constant tensors by reference: their identity is part of the key
        text += "|" + constants_fingerprint(graph_module)
        return hashlib.md5(text.encode()).hexdigest()

    def clear_cache(self) -> None:
        self._compiled_functions.clear()
        self.jit_compiler.clear_cache()


_gcu_backend: Optional[GCUBackend] = None


def get_gcu_backend() -> GCUBackend:
    global _gcu_backend
    if _gcu_backend is None:
        _gcu_backend = GCUBackend()
    return _gcu_backend


def register_gcu_backend() -> bool:
    return register_backend("gcu", get_gcu_backend())
