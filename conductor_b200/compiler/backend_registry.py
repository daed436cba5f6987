"""Registration with ``torch.compile`` (reference: ``conductor/compiler/backend_registry.py:17-48``)."""
from __future__ import annotations

from typing import Callable

import torch

from ..utils.logging import get_logger

logger = get_logger(__name__)
_registered_backends: set[str] = set()


def register_backend(name: str, compiler_fn: Callable) -> bool:
    """Register `compiler_fn` under `name`; idempotent.  Returns False when torch has no
    backend registry or the registration raises."""
    if name in _registered_backends:
        return True
    try:
        import torch._dynamo as dynamo

        if not hasattr(dynamo, "register_backend"):
            logger.error("this torch build has no torch._dynamo.register_backend")
            return False
        dynamo.register_backend(name=name, compiler_fn=compiler_fn)
        _registered_backends.add(name)
        return True
    except Exception as exc:  # same contract as the reference: report, do not raise
        logger.error("failed to register backend %r: %s", name, exc)
        return False


def is_backend_registered(name: str) -> bool:
    return name in _registered_backends
