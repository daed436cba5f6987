"""Logging setup (reference: ``conductor/utils/logging.py:13-52``).

Loggers are named ``conductor.<module>``.  The level comes from
``CONDUCTOR_LOG_LEVEL`` (default WARNING; the reference ships DEBUG, which prints
whole tensors on import).
"""
from __future__ import annotations

import logging
import os

_CONFIGURED = False


def setup_logging(level: str | None = None) -> None:
    global _CONFIGURED
    name = (level or os.environ.get("CONDUCTOR_LOG_LEVEL", "WARNING")).upper()
    root = logging.getLogger("conductor")
    root.setLevel(getattr(logging, name, logging.WARNING))
    if not _CONFIGURED and not root.handlers:
        handler = logging.StreamHandler()
        handler.setFormatter(logging.Formatter("%(asctime)s %(name)s %(levelname)s: %(message)s"))
        root.addHandler(handler)
        root.propagate = False
    _CONFIGURED = True


def get_logger(name: str) -> logging.Logger:
    if not _CONFIGURED:
        setup_logging()
    short = name.split(".", 1)[1] if name.startswith(("conductor_b200.", "conductor.")) else name
    return logging.getLogger(f"conductor.{short}")
