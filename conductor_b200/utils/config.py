"""Configuration (reference: ``conductor/utils/config.py:83-254`` + ``conductor_config.json``).

Same sections and switches as the reference (debug / cache / compilation /
runtime / logging), loaded from an optional JSON file and overridden by the
environment variables the reference honours (``CONDUCTOR_DEBUG``,
``CONDUCTOR_DISABLE_CACHE``, ``CONDUCTOR_LOG_LEVEL``; ``config.py:147,166``).
Added for the B200 runtime: ``runtime.devices`` (how many GPUs a compiled graph
is batch-sharded over), ``runtime.use_cuda_graphs`` and ``debug.dump_dir``.
Defaults differ from the shipped reference JSON on purpose: debug off, cache on,
level WARNING.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field, fields
from pathlib import Path
from typing import Optional


@dataclass
class DebugConfig:
    enabled: bool = False
    max_tensor_elements: int = 100
    indent_size: int = 2
    trace_dag: bool = True
    trace_dsl: bool = True          # here: trace the kernel plan
    trace_compilation: bool = True
    trace_execution: bool = False
    verbose_level: int = 1
    dump_dir: Optional[str] = None  # opt-in artifact directory (never the package tree)


@dataclass
class CacheConfig:
    enabled: bool = True
    max_size_mb: int = 1024
    cache_dir: Optional[str] = None


@dataclass
class CompilationConfig:
    timeout_seconds: int = 300
    optimization_level: str = "O2"
    enable_fusion: bool = True
    enable_graph_validation: bool = True
    enable_shape_inference: bool = True
    enable_buffer_optimization: bool = True


@dataclass
class RuntimeConfig:
    device: str = "gcu"             # backend name kept from the reference; executes on CUDA
    memory_pool_size_mb: int = 512
    enable_profiling: bool = False
    devices: int = 1                # GPUs a compiled graph is batch-sharded over
    use_cuda_graphs: bool = False
    # host-tensor calls of a batch-parallel graph are cut into row chunks of about this many input
    # bytes so that copies in, kernels and copies out overlap inside one call (0 = never chunk)
    host_chunk_bytes: int = 8 << 20
    host_max_chunks: int = 8


@dataclass
class LoggingConfig:
    level: str = "WARNING"
    enable_file_logging: bool = False
    log_file: str = "conductor.log"


def _fill(cls, data: dict):
    known = {f.name for f in fields(cls)}
    return cls(**{k: v for k, v in (data or {}).items() if k in known})


@dataclass
class ConductorConfig:
    debug: DebugConfig = field(default_factory=DebugConfig)
    cache: CacheConfig = field(default_factory=CacheConfig)
    compilation: CompilationConfig = field(default_factory=CompilationConfig)
    runtime: RuntimeConfig = field(default_factory=RuntimeConfig)
    logging: LoggingConfig = field(default_factory=LoggingConfig)
    config_file: Optional[str] = None

    @classmethod
    def load(cls, config_file: Optional[str] = None) -> "ConductorConfig":
        path = config_file or os.environ.get("CONDUCTOR_CONFIG")
        data: dict = {}
        if path and Path(path).is_file():
            text = Path(path).read_text()
            if str(path).endswith((".yaml", ".yml")):
                import yaml

                data = yaml.safe_load(text) or {}
            else:
                data = json.loads(text)
        cfg = cls(
            debug=_fill(DebugConfig, data.get("debug")),
            cache=_fill(CacheConfig, data.get("cache")),
            compilation=_fill(CompilationConfig, data.get("compilation")),
            runtime=_fill(RuntimeConfig, data.get("runtime")),
            logging=_fill(LoggingConfig, data.get("logging")),
            config_file=path,
        )
        cfg._apply_env()
        return cfg

    def _apply_env(self) -> None:
        env = os.environ
        if "CONDUCTOR_DEBUG" in env:
            self.debug.enabled = env["CONDUCTOR_DEBUG"].lower() in ("1", "true", "yes", "on")
        if env.get("CONDUCTOR_DISABLE_CACHE", "").lower() in ("1", "true", "yes", "on"):
            self.cache.enabled = False
        if "CONDUCTOR_LOG_LEVEL" in env:
            self.logging.level = env["CONDUCTOR_LOG_LEVEL"].upper()
        if "CONDUCTOR_DEVICES" in env:
            self.runtime.devices = max(1, int(env["CONDUCTOR_DEVICES"]))

    # accessors named as in the reference (config.py:200-254)
    def is_debug_enabled(self) -> bool:
        return self.debug.enabled

    def is_cache_enabled(self) -> bool:
        return self.cache.enabled

    def to_dict(self) -> dict:
        from dataclasses import asdict

        return asdict(self)


_config: Optional[ConductorConfig] = None


def get_config() -> ConductorConfig:
    global _config
    if _config is None:
        _config = ConductorConfig.load()
    return _config


def set_config(cfg: ConductorConfig) -> None:
    global _config
    _config = cfg


def reset_config() -> None:
    global _config
    _config = None
