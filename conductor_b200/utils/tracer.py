"""Compilation / execution trace for developers.

Counterpart of ``ConductorTracer`` (reference: ``conductor/utils/tracer.py:21-220``): the same
switches (``debug.enabled``, ``trace_dag``, ``trace_dsl``, ``trace_compilation``,
``trace_execution``, ``verbose_level``) and the same module-level helpers, but it logs through
the package logger instead of printing, dumps no tensor contents, and what it shows as "DSL" is
the kernel plan (template, operands and parameters of every cluster).
"""
from __future__ import annotations

import time
from dataclasses import dataclass
from typing import Any, Dict, List, Optional

import torch

from .logging import get_logger

logger = get_logger("conductor_b200.trace")


@dataclass
class TraceConfig:
    enabled: bool = False
    trace_dag: bool = True
    trace_dsl: bool = True
    trace_compilation: bool = True
    trace_execution: bool = False
    verbose_level: int = 1
    max_tensor_elements: int = 100
    indent_size: int = 2


def _describe_tensor(t: Any) -> str:
    if isinstance(t, torch.Tensor):
        return f"{str(t.dtype).replace('torch.', '')}{list(t.shape)}@{t.device}"
    return type(t).__name__


class ConductorTracer:
    def __init__(self, config: Optional[TraceConfig] = None):
        self.config = config if config is not None else self._load_trace_config()
        self.records: List[Dict[str, Any]] = []     # what was traced, for tools and tests
        self.max_records = 1000

    def _load_trace_config(self) -> TraceConfig:
        from .config import get_config

        d = get_config().debug
        return TraceConfig(enabled=d.enabled, trace_dag=d.trace_dag, trace_dsl=d.trace_dsl,
                           trace_compilation=d.trace_compilation, trace_execution=d.trace_execution,
                           verbose_level=d.verbose_level, max_tensor_elements=d.max_tensor_elements,
                           indent_size=d.indent_size)

    # ------------------------------------------------------------------ switches
    def is_enabled(self) -> bool:
        return self.config.enabled

    def should_trace_dag(self) -> bool:
        return self.config.enabled and self.config.trace_dag

    def should_trace_dsl(self) -> bool:
        return self.config.enabled and self.config.trace_dsl

    def should_trace_compilation(self) -> bool:
        return self.config.enabled and self.config.trace_compilation

    def should_trace_execution(self) -> bool:
        return self.config.enabled and self.config.trace_execution

    def get_verbose_level(self) -> int:
        return self.config.verbose_level

    # ------------------------------------------------------------------ sinks
    def _emit(self, kind: str, title: str, body: str, **fields) -> None:
        rec = {"kind": kind, "title": title, "time": time.time(), **fields}
        if len(self.records) < self.max_records:
            self.records.append(rec)
        pad = " " * self.config.indent_size
        text = "\n".join(pad + line for line in body.splitlines()) if body else ""
        logger.info("=== %s ===%s", title, "\n" + text if text else "")

    def trace_dag(self, dag: Any, title: str = "Internal DAG") -> None:
        if not self.should_trace_dag():
            return
        from ..optimization.graph_analyzer import GraphAnalyzer

        self._emit("dag", title, GraphAnalyzer().describe(dag), n_nodes=len(dag.nodes), n_buffers=len(dag.buffers))

    def trace_dsl(self, dsl_content: str, kernel_code: Optional[str] = None, title: str = "Kernel plan") -> None:
        if not self.should_trace_dsl():
            return
        body = dsl_content
        if kernel_code and self.config.verbose_level >= 2:
            body += "\n--- run-time instance ---\n" + kernel_code
        self._emit("plan", title, body)

    def trace_compilation(self, command: List[str], result: Any, title: str = "Compilation") -> None:
        """`command` is the list of pipeline stages that ran, `result` a dict of their outcome
        (the reference passes the compiler command line and the subprocess result)."""
        if not self.should_trace_compilation():
            return
        body = " -> ".join(command)
        if isinstance(result, dict):
            body += "\n" + "\n".join(f"{k}: {v}" for k, v in result.items())
        elif result is not None:
            body += f"\n{result}"
        self._emit("compilation", title, body, result=result if isinstance(result, dict) else None)

    def trace_execution(self, function_name: str, inputs: List[Any], outputs: List[Any], duration_ms: float) -> None:
        if not self.should_trace_execution():
            return
        body = (f"inputs:  {', '.join(_describe_tensor(t) for t in inputs)}\n"
                f"outputs: {', '.join(_describe_tensor(t) for t in outputs)}\n"
                f"host time: {duration_ms:.3f} ms (launch is asynchronous)")
        self._emit("execution", f"Execution of {function_name}", body, function=function_name, duration_ms=duration_ms)

    def trace_graph_hash(self, graph_hash: str, graph_info: Dict[str, Any]) -> None:
        if not self.should_trace_compilation():
            return
        self._emit("hash", f"Graph {graph_hash}", "\n".join(f"{k}: {v}" for k, v in graph_info.items()), graph_hash=graph_hash)

    def trace_cache_operation(self, operation: str, graph_hash: str, success: bool) -> None:
        if not self.should_trace_compilation():
            return
        self._emit("cache", f"Cache {operation}", f"{graph_hash}: {'hit' if success else 'miss'}",
                   operation=operation, graph_hash=graph_hash, success=success)


_tracer: Optional[ConductorTracer] = None


def get_tracer() -> ConductorTracer:
    global _tracer
    if _tracer is None:
        _tracer = ConductorTracer()
    return _tracer


def reset_tracer() -> None:
    """Forget the tracer so that the next use re-reads the configuration."""
    global _tracer
    _tracer = None


def trace_internal_dag(dag: Any) -> None:
    get_tracer().trace_dag(dag)


def trace_choreo_dsl(dsl_content: str, kernel_code: Optional[str] = None) -> None:
    get_tracer().trace_dsl(dsl_content, kernel_code)


def trace_compilation_result(command: List[str], result: Any) -> None:
    get_tracer().trace_compilation(command, result)


def trace_execution_result(function_name: str, inputs: List[Any], outputs: List[Any], duration_ms: float) -> None:
    get_tracer().trace_execution(function_name, inputs, outputs, duration_ms)
