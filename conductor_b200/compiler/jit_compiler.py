"""Compilation pipeline: FX graph -> DAG -> clusters -> kernel plan.

Counterpart of ``ChoreoJITCompiler`` (reference: ``conductor/compiler/jit_compiler.py:35-233``).
The reference's stages 5-6 (print Choreo DSL, run ``choreo -c -fpic`` and ``gcc -shared``,
``jit_compiler.py:150-207,235-382``) are replaced by template selection against the prebuilt
kernel library, so "compiling" a graph takes microseconds and produces a :class:`CompiledArtifact`
whose payload is an ordered list of kernel launches.
"""
from __future__ import annotations

import hashlib
import time
from dataclasses import dataclass, field
from typing import Any, Optional

import torch

from ..codegen.kernel_templates import KernelLaunch, KernelTemplateSelector, prune_dead_launches
from ..optimization.fusion import FusionCluster, LocalPriorityFusionEngine, schedule_clusters
from ..optimization.graph_analyzer import ComputationDAG, GraphAnalyzer
from ..utils.cache import CompilationCache
from ..utils.config import get_config
from ..utils.exceptions import CompilationError, ConductorError
from ..utils.artifacts import get_debug_manager
from ..utils.logging import get_logger
from ..utils.tracer import get_tracer
from .loader import library_path

logger = get_logger(__name__)


@dataclass
class CompiledArtifact:
    """Result of compiling one graph (reference: ``conductor/compiler/loader.py:20-60``)."""

    path: str                         # the kernel library the plan runs against
    artifact_type: str                # always "kernel_plan"
    entry_point: str                  # plan name, "kernel_<hash8>"
    metadata: dict[str, Any] = field(default_factory=dict)
    launches: list[KernelLaunch] = field(default_factory=list)
    dag: Optional[ComputationDAG] = None
    clusters: list[FusionCluster] = field(default_factory=list)

    def is_valid(self) -> bool:
        return bool(self.launches) or bool(self.dag and not self.dag.nodes)


def constants_fingerprint(graph_module: torch.fx.GraphModule) -> str:
    """Identity of every tensor the plan would capture by reference: ``get_attr`` tensors and the
    parameters of leaf modules reached by ``call_module``.  Two graphs with the same text but
    different modules (or the same module after a parameter was replaced) must not share a cached
    plan, because the plan holds these tensors.  The cached plan keeps the tensors alive, so an
    ``id`` cannot be recycled for another tensor while its entry exists."""
    parts = []
    for node in graph_module.graph.nodes:
        try:
            if node.op == "get_attr":
                obj = graph_module
                for part in str(node.target).split("."):
                    obj = getattr(obj, part)
                if isinstance(obj, torch.Tensor):
                    parts.append(f"{node.target}:{id(obj)}:{tuple(obj.shape)}:{obj.dtype}")
            elif node.op == "call_module":
                mod = graph_module.get_submodule(node.target)
                for name, t in list(mod.named_parameters(recurse=True)) + list(mod.named_buffers(recurse=True)):
                    parts.append(f"{node.target}.{name}:{id(t)}:{tuple(t.shape)}:{t.dtype}")
        except AttributeError:
            parts.append(f"{node.target}:?")
    return "|".join(parts)


class ChoreoJITCompiler:
    """Pipeline driver.  The class keeps the reference's name because ``GCUBackend.jit_compiler``
    is part of the plugin surface; nothing Choreo-related remains inside."""

    def __init__(self):
        self.config = get_config()
        self.graph_analyzer = GraphAnalyzer()
        self.fusion_engine = LocalPriorityFusionEngine()
        self.template_selector = KernelTemplateSelector()
        self.cache = CompilationCache(enabled=self.config.cache.enabled)
        self.stats = {"compiled": 0, "cache_hits": 0, "seconds": 0.0}

    # ------------------------------------------------------------------ hashing
    def _generate_graph_hash(self, graph_module: torch.fx.GraphModule, example_inputs=None) -> str:
        """16 hex digits over op/target/name of every node plus shape, dtype, stride and device
        kind of every example input (the reference hashes names and shapes only,
        ``jit_compiler.py:443-470``, so a dtype change would hit a stale entry)."""
        h = hashlib.sha256()
        for node in graph_module.graph.nodes:
            h.update(f"{node.op}:{node.target}:{node.name}:{node.args}:{node.kwargs};".encode())
        for t in example_inputs or []:
            if isinstance(t, torch.Tensor):
                h.update(f"{tuple(t.shape)}:{t.dtype}:{t.stride()}:{t.device.type};".encode())
            else:
                h.update(f"{t!r};".encode())
        h.update(constants_fingerprint(graph_module).encode())
        return h.hexdigest()[:16]

    # ------------------------------------------------------------------ pipeline
    def compile_graph(self, graph_module: torch.fx.GraphModule, example_inputs=None) -> CompiledArtifact:
        t0 = time.perf_counter()
        cfg = self.config
        graph_hash = self._generate_graph_hash(graph_module, example_inputs)
        self.cache.enabled = cfg.cache.enabled
        cached = self.cache.get(graph_hash)
        tracer = get_tracer()
        tracer.trace_cache_operation("lookup", graph_hash, cached is not None)
        if cached is not None:
            self.stats["cache_hits"] += 1
            return cached
        try:
            tensors = list(example_inputs) if example_inputs is not None else None
            dag = self.graph_analyzer.parse_fx_graph(
                graph_module, tensors, enable_shape_inference=cfg.compilation.enable_shape_inference)
            if cfg.compilation.enable_graph_validation and not dag.validate_graph_correctness():
                raise CompilationError("graph validation failed")
            clusters = self.fusion_engine.identify_fusion_opportunities(
                dag, enable_fusion=cfg.compilation.enable_fusion)
            for c in clusters:
                if not c.validate_fusion_safety():
                    raise CompilationError(f"fusion cluster {c.signature()} failed its safety check")
                for n in c.nodes:
                    n.fusion_group = c
            ordered = schedule_clusters(clusters)
            launches = []
            for c in ordered:
                sel = self.template_selector.select(c)
                launches.extend(sel if isinstance(sel, list) else [sel])
            launches = prune_dead_launches(launches)
            name = f"kernel_{graph_hash[:8]}"
            plan_text = self.template_selector.generate_plan_text(launches, name)
        except ConductorError:
            raise
        except Exception as exc:
            raise CompilationError(f"compilation failed: {exc}") from exc
        artifact = CompiledArtifact(
            path=str(library_path()), artifact_type="kernel_plan", entry_point=name,
            metadata={"graph_hash": graph_hash, "plan": plan_text, "dsl_content": plan_text,
                      "n_clusters": len(clusters), "n_nodes": len(dag.nodes)},
            launches=launches, dag=dag, clusters=ordered)
        self.cache.put(graph_hash, artifact)
        self.stats["compiled"] += 1
        self.stats["seconds"] += time.perf_counter() - t0
        logger.info("compiled %s: %d nodes -> %d kernels", name, len(dag.nodes),
                    sum(1 for l in launches if l.template))
        tracer.trace_graph_hash(graph_hash, {"kernel": name, "nodes": len(dag.nodes), "clusters": len(clusters)})
        tracer.trace_dag(dag)
        tracer.trace_dsl(plan_text)
        tracer.trace_compilation(
            ["parse_fx_graph", "identify_fusion_opportunities", "schedule_clusters", "select_templates"],
            {"kernel": name, "kernels": sum(1 for l in launches if l.template), "aliases": sum(1 for l in launches if not l.template),
             "seconds": round(time.perf_counter() - t0, 6), "library": str(library_path())})
        manager = get_debug_manager()
        if manager.enabled():
            manager.save_compilation(name, graph_module, self.graph_analyzer.describe(dag), plan_text, launches)
        return artifact

    def clear_cache(self) -> None:
        self.cache.clear()
