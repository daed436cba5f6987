"""FX -> DAG analysis, buffer scoping and fusion clustering (reference: ``conductor/optimization/``)."""
from .buffers import Buffer, BufferManager, BufferScope
from .fusion import FusionCluster, FusionEngine, FusionHeuristics, FusionType, LocalPriorityFusionEngine
from .graph_analyzer import ComputationDAG, GraphAnalyzer
from .graph_nodes import ConductorNode

__all__ = ["Buffer", "BufferManager", "BufferScope", "FusionCluster", "FusionEngine", "FusionHeuristics",
           "FusionType", "LocalPriorityFusionEngine", "ComputationDAG", "GraphAnalyzer", "ConductorNode"]
