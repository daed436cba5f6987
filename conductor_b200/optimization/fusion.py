"""Fusion clustering (reference: ``conductor/optimization/fusion.py:30-1103``).

The data model is the reference's: a :class:`FusionCluster` owns nodes, a
:class:`FusionType`, external inputs / outputs and internal buffers, and can validate
itself; :class:`FusionEngine.identify_fusion_opportunities` returns the clusters of a DAG,
:class:`LocalPriorityFusionEngine` is the entry the compiler uses.

The rules are new.  The reference's engine only ever yields ``elementwise[mul,add]`` for
the benchmark graphs (relu is typed ACTIVATION and blocks chains; softmax / linear / sdpa
are unknown to it).  Here every kernel-bearing node lands in exactly one cluster and each
cluster maps to one hand-written kernel template:

=================  ==========================================  =====================
cluster type       pattern                                     kernel template
=================  ==========================================  =====================
ELEMENTWISE        connected elementwise nodes of one shape    elementwise chain
REDUCTION          elementwise producers -> sum/mean/amax      chain + row reduce
SOFTMAX            softmax | _softmax_backward_data |          online softmax fwd/bwd
                   mul,sum(keepdim),sub,mul written out
GEMM_EPILOGUE      linear [-> relu]                            tcgen05 GEMM epilogue
ATTENTION          scaled_dot_product_attention                fused attention
SHAPE              view / reshape / flatten ...                none (alias)
=================  ==========================================  =====================
"""
from __future__ import annotations

from dataclasses import dataclass, field
from enum import Enum
from typing import Dict, Optional

from ..codegen.operator_registry import OpType, get_op_desc
from ..utils.constants import BufferScope, FusionLevel
from ..utils.logging import get_logger
from .buffers import Buffer
from .graph_nodes import ConductorNode

logger = get_logger(__name__)

# limits of one elementwise program (include/conductor_b200.h)
MAX_EW_INSTR = 24
# instructions the program builder emits for each written-out activation / selection
_COMPOSITE_INSTR = {"leaky_relu": 5, "elu": 6, "softplus": 8, "hardswish": 7, "hardsigmoid": 6, "masked_fill": 2,
                    "lerp": 3, "dropout": 1}
MAX_EW_INPUTS = 8
MAX_EW_OUTPUTS = 4

HBM_BYTES_PER_S = 6.5e12     # measured copy bandwidth class of one B200
LAUNCH_SECONDS = 3e-6        # cost of one extra kernel launch


class FusionType(Enum):
    ELEMENTWISE = "elementwise"
    REDUCTION = "reduction"
    MIXED = "mixed"
    MEMORY_BOUND = "memory_bound"
    COMPUTE_BOUND = "compute_bound"
    SOFTMAX = "softmax"
    GEMM_EPILOGUE = "gemm_epilogue"
    ATTENTION = "attention"
    NORM = "norm"
    SHAPE = "shape"
    UNKNOWN = "unknown"


@dataclass(eq=False)
class FusionCluster:
    nodes: list[ConductorNode] = field(default_factory=list)
    cluster_type: FusionType = FusionType.ELEMENTWISE
    external_inputs: list[Buffer] = field(default_factory=list)
    external_outputs: list[Buffer] = field(default_factory=list)
    internal_buffers: list[Buffer] = field(default_factory=list)
    dsl_function_name: str = ""          # name of the kernel instance in plans and traces
    fusion_level: FusionLevel = FusionLevel.GLOBAL
    pattern: str = ""                    # sub-kind, e.g. "softmax_bwd_written_out"

    def __hash__(self) -> int:
        return id(self)

    # -- description ---------------------------------------------------------
    def signature(self) -> str:
        return f"{self.cluster_type.value}[{','.join(n.op_name for n in self.nodes)}]"

    # -- validation (reference: fusion.py:61-185) -----------------------------
    def validate_fusion_safety(self) -> bool:
        if not self.nodes:
            return True
        if self.cluster_type in (FusionType.ELEMENTWISE, FusionType.REDUCTION):
            for i, a in enumerate(self.nodes):
                for b in self.nodes[i + 1:]:
                    if not a.can_fuse_with(b):
                        return False
        return self._validate_data_dependencies() and not self._has_cycles() and self._validate_buffer_usage()

    def _validate_data_dependencies(self) -> bool:
        produced = {b for n in self.nodes for b in n.outputs}
        ext = set(self.external_inputs)
        return all(b in produced or b in ext for n in self.nodes for b in n.inputs)

    def _has_cycles(self) -> bool:
        try:
            self._topological_sort()
            return False
        except ValueError:
            return True

    def _validate_buffer_usage(self) -> bool:
        inside = set(self.nodes)
        for buf in self.internal_buffers:
            if buf.producer not in inside:
                return False
            if buf.is_output or any(c not in inside for c in buf.consumers):
                return False
        return True

    def _topological_sort(self) -> list[ConductorNode]:
        inside = set(self.nodes)
        indeg = {n: 0 for n in self.nodes}
        succ: Dict[ConductorNode, list] = {n: [] for n in self.nodes}
        for n in self.nodes:
            for p in {b.producer for b in n.inputs if b.producer in inside and b.producer is not n}:
                succ[p].append(n)
                indeg[n] += 1
        ready = [n for n in self.nodes if indeg[n] == 0]
        order = []
        while ready:
            n = ready.pop(0)
            order.append(n)
            for m in succ[n]:
                indeg[m] -= 1
                if indeg[m] == 0:
                    ready.append(m)
        if len(order) != len(self.nodes):
            raise ValueError("cycle inside fusion cluster")
        return order

    # -- heuristics (reference: fusion.py:268-353) ------------------------------
    def estimate_performance_gain(self) -> float:
        """Seconds saved against running every node as its own kernel: each internal buffer
        is one HBM write plus one read avoided, each extra node one launch avoided."""
        saved_bytes = sum(2 * max(b.memory_size, 0) for b in self.internal_buffers)
        return saved_bytes / HBM_BYTES_PER_S + max(len(self.nodes) - 1, 0) * LAUNCH_SECONDS

    def get_fusion_priority(self) -> int:
        base = self.fusion_level.priority * 100
        return base + min(len(self.nodes), 50)

    def generate_fused_dsl(self) -> str:
        """Text form of the cluster (the reference prints Choreo DSL here, ``fusion.py:187-226``);
        this build prints the kernel-plan line the cluster lowers to."""
        ins = ", ".join(b.name for b in self.external_inputs)
        outs = ", ".join(b.name for b in self.external_outputs)
        return f"{outs} = {self.signature()}({ins})"


class FusionHeuristics:
    """Pairwise fusability and cost estimates (reference: ``fusion.py:914-1103``)."""

    def can_fuse_elementwise(self, op1: str, op2: str) -> bool:
        a, b = get_op_desc(op1), get_op_desc(op2)
        if a is None or b is None:
            return False
        ta, tb = a.operation_type, b.operation_type
        ew, red = OpType.ELEMENTWISE, OpType.REDUCTION
        if ta is ew and tb is ew:
            return a.fusable and b.fusable
        if {ta, tb} == {ew, red}:
            return True
        if ta is OpType.MATRIX and tb is ew:      # GEMM epilogue
            return op2 in ("relu", "add")
        return False

    def estimate_fusion_benefit(self, nodes: list[ConductorNode]) -> float:
        inside = set(nodes)
        internal = [b for n in nodes for b in n.outputs
                    if b.consumers and all(c in inside for c in b.consumers) and not b.is_output]
        return FusionCluster(nodes=list(nodes), internal_buffers=internal).estimate_performance_gain()

    @staticmethod
    def instruction_estimate(node: ConductorNode) -> int:
        """Upper bound on the program instructions one elementwise node lowers to: composites and
        clamps expand into several opcodes, and every Python-number operand may cost a CONST."""
        if not node.is_elementwise():
            return 0
        info = get_op_desc(node.op_name)
        canon = info.canonical_name if info is not None else node.op_name
        if canon == "composite":
            return _COMPOSITE_INSTR.get(node.op_name.rstrip("_"), 8)
        if canon == "clamp":
            return 4
        if canon in ("add", "sub", "mul", "div"):            # immediate forms: no CONST
            return 1
        consts = sum(1 for k, _ in node.metadata.get("arg_spec", []) if k == "const")
        return 1 + consts

    def check_memory_constraints(self, cluster: FusionCluster) -> bool:
        n_instr = sum(self.instruction_estimate(n) for n in cluster.nodes)
        return (n_instr <= MAX_EW_INSTR and len(cluster.external_inputs) <= MAX_EW_INPUTS
                and len(cluster.external_outputs) <= max(MAX_EW_OUTPUTS, 1))


def _is_last_dim_reduction(node: ConductorNode) -> Optional[bool]:
    """True: reduces exactly the last dim; None: reduces everything; False: anything else."""
    if not node.is_reduction() or not node.inputs or node.inputs[0].shape is None:
        return False
    rank = len(node.inputs[0].shape)
    kw = node.metadata.get("kwargs", {})
    consts = [v for k, v in node.metadata.get("arg_spec", []) if k == "const"]
    dim = kw.get("dim", consts[0] if consts else None)
    if dim is None:
        return None
    if isinstance(dim, (list, tuple)):
        if len(dim) != 1:
            return sorted(d % rank for d in dim) == list(range(rank)) and None
        dim = dim[0]
    if not isinstance(dim, int) or rank == 0:
        return False
    return (dim % rank) == rank - 1


class FusionEngine:
    """Builds the cluster list of a DAG (reference: ``fusion.py:592-911``)."""

    def __init__(self):
        self.heuristics = FusionHeuristics()

    # ------------------------------------------------------------------ entry
    def identify_fusion_opportunities(self, dag, enable_fusion: bool = True) -> list[FusionCluster]:
        from .dag_naming import DAGTopologicalSorter

        order = DAGTopologicalSorter().sort(dag)
        pos = {n: i for i, n in enumerate(order)}
        ancestors = self._ancestors(order)
        claimed: Dict[ConductorNode, FusionCluster] = {}
        clusters: list[FusionCluster] = []

        def claim(nodes, ctype, level=FusionLevel.GLOBAL, pattern=""):
            nodes = sorted(nodes, key=pos.get)
            c = FusionCluster(nodes=nodes, cluster_type=ctype, fusion_level=level, pattern=pattern)
            for n in nodes:
                claimed[n] = c
            clusters.append(c)
            return c

        if enable_fusion:
            for n in order:                                   # written-out softmax backward
                if n not in claimed:
                    grp = self._match_softmax_backward(n, claimed)
                    if grp:
                        claim(grp, FusionType.SOFTMAX, pattern="softmax_bwd_written_out")
            for n in order:                                   # linear / matmul / addmm (+relu epilogue)
                info = get_op_desc(n.op_name)
                if n in claimed or info is None or info.operation_type is not OpType.MATRIX:
                    continue
                grp = [n]
                out = n.outputs[0]
                if len(out.consumers) == 1 and not out.is_output:
                    c = out.consumers[0]
                    if c.op_name == "relu" and c not in claimed:
                        grp.append(c)
                claim(grp, FusionType.GEMM_EPILOGUE)
            for n in order:                                   # elementwise producers -> reduction
                if n in claimed or not n.is_reduction():
                    continue
                if _is_last_dim_reduction(n) is False:
                    continue
                grp = self._grow_reduction(n, claimed)
                claim(grp, FusionType.REDUCTION)
            for n in order:                                   # elementwise groups
                if n in claimed or not n.is_elementwise():
                    continue
                grp = self._grow_elementwise(n, order, pos, claimed, ancestors)
                claim(grp, FusionType.ELEMENTWISE, FusionLevel.LOCAL)

        for n in order:                                       # everything else: one node each
            if n in claimed:
                continue
            info = get_op_desc(n.op_name)
            if info is None:
                ctype = FusionType.UNKNOWN
            else:
                ctype = {
                    OpType.ELEMENTWISE: FusionType.ELEMENTWISE, OpType.REDUCTION: FusionType.REDUCTION,
                    OpType.MATRIX: FusionType.GEMM_EPILOGUE, OpType.SOFTMAX: FusionType.SOFTMAX,
                    OpType.ATTENTION: FusionType.ATTENTION, OpType.SHAPE: FusionType.SHAPE,
                    OpType.NORM: FusionType.NORM,
                }.get(info.operation_type, FusionType.UNKNOWN)
            claim([n], ctype)

        for i, c in enumerate(clusters):
            self._populate_cluster_buffers(c, dag)
            self.optimize_buffer_usage(c)
            c.dsl_function_name = f"k{i}_{c.cluster_type.value}_" + "_".join(n.op_name for n in c.nodes)[:48]
        clusters.sort(key=lambda c: (-c.get_fusion_priority(), -c.estimate_performance_gain()))
        return clusters

    # ------------------------------------------------------------------ helpers
    @staticmethod
    def _ancestors(order) -> Dict[ConductorNode, set]:
        anc: Dict[ConductorNode, set] = {}
        for n in order:
            s = set()
            for b in n.inputs:
                p = b.producer
                if p is not None and p in anc:
                    s.add(p)
                    s |= anc[p]
            anc[n] = s
        return anc

    def _is_elementwise_op(self, op_name: str) -> bool:
        info = get_op_desc(op_name)
        return bool(info and info.is_elementwise() and info.fusable)

    def _is_reduction_op(self, op_name: str) -> bool:
        info = get_op_desc(op_name)
        return bool(info and info.is_reduction())

    def _grow_elementwise(self, seed, order, pos, claimed, ancestors) -> list[ConductorNode]:
        """Largest connected set of unclaimed elementwise nodes with the seed's output shape that
        can run as one kernel: joining a consumer must not pull in a dependency on the cluster
        through a node outside it."""
        shape = seed.outputs[0].shape
        group = [seed]
        inside = {seed}
        changed = True
        while changed:
            changed = False
            for n in order:
                if n in inside or n in claimed or not n.is_elementwise() or not self._is_elementwise_op(n.op_name):
                    continue
                if n.outputs[0].shape != shape or shape is None:
                    continue
                producers = {b.producer for b in n.inputs if b.producer is not None}
                consumers = {c for b in n.outputs for c in b.consumers}
                touches = bool(producers & inside) or bool(consumers & inside)
                if not touches:
                    continue
                # outside producers of n must not descend from the cluster, and outside
                # consumers of the cluster that feed n are excluded by the same test
                if any((ancestors[p] & inside) for p in producers - inside):
                    continue
                # n as a producer of the cluster: cluster members must not reach n via outsiders
                bad = False
                for m in inside:
                    for p in {b.producer for b in m.inputs if b.producer is not None} - inside - {n}:
                        if n in ancestors[p]:
                            bad = True
                if bad:
                    continue
                trial = group + [n]
                if not self._fits_one_program(trial):
                    continue
                group.append(n)
                inside.add(n)
                changed = True
        return group

    def _fits_one_program(self, nodes) -> bool:
        inside = set(nodes)
        ext_in = {b for n in nodes for b in n.inputs if b.producer not in inside}
        ext_out = {b for n in nodes for b in n.outputs
                   if b.is_output or any(c not in inside for c in b.consumers)}
        n_instr = sum(FusionHeuristics.instruction_estimate(n) for n in nodes)
        return n_instr <= MAX_EW_INSTR - 4 and len(ext_in) <= MAX_EW_INPUTS and len(ext_out) <= MAX_EW_OUTPUTS

    def _grow_reduction(self, red, claimed) -> list[ConductorNode]:
        """The reduction plus the elementwise producers that feed only it (transitively)."""
        group = [red]
        inside = {red}
        full_shape = red.inputs[0].shape
        frontier = [red]
        while frontier:
            n = frontier.pop()
            for b in n.inputs:
                p = b.producer
                if p is None or p in inside or p in claimed or not self._is_elementwise_op(p.op_name):
                    continue
                if b.is_output or any(c not in inside for c in b.consumers):
                    continue
                if b.shape != full_shape:
                    continue
                trial_in = {x for m in group + [p] for x in m.inputs if x.producer not in inside | {p}}
                n_instr = sum(FusionHeuristics.instruction_estimate(m) for m in group + [p])
                if n_instr > MAX_EW_INSTR - 4 or len(trial_in) > MAX_EW_INPUTS:
                    continue
                group.append(p)
                inside.add(p)
                frontier.append(p)
        return group

    def _match_softmax_backward(self, last, claimed) -> Optional[list[ConductorNode]]:
        """``mul(y, sub(g, sum(mul(g, y), -1, keepdim=True)))`` in any operand order."""
        if last.op_name != "mul" or len(last.inputs) != 2:
            return None
        for y, sub_buf in (last.inputs, last.inputs[::-1]):
            sub = sub_buf.producer
            if sub is None or sub.op_name != "sub" or sub in claimed or len(sub.inputs) != 2:
                continue
            if len(sub_buf.consumers) != 1 or sub_buf.is_output:
                continue
            spec = sub.metadata.get("arg_spec", [])
            if len(spec) != 2 or spec[0][0] != "buf" or spec[1][0] != "buf":
                continue
            g, s_buf = sub.inputs[spec[0][1]], sub.inputs[spec[1][1]]
            red = s_buf.producer
            if red is None or red.op_name != "sum" or red in claimed or len(s_buf.consumers) != 1 or s_buf.is_output:
                continue
            if _is_last_dim_reduction(red) is not True:
                continue
            kw = red.metadata.get("kwargs", {})
            consts = [v for k, v in red.metadata.get("arg_spec", []) if k == "const"]
            keep = kw.get("keepdim", consts[1] if len(consts) > 1 else False)
            if not keep:
                continue
            inner_buf = red.inputs[0]
            inner = inner_buf.producer
            if inner is None or inner.op_name != "mul" or inner in claimed or len(inner.inputs) != 2:
                continue
            if len(inner_buf.consumers) != 1 or inner_buf.is_output:
                continue
            if set(inner.inputs) != {g, y} or g is y:
                continue
            if g.shape != y.shape or g.dtype != y.dtype or last.outputs[0].shape != y.shape:
                continue
            grp = [inner, red, sub, last]
            for n in grp:
                n.metadata["softmax_bwd_roles"] = {"grad": g, "y": y}
            return grp
        return None

    def _populate_cluster_buffers(self, cluster: FusionCluster, dag) -> None:
        """External inputs: read by the cluster, produced outside.  External outputs: produced
        inside and either a graph output or read outside.  The rest is internal
        (reference: ``fusion.py:746-785``)."""
        inside = set(cluster.nodes)
        ext_in, ext_out, internal = [], [], []
        for n in cluster.nodes:
            for b in n.inputs:
                if b.producer not in inside and b not in ext_in:
                    ext_in.append(b)
        for n in cluster.nodes:
            for b in n.outputs:
                if b.is_output or not b.consumers or any(c not in inside for c in b.consumers):
                    if b not in ext_out:
                        ext_out.append(b)
                elif b not in internal:
                    internal.append(b)
        cluster.external_inputs, cluster.external_outputs, cluster.internal_buffers = ext_in, ext_out, internal

    def optimize_buffer_usage(self, cluster: FusionCluster) -> None:
        """Values that never leave the kernel live in registers: LOCAL; values written to HBM
        for a later kernel of the same plan are SHARED unless they cross the graph boundary
        (reference: ``fusion.py:839-844,892-911``)."""
        for b in cluster.internal_buffers:
            b.scope = BufferScope.LOCAL
            b.is_temporary = True
        for b in cluster.external_outputs:
            if not b.is_output and b.scope is BufferScope.LOCAL:
                b.scope = BufferScope.SHARED

    # kept for API parity with the reference (fusion.py:846-890)
    def apply_elementwise_fusion(self, nodes: list[ConductorNode]) -> FusionCluster:
        c = FusionCluster(nodes=list(nodes), cluster_type=FusionType.ELEMENTWISE, fusion_level=FusionLevel.LOCAL)
        self._populate_cluster_buffers(c, None)
        return c

    def apply_reduction_fusion(self, nodes: list[ConductorNode]) -> FusionCluster:
        c = FusionCluster(nodes=list(nodes), cluster_type=FusionType.REDUCTION)
        self._populate_cluster_buffers(c, None)
        return c


class LocalPriorityFusionEngine(FusionEngine):
    """Entry point used by the compiler (reference: ``fusion.py:356-589``).  The reference runs a
    local phase, an (empty) adjacent phase and a global phase; here the phases are the rule
    order inside :meth:`FusionEngine.identify_fusion_opportunities` and the phase that formed a
    cluster is recorded in ``FusionCluster.fusion_level``."""


def schedule_clusters(clusters: list[FusionCluster]) -> list[FusionCluster]:
    """Execution order: topological over cluster-level producer/consumer edges."""
    owner = {n: c for c in clusters for n in c.nodes}
    indeg = {c: 0 for c in clusters}
    succ: Dict[FusionCluster, list] = {c: [] for c in clusters}
    first_pos = {}
    for c in clusters:
        for b in c.external_inputs:
            p = owner.get(b.producer)
            if p is not None and p is not c and c not in succ[p]:
                succ[p].append(c)
                indeg[c] += 1
    for c in clusters:
        first_pos[c] = min((b.birth_time for n in c.nodes for b in n.outputs), default=0)
    ready = sorted((c for c in clusters if indeg[c] == 0), key=first_pos.get)
    order = []
    while ready:
        c = ready.pop(0)
        order.append(c)
        for m in succ[c]:
            indeg[m] -= 1
            if indeg[m] == 0:
                ready.append(m)
        ready.sort(key=first_pos.get)
    if len(order) != len(clusters):
        raise ValueError("cluster graph contains a cycle")
    return order
