"""FX graph -> internal DAG (reference: ``conductor/optimization/graph_analyzer.py:24-809``).

Same public surface as the reference (``ComputationDAG``, ``GraphAnalyzer.parse_fx_graph``,
``identify_data_dependencies``, ``validate_graph_correctness``) with two behavioural fixes
the kernel-template path depends on:

* shapes and dtypes of every intermediate come from the FakeTensor Dynamo stores in
  ``node.meta['example_value']`` (the reference reads only ``tensor_meta`` / ``val``,
  ``graph_analyzer.py:502-531``, so ``linear`` / ``softmax`` / ``sdpa`` outputs end up
  shapeless); graphs from ``fx.symbolic_trace`` get the same information by running
  FakeTensor propagation over the example inputs;
* operands keep their positions (``metadata['arg_spec']``), python scalars included, so
  that ``x * 2`` or ``addcdiv(a, b, c, value=v)`` can be lowered.
"""
from __future__ import annotations

import re
from dataclasses import dataclass, field
from typing import Any, Optional

import torch

from ..codegen.operation_factory import get_operation_factory
from ..utils.constants import BufferScope
from ..utils.exceptions import UnsupportedOperationError
from ..utils.logging import get_logger
from .buffers import Buffer, BufferManager
from .graph_nodes import ConductorNode

logger = get_logger(__name__)


@dataclass
class ComputationDAG:
    """Nodes, buffers and the graph boundary (reference: ``graph_analyzer.py:24-78``)."""

    nodes: list[ConductorNode] = field(default_factory=list)
    buffers: list[Buffer] = field(default_factory=list)
    inputs: list[Buffer] = field(default_factory=list)
    outputs: list[Buffer] = field(default_factory=list)
    # how the FX output node is rebuilt: entries are Buffer objects or python constants
    output_spec: list[Any] = field(default_factory=list)
    output_is_sequence: bool = True

    def add_node(self, node: ConductorNode) -> None:
        self.nodes.append(node)

    def add_buffer(self, buffer: Buffer) -> None:
        self.buffers.append(buffer)

    def get_buffer(self, name: str) -> Optional[Buffer]:
        for b in self.buffers:
            if b.name == name:
                return b
        return None

    def validate_graph_correctness(self) -> bool:
        """Every buffer a node or the boundary names must be registered in the DAG, every
        non-input buffer must have a producer, and the producer graph must be acyclic."""
        try:
            known = set(self.buffers)
            for node in self.nodes:
                if any(b not in known for b in node.inputs) or any(b not in known for b in node.outputs):
                    return False
            if any(b not in known for b in self.inputs) or any(b not in known for b in self.outputs):
                return False
            from .dag_naming import DAGTopologicalSorter

            DAGTopologicalSorter().sort(self)
            return True
        except Exception:
            return False


def _sanitize(name: str) -> str:
    s = re.sub(r"[^0-9a-zA-Z_]", "_", str(name))
    return s if s and not s[0].isdigit() else f"buf_{s}"


# calls that return a tuple of views of their first argument
_MULTI_VIEW_OPS = ("chunk", "split", "unbind", "tensor_split", "split_with_sizes")


def _meta_tensor(node: torch.fx.Node):
    """(shape, dtype) recorded on an FX node, or None."""
    meta = node.meta
    for key in ("example_value", "val"):
        v = meta.get(key)
        if isinstance(v, torch.Tensor):
            try:
                return tuple(int(d) for d in v.shape), v.dtype
            except Exception:  # symbolic dims
                return None
    tm = meta.get("tensor_meta")
    if tm is not None and hasattr(tm, "shape"):
        return tuple(int(d) for d in tm.shape), tm.dtype
    return None


class GraphAnalyzer:
    """Builds the :class:`ComputationDAG` for one FX graph."""

    def __init__(self):
        self.buffer_manager = BufferManager()
        self._node_to_buffer: dict[torch.fx.Node, Buffer] = {}
        self._buffer_to_node: dict[Buffer, ConductorNode] = {}
        self._factory = get_operation_factory()

    # ------------------------------------------------------------------ entry
    def parse_fx_graph(
        self,
        graph_module: torch.fx.GraphModule,
        example_inputs: Optional[list[torch.Tensor]] = None,
        enable_shape_inference: bool = True,
    ) -> ComputationDAG:
        if graph_module is None:
            raise ValueError("graph_module cannot be None")
        self.buffer_manager.reset()
        self._node_to_buffer.clear()
        self._buffer_to_node.clear()
        dag = ComputationDAG()

        if enable_shape_inference:
            self._ensure_meta(graph_module, example_inputs)

        for node in graph_module.graph.nodes:          # pass 1: one buffer per FX value
            self._create_buffer_for_node(node, dag, graph_module)
        for node in graph_module.graph.nodes:          # pass 2: operation nodes
            cnode = self._convert_fx_node(node, dag, graph_module)
            if cnode is not None:
                dag.add_node(cnode)
        self._identify_graph_inputs_outputs(graph_module.graph, dag, example_inputs)
        if enable_shape_inference:
            self._propagate_shapes(dag)
        self.identify_data_dependencies(dag)
        self.buffer_manager.analyze_buffer_lifetimes(dag)
        return dag

    # ------------------------------------------------------------------ meta
    def _ensure_meta(self, gm: torch.fx.GraphModule, example_inputs) -> None:
        """Run FakeTensor propagation when the tracer left no shape information."""
        nodes = [n for n in gm.graph.nodes if n.op in ("call_function", "call_method", "call_module")]
        if not nodes or all(_meta_tensor(n) is not None for n in nodes):
            return
        placeholders = [n for n in gm.graph.nodes if n.op == "placeholder"]
        if example_inputs is None or len(example_inputs) != len(placeholders):
            return
        if not all(isinstance(t, torch.Tensor) for t in example_inputs):
            return
        try:
            from torch.fx.passes.fake_tensor_prop import FakeTensorProp

            FakeTensorProp(gm).propagate(*example_inputs)
        except Exception as exc:  # unsupported op under fake mode: keep going without shapes
            logger.debug("fake tensor propagation failed: %s", exc)

    # ------------------------------------------------------------------ pass 1
    def _create_buffer_for_node(self, node: torch.fx.Node, dag: ComputationDAG, gm) -> None:
        if node.op == "output":
            return
        shape, dtype = None, torch.float32
        info = _meta_tensor(node)
        if info is not None:
            shape, dtype = info
        const = None
        if node.op == "get_attr":
            const = self._fetch_attr(gm, node.target)
            if isinstance(const, torch.Tensor):
                shape, dtype = tuple(const.shape), const.dtype
        buf = self.buffer_manager.allocate_buffer(_sanitize(node.name), dtype, shape, BufferScope.LOCAL)
        buf.constant_value = const
        self._node_to_buffer[node] = buf
        dag.add_buffer(buf)

    @staticmethod
    def _fetch_attr(gm, target: str):
        obj = gm
        for part in str(target).split("."):
            obj = getattr(obj, part)
        return obj

    # ------------------------------------------------------------------ pass 2
    def _convert_fx_node(self, node: torch.fx.Node, dag: ComputationDAG, gm) -> Optional[ConductorNode]:
        if node.op not in ("call_function", "call_method", "call_module"):
            return None
        op_name = self._factory.extract_operation_name(node)
        args = list(node.args)
        kwargs = dict(node.kwargs)
        extra_const: list[Buffer] = []
        if op_name in _MULTI_VIEW_OPS:
            # chunk / split / unbind return a tuple of views; the tuple itself is no value of the
            # plan -- each getitem on it becomes a slice of the tuple op's own input
            if any(u.op != "call_function" or self._factory.extract_operation_name(u) not in ("getitem", "__getitem__")
                   for u in node.users):
                raise UnsupportedOperationError(op_name, "the tuple of views is used other than by indexing")
            return None
        view_call = None
        if op_name in ("getitem", "__getitem__") and isinstance(args[0], torch.fx.Node) and \
                args[0].op in ("call_function", "call_method") and \
                self._factory.extract_operation_name(args[0]) in _MULTI_VIEW_OPS:
            tup = args[0]
            if not isinstance(args[1], int) or not tup.args or not isinstance(tup.args[0], torch.fx.Node) or \
                    any(isinstance(a, torch.fx.Node) for a in list(tup.args[1:]) + list(tup.kwargs.values())):
                raise UnsupportedOperationError(op_name, "unsupported indexing of a tuple of views")
            view_call = (self._factory.extract_operation_name(tup), tuple(tup.args[1:]), dict(tup.kwargs), args[1])
            op_name, args, kwargs = "view_of", [tup.args[0]], {}
        if node.op == "call_module":
            op_name, args, kwargs, extra_const = self._lower_module_call(node, gm, dag)

        cnode = ConductorNode(op_name=op_name)
        cnode.metadata["fx_name"] = node.name
        cnode.metadata["fx_op"] = node.op
        cnode.metadata["fx_target"] = node.target
        if view_call is not None:
            cnode.metadata["view_call"] = view_call
        arg_spec = []
        for a in args:
            arg_spec.append(self._bind_operand(a, cnode))
        kw_spec = {k: self._bind_operand(v, cnode) for k, v in kwargs.items()}
        for cbuf in extra_const:
            cnode.add_input(cbuf)
            arg_spec.append(("buf", cnode.inputs.index(cbuf)))
        cnode.metadata["arg_spec"] = arg_spec
        cnode.metadata["kwarg_spec"] = kw_spec
        cnode.metadata["kwargs"] = {k: v[1] for k, v in kw_spec.items() if v[0] == "const"}

        out = self._node_to_buffer[node]
        out.producer = cnode
        cnode.add_output(out)
        self._buffer_to_node[out] = cnode
        self._rebind_mutated_operand(node, op_name, out)
        return cnode

    # in-place updates ------------------------------------------------------------------
    _INPLACE_OPERATORS = ("iadd", "isub", "imul", "itruediv", "ifloordiv", "ipow", "imod", "iand", "ior", "ixor")

    def _rebind_mutated_operand(self, node: torch.fx.Node, op_name: str, out: Buffer) -> None:
        """``h.relu_()``, ``h += y`` and ``F.relu(h, inplace=True)`` change ``h`` itself, but FX keeps
        later readers pointing at the node that produced ``h``.  The plan computes the update out
        of place, so every later reader of the mutated value is redirected to the update's result.
        Updating a graph input in place (the caller's tensor would have to change) or a view of
        another value (the base would have to change too) is refused instead of computed wrongly."""
        raw = str(node.target) if node.op == "call_method" else getattr(node.target, "__name__", str(node.target))
        inplace = (raw.endswith("_") and not raw.endswith("__")) or raw.strip("_") in self._INPLACE_OPERATORS \
            or node.kwargs.get("inplace") is True
        if not inplace or not node.args or not isinstance(node.args[0], torch.fx.Node):
            return
        target = node.args[0]
        if target.op in ("placeholder", "get_attr"):
            raise UnsupportedOperationError(op_name, "in-place update of a graph input or constant; write the result to a new tensor")
        from ..codegen.operator_registry import OpType, get_operator_registry

        producer = self._buffer_to_node.get(self._node_to_buffer[target])
        info = get_operator_registry().get_operation(producer.op_name) if producer is not None else None
        if info is not None and info.operation_type == OpType.SHAPE and producer.op_name not in ("cat", "concat", "concatenate", "contiguous"):
            raise UnsupportedOperationError(op_name, "in-place update through a view of another value")
        self._node_to_buffer[target] = out

    def _bind_operand(self, a: Any, cnode: ConductorNode):
        if isinstance(a, torch.fx.Node):
            buf = self._node_to_buffer[a]
            cnode.add_input(buf)
            return ("buf", cnode.inputs.index(buf))
        if isinstance(a, (list, tuple)) and any(isinstance(x, torch.fx.Node) for x in a):
            return ("seq", [self._bind_operand(x, cnode) for x in a])
        return ("const", a)

    def _lower_module_call(self, node, gm, dag):
        """``call_module`` of a leaf nn.Module -> functional op + constant buffers."""
        mod = gm.get_submodule(node.target)
        args, kwargs, consts = list(node.args), dict(node.kwargs), []

        def const_buffer(suffix: str, tensor: torch.Tensor) -> Buffer:
            buf = self.buffer_manager.allocate_buffer(_sanitize(f"{node.target}_{suffix}"), tensor.dtype,
                                                      tuple(tensor.shape), BufferScope.GLOBAL)
            buf.constant_value = tensor
            dag.add_buffer(buf)
            return buf

        if isinstance(mod, torch.nn.Linear):
            consts.append(const_buffer("weight", mod.weight))
            if mod.bias is not None:
                consts.append(const_buffer("bias", mod.bias))
            return "linear", args, kwargs, consts
        if isinstance(mod, torch.nn.ReLU):
            return "relu", args, kwargs, consts
        if isinstance(mod, torch.nn.Sigmoid):
            return "sigmoid", args, kwargs, consts
        if isinstance(mod, torch.nn.Tanh):
            return "tanh", args, kwargs, consts
        if isinstance(mod, torch.nn.Softmax):
            kwargs = dict(kwargs, dim=mod.dim)
            return "softmax", args, kwargs, consts
        return type(mod).__name__.lower(), args, kwargs, consts

    # ------------------------------------------------------------------ boundary
    def _identify_graph_inputs_outputs(self, graph: torch.fx.Graph, dag: ComputationDAG,
                                       example_inputs: Optional[list[torch.Tensor]] = None) -> None:
        placeholders = [n for n in graph.nodes if n.op == "placeholder"]
        if example_inputs is not None and len(example_inputs) != len(placeholders):
            raise ValueError(
                f"graph has {len(placeholders)} placeholders but {len(example_inputs)} example inputs were given")
        for i, node in enumerate(placeholders):
            buf = self._node_to_buffer[node]
            buf.is_input = True
            buf.scope = BufferScope.GLOBAL
            if example_inputs is not None and isinstance(example_inputs[i], torch.Tensor):
                buf.set_shape(tuple(example_inputs[i].shape), example_inputs[i].dtype)
            dag.inputs.append(buf)
        for node in graph.nodes:
            if node.op != "output":
                continue
            ret = node.args[0] if node.args else None
            dag.output_is_sequence = isinstance(ret, (list, tuple))
            items = list(ret) if dag.output_is_sequence else [ret]
            for item in items:
                if isinstance(item, torch.fx.Node):
                    buf = self._node_to_buffer[item]
                    buf.is_output = True
                    buf.scope = BufferScope.GLOBAL
                    if buf not in dag.outputs:
                        dag.outputs.append(buf)
                    dag.output_spec.append(buf)
                else:
                    dag.output_spec.append(item)

    # ------------------------------------------------------------------ shapes
    def _propagate_shapes(self, dag: ComputationDAG) -> None:
        """Fill in shapes the tracer did not record: broadcasting for elementwise ops,
        last-dim removal for reductions, [m,k]x[k,n] for matmul, [..,k]x[n,k] for linear
        (reference: ``graph_analyzer.py:217-343``)."""
        from .dag_naming import DAGTopologicalSorter

        try:
            order = DAGTopologicalSorter().sort(dag)
        except ValueError:
            order = dag.nodes
        for node in order:
            out = node.outputs[0] if node.outputs else None
            if out is None or out.shape is not None:
                continue
            shapes = [b.shape for b in node.inputs]
            if not shapes or any(s is None for s in shapes):
                continue
            dtypes = [b.dtype for b in node.inputs]
            try:
                if node.is_elementwise() or node.op_name in ("softmax", "_softmax_backward_data"):
                    out.set_shape(tuple(torch.broadcast_shapes(*shapes)), self._promote(dtypes))
                elif node.is_reduction():
                    kw = node.metadata.get("kwargs", {})
                    consts = [v for k, v in node.metadata.get("arg_spec", []) if k == "const"]
                    dim = kw.get("dim", consts[0] if consts else None)
                    keep = kw.get("keepdim", consts[1] if len(consts) > 1 else False)
                    s = list(shapes[0])
                    if dim is None:
                        s = []
                    else:
                        dims = sorted({d % len(s) for d in ([dim] if isinstance(dim, int) else dim)}, reverse=True)
                        for d in dims:
                            if keep:
                                s[d] = 1
                            else:
                                del s[d]
                    out.set_shape(tuple(s), kw.get("dtype") or dtypes[0])
                elif node.op_name == "matmul" and len(shapes) >= 2:
                    a, b = shapes[0], shapes[1]
                    if len(a) >= 2 and len(b) >= 2:
                        batch = torch.broadcast_shapes(a[:-2], b[:-2])
                        out.set_shape(tuple(batch) + (a[-2], b[-1]), self._promote(dtypes[:2]))
                elif node.op_name == "linear" and len(shapes) >= 2:
                    out.set_shape(tuple(shapes[0][:-1]) + (shapes[1][0],), dtypes[0])
                elif node.op_name == "scaled_dot_product_attention" and len(shapes) >= 3:
                    out.set_shape(tuple(shapes[0][:-1]) + (shapes[2][-1],), dtypes[0])
            except Exception as exc:
                logger.debug("shape propagation failed at %s: %s", node.name, exc)

    @staticmethod
    def _promote(dtypes):
        out = dtypes[0]
        for d in dtypes[1:]:
            out = torch.promote_types(out, d)
        return out

    # ------------------------------------------------------------------ dependencies / scopes
    def identify_data_dependencies(self, dag: ComputationDAG) -> None:
        """Record consumers on every buffer, then assign scopes (reference:
        ``graph_analyzer.py:600-647``): graph inputs/outputs and constants are GLOBAL, a value
        read by more than one node is SHARED, everything else stays LOCAL."""
        for buf in dag.buffers:
            buf.consumers = []
        for node in dag.nodes:
            for buf in node.inputs:
                if node not in buf.consumers:
                    buf.consumers.append(node)
        self._optimize_buffer_scopes(dag)

    def _optimize_buffer_scopes(self, dag: ComputationDAG) -> None:
        for buf in dag.buffers:
            if buf.is_input or buf.is_output or buf.constant_value is not None:
                buf.scope = BufferScope.GLOBAL
            elif len(buf.consumers) > 1:
                buf.scope = BufferScope.SHARED
            else:
                buf.scope = BufferScope.LOCAL
            buf.is_temporary = buf.scope is not BufferScope.GLOBAL

    # ------------------------------------------------------------------ reporting
    def describe(self, dag: ComputationDAG) -> str:
        """Human-readable buffer / node table (replaces the reference's
        ``_dump_buffer_state_table``, ``graph_analyzer.py:649-700``)."""
        lines = ["buffers:"]
        for b in dag.buffers:
            lines.append(f"  {b.name:<28} {b.scope.value:<7} {str(b.dtype):<15} {b.shape}")
        lines.append("nodes:")
        for n in dag.nodes:
            lines.append(f"  {n.name:<28} {n.op_name:<12} <- {[b.name for b in n.inputs]}")
        return "\n".join(lines)
