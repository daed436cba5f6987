"""FX graph -> DAG structure tests, written against the reference's import paths
(`conductor.optimization.*`).  They mirror what the reference's own suite checks
(tests/test_fx_to_dag_conversion.py, tests/unit/test_graph_simple.py): node counts, op names,
boundary buffers, shapes, dtypes, validation, error handling, long chains."""
import pytest
import torch
import torch.fx as fx
import torch.nn as nn

from conductor.optimization.buffers import Buffer, BufferManager, BufferScope
from conductor.optimization.graph_analyzer import ComputationDAG, GraphAnalyzer
from conductor.optimization.graph_nodes import ConductorNode


def parse(fn, *inputs):
    return GraphAnalyzer().parse_fx_graph(fx.symbolic_trace(fn), list(inputs))


def test_single_add():
    dag = parse(lambda x, y: torch.add(x, y), torch.randn(4, 4), torch.randn(4, 4))
    assert isinstance(dag, ComputationDAG)
    assert (len(dag.inputs), len(dag.outputs), len(dag.nodes)) == (2, 1, 1)
    node = dag.nodes[0]
    assert isinstance(node, ConductorNode) and node.op_name == "add"
    assert len(node.inputs) == 2 and len(node.outputs) == 1
    for buf in dag.inputs + dag.outputs:
        assert isinstance(buf, Buffer)
        assert buf.shape == (4, 4) and buf.dtype == torch.float32


def test_single_mul_keeps_shapes():
    dag = parse(lambda x, y: torch.mul(x, y), torch.randn(2, 8), torch.randn(2, 8))
    assert [n.op_name for n in dag.nodes] == ["mul"]
    assert all(b.shape == (2, 8) for b in dag.inputs + dag.outputs)


def test_three_op_chain():
    def model(x, y, z):
        return torch.relu((x + y) * z)

    dag = parse(model, *(torch.randn(3, 3) for _ in range(3)))
    assert [n.op_name for n in dag.nodes] == ["add", "mul", "relu"]
    assert len(dag.inputs) == 3 and len(dag.outputs) == 1
    assert dag.validate_graph_correctness()
    assert all(b.shape == (3, 3) for b in dag.buffers)


def test_branching_marks_shared_scope():
    def model(x):
        return torch.relu(x) + torch.sigmoid(x)

    dag = parse(model, torch.randn(5, 5))
    assert sorted(n.op_name for n in dag.nodes) == ["add", "relu", "sigmoid"]
    x = dag.inputs[0]
    assert len(x.consumers) == 2 and x.scope is BufferScope.GLOBAL


def test_scopes_local_shared_global():
    def model(x, y):
        t = x + y            # two consumers -> SHARED
        u = t * x            # one consumer  -> LOCAL
        return torch.relu(u) + t

    dag = parse(model, torch.randn(4, 4), torch.randn(4, 4))
    by_name = {b.name: b for b in dag.buffers}
    assert by_name["add"].scope is BufferScope.SHARED
    assert by_name["mul"].scope is BufferScope.LOCAL
    assert dag.outputs[0].scope is BufferScope.GLOBAL and all(b.scope is BufferScope.GLOBAL for b in dag.inputs)


def test_reduction_shape():
    def model(x, y):
        return torch.sum(torch.relu(x + y) * x)

    dag = parse(model, torch.randn(6, 7), torch.randn(6, 7))
    assert [n.op_name for n in dag.nodes] == ["add", "relu", "mul", "sum"]
    assert dag.outputs[0].shape == ()


def test_matmul_shape():
    dag = parse(lambda a, b: torch.matmul(a, b), torch.randn(4, 3), torch.randn(3, 5))
    assert dag.nodes[0].op_name == "matmul"
    assert dag.outputs[0].shape == (4, 5)


@pytest.mark.parametrize("shape", [(4,), (4, 4), (2, 3, 4), (1, 2, 3, 4)])
def test_ranks(shape):
    dag = parse(lambda x, y: x + y, torch.randn(shape), torch.randn(shape))
    assert dag.outputs[0].shape == shape


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64, torch.int32, torch.int64, torch.bfloat16])
def test_dtypes(dtype):
    a = torch.ones(4, 4, dtype=dtype)
    dag = parse(lambda x, y: x + y, a, a)
    assert all(b.dtype == dtype for b in dag.inputs + dag.outputs)


def test_no_none_shapes_for_intermediates():
    class M(nn.Module):
        def forward(self, x, y, z):
            return (x + y) * z

    dag = GraphAnalyzer().parse_fx_graph(fx.symbolic_trace(M()), [torch.randn(16, 32)] * 3)
    assert [b for b in dag.buffers if b.shape is None] == []
    assert all(b.shape == (16, 32) for b in dag.buffers)


def test_errors():
    with pytest.raises(ValueError):
        GraphAnalyzer().parse_fx_graph(None, [])
    gm = fx.symbolic_trace(lambda x, y: x + y)
    with pytest.raises(ValueError):
        GraphAnalyzer().parse_fx_graph(gm, [torch.randn(2)])          # wrong input count
    dag = GraphAnalyzer().parse_fx_graph(gm, None)                    # no example inputs: still a DAG
    assert len(dag.nodes) == 1 and len(dag.inputs) == 2


def test_long_chain_and_lifetimes():
    def model(x):
        for _ in range(20):
            x = x + 1.0
        return x

    dag = parse(model, torch.randn(8))
    assert len(dag.nodes) == 20 and dag.validate_graph_correctness()
    births = [b.birth_time for b in dag.buffers if b.producer is not None]
    assert births == sorted(births)
    out = dag.outputs[0]
    assert out.death_time == 20 and out.is_alive_at(20)


def test_python_scalars_and_kwargs_are_kept():
    dag = parse(lambda a, b, c: torch.addcdiv(a, b, c, value=0.5), *(torch.randn(3, 3) for _ in range(3)))
    node = dag.nodes[0]
    assert node.op_name == "addcdiv" and node.metadata["kwargs"] == {"value": 0.5}
    dag = parse(lambda x: x * 2.0, torch.randn(3))
    assert dag.nodes[0].metadata["arg_spec"] == [("buf", 0), ("const", 2.0)]


def test_module_calls_become_functional_ops():
    m = nn.Sequential(nn.Linear(8, 16), nn.ReLU(), nn.Linear(16, 4))
    dag = GraphAnalyzer().parse_fx_graph(fx.symbolic_trace(m), [torch.randn(5, 8)])
    assert [n.op_name for n in dag.nodes] == ["linear", "relu", "linear"]
    assert dag.outputs[0].shape == (5, 4)
    w = dag.nodes[0].inputs[1]
    assert w.constant_value is not None and w.shape == (16, 8) and w.scope is BufferScope.GLOBAL


def test_buffer_manager_reuse_and_promotion():
    bm = BufferManager()
    a = bm.allocate_buffer("t", torch.float32, (4, 4))
    b = bm.allocate_buffer("t", torch.float32, (4, 4))
    assert a.name != b.name and bm.get_buffer(a.name) is a
    a.promote_scope(BufferScope.SHARED)
    a.promote_scope(BufferScope.LOCAL)                               # never demotes
    assert a.scope is BufferScope.SHARED
    a.set_lifetime(0, 1)
    b.set_lifetime(2, 3)
    a.scope = b.scope = BufferScope.LOCAL
    assert not a.overlaps_with(b) and b.can_reuse_memory_with(a)
    assert bm.optimize_buffer_reuse([a, b]) == {b.name: a.name}
    assert a.get_memory_footprint() == 64


# ---------------------------------------------------------------- in-place updates
def _plan_of(fn, inputs):
    import conductor  # noqa: F401
    from conductor_b200.compiler.jit_compiler import ChoreoJITCompiler

    box = {}

    def backend(gm, ex):
        box["artifact"] = ChoreoJITCompiler().compile_graph(gm, ex)
        return gm.forward

    torch._dynamo.reset()
    with torch.no_grad():
        torch.compile(fn, backend=backend)(*inputs)
    torch._dynamo.reset()
    return box["artifact"]


def test_later_readers_see_an_in_place_update():
    """`h.relu_()` changes h; the add after it must read the relu's result, not the product."""
    def f(x):
        h = x * 2
        h.relu_()
        return h + 1

    art = _plan_of(f, [torch.randn(4, 8)])
    dag = art.dag
    add = [n for n in dag.nodes if n.op_name == "add"][0]
    relu = [n for n in dag.nodes if n.op_name in ("relu", "relu_")][0]
    assert add.inputs[0] is relu.outputs[0]
    assert dag.output_spec[0] is add.outputs[0]

    def g(x, y):
        h = x + y
        h += y                      # operator.iadd
        return torch.nn.functional.relu(h, inplace=True), h

    dag = _plan_of(g, [torch.randn(4, 8), torch.randn(4, 8)]).dag
    last = [n for n in dag.nodes if n.op_name == "relu"][0]
    # both returned values are the mutated h, i.e. the relu's result
    assert dag.output_spec[0] is last.outputs[0] and dag.output_spec[1] is last.outputs[0]


def test_in_place_update_of_a_graph_input_is_refused():
    from conductor_b200.utils.exceptions import UnsupportedOperationError

    def f(x):
        x.mul_(2)
        return x + 1

    with pytest.raises(Exception) as err:
        _plan_of(f, [torch.randn(4, 8)])
    assert "in-place" in str(err.value) or isinstance(err.value, UnsupportedOperationError)
