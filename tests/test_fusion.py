"""Clustering and template selection on the five benchmark graphs (as Dynamo traces them) and
on edge cases; CPU only -- nothing is launched."""
import ctypes

import pytest
import torch

import conductor  # noqa: F401  registers 'gcu'
from conductor.compiler.jit_compiler import ChoreoJITCompiler
from conductor.optimization.fusion import FusionCluster, FusionHeuristics, FusionType, LocalPriorityFusionEngine
from conductor.optimization.graph_analyzer import GraphAnalyzer
from conductor.utils.exceptions import UnsupportedOperationError
from conductor_b200.codegen.kernel_templates import IN_COL, IN_FULL, IN_ROW, IN_SCALAR, classify_broadcast
from conductor_b200.codegen.operator_registry import EwOp, ReduceOp, Template
from examples import workloads as wl


def compile_with_dynamo(fn, inputs):
    """Trace `fn` with Dynamo and run this package's compile pipeline on the graph it hands a
    backend; returns the CompiledArtifact (nothing executes)."""
    box = {}

    def backend(gm, example_inputs):
        from conductor_b200.utils.config import get_config

        box["artifact"] = ChoreoJITCompiler().compile_graph(gm, example_inputs)
        return gm.forward

    torch._dynamo.reset()
    with torch.no_grad():
        torch.compile(fn, backend=backend)(*inputs)
    torch._dynamo.reset()
    return box["artifact"]


def assert_unsupported(fn, inputs):
    """Dynamo wraps what a backend raises in BackendCompilerFailed; the cause must be ours."""
    with pytest.raises(Exception) as info:
        compile_with_dynamo(fn, inputs)
    exc = info.value
    inner = getattr(exc, "inner_exception", None) or exc.__cause__ or exc
    assert isinstance(inner, UnsupportedOperationError), repr(exc)


def kernels(artifact):
    return [l for l in artifact.launches if l.template]


def test_c1_mul_add_is_one_elementwise_cluster():
    art = compile_with_dynamo(wl.mul_add, wl.inputs_mul_add(8, 16))
    (k,) = kernels(art)
    assert k.template == Template.ELEMENTWISE and k.name == "elementwise[mul,add]"
    c = k.cluster
    assert [b.name for b in c.external_inputs] == ["l_a_", "l_b_", "l_c_"]
    assert len(c.external_outputs) == 1 and len(c.internal_buffers) == 1
    assert c.internal_buffers[0].scope.value == "local"
    p = k.params
    assert (p.n_inputs, p.n_instr, p.n_outputs, p.out_reg[0]) == (3, 2, 1, 4)
    assert (p.instr[0].op, p.instr[1].op) == (EwOp.MUL, EwOp.ADD)
    assert c.validate_fusion_safety()


def test_c2_reduce_mean_is_one_reduction_cluster():
    art = compile_with_dynamo(wl.reduce_mean_fusion, wl.inputs_reduce_mean(8, 64))
    (k,) = kernels(art)
    assert k.template == Template.ROW_REDUCE and k.name == "reduction[mul,add,relu,reduce_mean]"
    p = k.params
    assert p.reduce_op == ReduceOp.MEAN
    assert [p.chain.input_mode[i] for i in range(3)] == [IN_FULL, IN_ROW, IN_ROW]
    assert [p.chain.instr[i].op for i in range(p.chain.n_instr)] == [EwOp.MUL, EwOp.ADD, EwOp.RELU]
    assert all(p.chain.instr[i].round_to == 1 for i in range(3))           # every op rounds to bf16
    assert k.out_dtypes == [torch.float32] and k.out_shapes == [(8,)]
    assert len(k.cluster.internal_buffers) == 3


def test_float_cast_before_mean_is_folded_away():
    fn = lambda x, w, b: torch.relu(x * w + b).float().mean(-1)  # noqa: E731
    (k,) = kernels(compile_with_dynamo(fn, wl.inputs_reduce_mean(8, 64)))
    assert k.template == Template.ROW_REDUCE and k.params.chain.n_instr == 3


def test_c3_softmax_forward_and_backward():
    logits, grad = wl.inputs_softmax(4, 32)
    (k,) = kernels(compile_with_dynamo(wl.softmax_forward, [logits]))
    assert k.template == Template.SOFTMAX_FWD
    y = torch.softmax(logits, -1)
    (k,) = kernels(compile_with_dynamo(wl.softmax_backward, [grad, y]))
    assert k.template == Template.SOFTMAX_BWD and [b.name for b in k.inputs] == ["l_grad_", "l_y_"]
    (k,) = kernels(compile_with_dynamo(wl.softmax_backward_written_out, [grad, y]))
    assert k.template == Template.SOFTMAX_BWD and k.name == "softmax[mul,sum,sub,mul]"
    assert [b.name for b in k.inputs] == ["l_grad_", "l_y_"]


def test_softmax_with_a_dtype_change_is_refused():
    assert_unsupported(lambda x: torch.softmax(x, -1, dtype=torch.float32), [torch.randn(4, 8).bfloat16()])


def test_c4_mlp_two_gemm_epilogue_clusters():
    mlp = wl.make_mlp(32, 64, 32)
    ks = kernels(compile_with_dynamo(mlp, wl.inputs_mlp(16, 32)))
    assert [k.name for k in ks] == ["gemm_epilogue[linear,relu]", "gemm_epilogue[linear]"]
    assert (ks[0].params.activation, ks[0].params.has_bias) == (1, 1)
    assert (ks[1].params.activation, ks[1].params.has_bias) == (0, 1)
    assert ks[0].outputs[0] is ks[1].inputs[0] and ks[0].outputs[0].scope.value == "shared"
    assert ks[0].out_shapes == [(16, 64)] and ks[1].out_shapes == [(16, 32)]


def test_c5_attention_cluster():
    (k,) = kernels(compile_with_dynamo(wl.causal_attention, wl.inputs_attention(1, 2, 16, 32)))
    assert k.template == Template.ATTENTION and k.params.causal == 1
    assert abs(k.params.scale - 32 ** -0.5) < 1e-7


def test_unknown_op_raises_instead_of_falling_back():
    assert_unsupported(lambda x: torch.cumsum(x, 0), [torch.randn(4)])


def test_fusion_disabled_gives_one_kernel_per_node():
    from conductor_b200.utils.config import get_config

    cfg = get_config()
    cfg.compilation.enable_fusion = False
    try:
        ks = kernels(compile_with_dynamo(wl.mul_add, wl.inputs_mul_add(8, 16, seed=3)))
        assert [k.name for k in ks] == ["elementwise[mul]", "elementwise[add]"]
    finally:
        cfg.compilation.enable_fusion = True


def test_diamond_graph_stays_acyclic():
    def model(x, y):
        t = x + y
        s = t.sum(-1, keepdim=True)      # reduction between two elementwise groups
        return (t - s) * x

    art = compile_with_dynamo(model, [torch.randn(4, 8), torch.randn(4, 8)])
    names = [k.name for k in kernels(art)]
    assert len(names) == 3 and names[1].startswith("reduction[")
    produced = set()
    for k in kernels(art):                                   # every input is produced earlier
        for b in k.inputs:
            assert b.is_input or b in produced
        produced.update(k.outputs)


def test_scalars_lower_to_immediates():
    (k,) = kernels(compile_with_dynamo(lambda x: (x * 2.0 + 1.0) / 3.0 - x, [torch.randn(4, 4)]))
    ops = [k.params.instr[i].op for i in range(k.params.n_instr)]
    assert ops[:2] == [EwOp.MUL_IMM, EwOp.ADD_IMM] and EwOp.DIV in ops and ops[-1] == EwOp.SUB


def test_comparison_where_clamp_and_pow_lowering():
    F = torch.nn.functional
    x, y = torch.randn(4, 16), torch.randn(4, 16)

    def ops_of(fn, inputs):
        (k,) = kernels(compile_with_dynamo(fn, inputs))
        return [(k.params.instr[i].op, round(k.params.instr[i].imm, 3)) for i in range(k.params.n_instr)]

    ops = ops_of(lambda a, b: torch.where(a > 0, a, b * 0.5), [x, y])
    assert [o for o, _ in ops] == [EwOp.CONST, EwOp.GT, EwOp.MUL_IMM, EwOp.WHERE]
    ops = ops_of(lambda a: torch.clamp(a, -1.0, 2.0), [x])
    assert ops == [(EwOp.CONST, -1.0), (EwOp.MAX, 0.0), (EwOp.CONST, 2.0), (EwOp.MIN, 0.0)]
    assert ops_of(lambda a: F.relu6(a), [x]) == [(EwOp.CONST, 0.0), (EwOp.MAX, 0.0), (EwOp.CONST, 6.0), (EwOp.MIN, 0.0)]
    assert [o for o, _ in ops_of(lambda a: a ** 2 + a.pow(3), [x])] == [EwOp.MUL, EwOp.MUL, EwOp.MUL, EwOp.ADD]
    got = [o for o, _ in ops_of(lambda a: F.silu(a) + F.gelu(a) + torch.rsqrt(a) + torch.erf(a), [x])]
    assert sorted(got) == sorted([EwOp.SILU, EwOp.GELU, EwOp.RSQRT, EwOp.ERF, EwOp.ADD, EwOp.ADD, EwOp.ADD])
    assert_unsupported(lambda a: F.gelu(a, approximate="tanh"), [x])
    assert_unsupported(lambda a: a ** 2.5, [x])


def test_matmul_lowers_to_the_gemm_template_with_the_weight_in_place():
    x, w = torch.randn(2, 64, 32).bfloat16(), torch.randn(32, 48).bfloat16()
    art = compile_with_dynamo(lambda a, b: torch.relu(a @ b), [x, w])
    ks = kernels(art)
    assert [k.template for k in ks] == [Template.GEMM_EPILOGUE]          # the relu joins as the epilogue
    assert ks[0].params.activation == 1
    assert ks[0].params.weight_layout == 1 and ks[0].params.x_layout == 0 and ks[0].out_shapes == [(2, 64, 48)]
    assert_unsupported(lambda a, b: a @ b, [torch.randn(2, 8, 16), torch.randn(2, 16, 8)])     # batched right operand


def test_layer_norm_lowering():
    F = torch.nn.functional
    art = compile_with_dynamo(lambda x, w, b: F.layer_norm(x, (32,), w, b), [torch.randn(4, 32), torch.randn(32), torch.randn(32)])
    (k,) = kernels(art)                     # whole vectors, one dtype: the fused template
    assert k.template == Template.LAYER_NORM and k.params.has_weight == 1 and k.params.has_bias == 1
    assert abs(k.params.eps - 1e-5) < 1e-12 and len(k.inputs) == 3
    # a ragged row (30 floats) falls back to two reductions and a chain
    art = compile_with_dynamo(lambda x, w, b: F.layer_norm(x, (30,), w, b), [torch.randn(4, 30), torch.randn(30), torch.randn(30)])
    ks = kernels(art)
    assert [k.template for k in ks] == [Template.ROW_REDUCE, Template.ROW_REDUCE, Template.ELEMENTWISE]
    assert ks[0].out_shapes == [(4, 1)] and ks[1].params.reduce_op == ReduceOp.MEAN
    assert list(ks[2].params.input_mode[:5]) == [IN_FULL, IN_COL, IN_COL, IN_ROW, IN_ROW]
    assert_unsupported(lambda x: F.layer_norm(x, (4, 32)), [torch.randn(4, 32)])


def test_linear_chain_is_recognised_for_autograd():
    from conductor_b200.compiler.autograd import differentiable_kind, linear_chain_layers

    mlp, x = wl.make_mlp(32, 64, 16), torch.randn(8, 32).bfloat16()
    art = compile_with_dynamo(mlp, [x])
    assert differentiable_kind(art.launches, art.dag.inputs) == "linear_chain"
    layers = linear_chain_layers(art.launches, art.dag.inputs)
    assert [has_bias for _, has_bias in layers] == [True, True] and layers[0][0].params.activation == 1
    art2 = compile_with_dynamo(lambda a, b, c: a * b + c, [torch.randn(4, 4)] * 3)
    assert differentiable_kind(art2.launches, art2.dag.inputs) == ""


def test_broadcast_classification():
    assert classify_broadcast((4, 8), (4, 8)) == IN_FULL
    assert classify_broadcast((8,), (4, 8)) == IN_ROW
    assert classify_broadcast((1, 8), (4, 8)) == IN_ROW
    assert classify_broadcast((4, 1), (4, 8)) == IN_COL
    assert classify_broadcast((), (4, 8)) == IN_SCALAR
    assert classify_broadcast((2, 3, 1), (2, 3, 5)) == IN_COL
    with pytest.raises(UnsupportedOperationError):
        classify_broadcast((4, 1, 8), (4, 3, 8))


def test_heuristics_and_cluster_api():
    h = FusionHeuristics()
    assert h.can_fuse_elementwise("mul", "add") and h.can_fuse_elementwise("add", "relu")
    assert h.can_fuse_elementwise("relu", "reduce_mean") and h.can_fuse_elementwise("linear", "relu")
    assert not h.can_fuse_elementwise("softmax", "add") and not h.can_fuse_elementwise("nope", "add")
    import torch.fx as fx

    dag = GraphAnalyzer().parse_fx_graph(fx.symbolic_trace(lambda a, b, c: a * b + c), [torch.randn(64, 64)] * 3)
    (c,) = LocalPriorityFusionEngine().identify_fusion_opportunities(dag)
    assert isinstance(c, FusionCluster) and c.cluster_type is FusionType.ELEMENTWISE
    assert c.estimate_performance_gain() > 0 and c.get_fusion_priority() > 300
    assert "elementwise[mul,add]" in c.generate_fused_dsl()
    assert h.check_memory_constraints(c)


def test_params_struct_sizes_match_header():
    from conductor_b200.codegen import kernel_templates as kt

    assert ctypes.sizeof(kt.CdrTensor) == 8 + 4 + 4 + 64 + 64
    assert ctypes.sizeof(kt.CdrEwInstr) == 24
    assert ctypes.sizeof(kt.CdrEwParams) == 16 + 32 + 16 + 24 * 24
    assert ctypes.sizeof(kt.CdrReduceParams) == ctypes.sizeof(kt.CdrEwParams) + 8


def test_basic_slicing_lowers_to_a_strided_copy_with_an_offset():
    """x[:, 4:12:2] is a view of the input with strides (16, 2) starting at element 4: one COPY launch
    carrying those, then the elementwise chain on the contiguous result.  Indexing by a tensor is not
    a view and is refused."""
    art = compile_with_dynamo(lambda x: x[:, 4:12:2] * 2.0, [torch.randn(8, 16)])
    copy = [l for l in art.launches if l.template == Template.COPY]
    assert len(copy) == 1
    assert copy[0].view_strides == (16, 2) and copy[0].view_offset == 4 and tuple(copy[0].out_shapes[0]) == (8, 4)
    art = compile_with_dynamo(lambda x: x.select(0, 3) + 1.0, [torch.randn(8, 16)])
    copy = [l for l in art.launches if l.template == Template.COPY]
    assert copy[0].view_strides == (1,) and copy[0].view_offset == 48
    with pytest.raises(Exception):
        compile_with_dynamo(lambda x, i: x[i] * 2.0, [torch.randn(8, 16), torch.tensor([1, 3])])


def test_chunk_split_unbind_members_become_slices_of_the_source():
    """chunk / split / unbind return a tuple of views; the tuple is no value of the plan -- every
    getitem on it lowers to one strided copy of the tuple op's own input."""
    art = compile_with_dynamo(lambda x: x.chunk(2, -1)[0] * x.chunk(2, -1)[1], [torch.randn(8, 16)])
    views = sorted((l.view_offset, l.view_strides, tuple(l.out_shapes[0])) for l in art.launches if l.template == Template.COPY)
    assert views == [(0, (16, 1), (8, 8)), (8, (16, 1), (8, 8))]
    art = compile_with_dynamo(lambda x: (lambda q, k, v: q * k + v)(*x.unbind(0)), [torch.randn(3, 8, 16)])
    assert sorted(l.view_offset for l in art.launches if l.template == Template.COPY) == [0, 128, 256]
    art = compile_with_dynamo(lambda x: torch.split(x, [4, 12], dim=-1)[1] + 1.0, [torch.randn(8, 16)])
    copy = [l for l in art.launches if l.template == Template.COPY]
    assert len(copy) == 1 and copy[0].view_offset == 4 and tuple(copy[0].out_shapes[0]) == (8, 12)


def test_composite_activations_stay_one_elementwise_launch():
    """leaky_relu, elu, softplus, hardswish, masked_fill, lerp expand into a few opcodes inside the
    chain they belong to -- still one launch; training-mode dropout is refused."""
    F = torch.nn.functional
    x, y = torch.randn(8, 16), torch.randn(8, 16)
    fn = lambda a, b: torch.lerp(F.leaky_relu(a, 0.1), F.elu(b), 0.25).masked_fill(b > 0, 0.0)  # noqa: E731
    art = compile_with_dynamo(fn, [x, y])
    assert [l.template for l in art.launches] == [Template.ELEMENTWISE]
    ops = [ins.op for ins in art.launches[0].params.instr[: art.launches[0].params.n_instr]]
    assert EwOp.WHERE in ops and EwOp.EXP in ops and EwOp.MIN in ops
    with pytest.raises(Exception):
        compile_with_dynamo(lambda a: F.dropout(a, 0.5, training=True) * 2.0, [x])
    # a chain whose expansion would not fit one 24-instruction program is split by the fusion pass
    long = lambda a, b: (F.softplus(F.elu(F.hardswish(F.leaky_relu(a)))) + b).sum(-1)  # noqa: E731
    art = compile_with_dynamo(long, [x, y])
    assert [l.template for l in art.launches] == [Template.ELEMENTWISE, Template.ROW_REDUCE]


def test_reduction_over_inner_dimensions_moves_them_to_the_back():
    """x.sum(0) of [4, 8, 16]: one strided copy to [8, 16, 4] (strides 16, 1, 128), an alias to
    [128, 4], one row reduction.  Trailing dimensions need no copy."""
    art = compile_with_dynamo(lambda x: x.sum(0), [torch.randn(4, 8, 16)])
    assert [l.template for l in art.launches] == [Template.COPY, 0, Template.ROW_REDUCE]
    assert art.launches[0].view_strides == (16, 1, 128) and tuple(art.launches[1].out_shapes[0]) == (128, 4)
    art = compile_with_dynamo(lambda x: x.amax((1, 2)), [torch.randn(4, 8, 16)])
    assert [l.template for l in art.launches] == [0, Template.ROW_REDUCE]
    assert tuple(art.launches[0].out_shapes[0]) == (4, 128)


def test_general_broadcast_is_materialised_by_a_stride_zero_copy():
    """[6, 1, 8] against [6, 4, 8] is neither a row, a column nor a scalar of the [rows, cols] view:
    the operand is expanded by one COPY launch whose view has stride 0 on the broadcast dimension."""
    art = compile_with_dynamo(lambda a, b: a * b, [torch.randn(6, 4, 8), torch.randn(6, 1, 8)])
    assert [l.template for l in art.launches] == [Template.COPY, Template.ELEMENTWISE]
    assert art.launches[0].view_strides == (8, 0, 1) and tuple(art.launches[0].out_shapes[0]) == (6, 4, 8)
    assert list(art.launches[1].params.input_mode[:2]) == [IN_FULL, IN_FULL]
    art = compile_with_dynamo(lambda a: a.expand(3, 4, 8) + 1.0, [torch.randn(4, 8)])
    assert art.launches[0].template == Template.COPY and art.launches[0].view_strides == (0, 8, 1)


def test_row_statistics_lower_to_reduce_and_elementwise_launches():
    """rms_norm: mean of squares then the normalising chain; log_softmax / logsumexp: row maximum,
    shifted exp-sum, finish; var / std: two-pass.  Only the last dimension."""
    F = torch.nn.functional
    x, w = torch.randn(8, 16), torch.randn(16)
    art = compile_with_dynamo(lambda a, g: F.rms_norm(a, (16,), g, 1e-6), [x, w])
    assert [l.template for l in art.launches] == [Template.ROW_REDUCE, Template.ELEMENTWISE]
    assert art.launches[0].params.reduce_op == ReduceOp.MEAN
    art = compile_with_dynamo(lambda a: F.log_softmax(a, -1), [x])
    assert [l.template for l in art.launches] == [Template.ROW_REDUCE, Template.ROW_REDUCE, Template.ELEMENTWISE]
    assert [l.params.reduce_op for l in art.launches[:2]] == [ReduceOp.MAX, ReduceOp.SUM]
    art = compile_with_dynamo(lambda a: a.std(-1), [x])
    ops = [i.op for i in art.launches[2].params.instr[: art.launches[2].params.n_instr]]
    assert ops == [EwOp.MUL_IMM, EwOp.SQRT] and abs(art.launches[2].params.instr[0].imm - 1.0 / 15.0) < 1e-7
    with pytest.raises(Exception):
        compile_with_dynamo(lambda a: F.log_softmax(a, 0), [x])


def test_addmm_lowers_to_the_gemm_template_with_a_bias_row():
    b, x, w = torch.randn(48).bfloat16(), torch.randn(64, 32).bfloat16(), torch.randn(32, 48).bfloat16()
    art = compile_with_dynamo(lambda c, a, m: torch.addmm(c, a, m), [b, x, w])
    (launch,) = art.launches
    assert launch.template == Template.GEMM_EPILOGUE and launch.params.has_bias == 1 and launch.params.weight_layout == 1
    assert [t.name for t in launch.inputs] == ["l_a_", "l_m_", "l_c_"]
    with pytest.raises(Exception):            # a full [M, N] addend is not an epilogue bias
        compile_with_dynamo(lambda c, a, m: torch.addmm(c, a, m), [torch.randn(64, 48).bfloat16(), x, w])


def test_softmax_over_an_inner_dimension_is_bracketed_by_transposing_copies():
    art = compile_with_dynamo(lambda a: torch.softmax(a, 1), [torch.randn(4, 8, 16)])
    assert [l.template for l in art.launches] == [Template.COPY, Template.SOFTMAX_FWD, Template.COPY]
    assert art.launches[0].view_strides == (128, 1, 16) and tuple(art.launches[1].out_shapes[0]) == (4, 16, 8)
    assert art.launches[2].view_strides == (128, 1, 8) and tuple(art.launches[2].out_shapes[0]) == (4, 8, 16)


def test_cat_lowers_to_one_copy_per_part_into_the_result():
    x, y = torch.randn(4, 8, 16), torch.randn(4, 2, 16)
    art = compile_with_dynamo(lambda a, b: torch.cat((a, b), dim=1), [x, y])
    assert [l.template for l in art.launches] == [Template.COPY, Template.COPY]
    assert art.launches[0].outputs[0] is art.launches[1].outputs[0]
    assert [l.out_view for l in art.launches] == [((4, 8, 16), (160, 16, 1), 0), ((4, 2, 16), (160, 16, 1), 128)]
    assert tuple(art.launches[0].out_shapes[0]) == (4, 10, 16)


def test_layout_changes_compose_into_one_copy():
    """chunk -> view -> transpose: each step is a view of the projection's output, so the transposed
    head layout is gathered straight from it by ONE copy; the intermediate copies and aliases have
    no reader left and are dropped.  A value that something else reads is still materialised."""
    B, S, E, H = 2, 8, 32, 4

    def heads(x):
        q, k, v = x.chunk(3, dim=-1)
        return tuple(t.view(B, S, H, E // H).transpose(1, 2) * 2.0 for t in (q, k, v))

    art = compile_with_dynamo(heads, [torch.randn(B, S, 3 * E)])
    copies = [l for l in art.launches if l.template == Template.COPY]
    assert len(copies) == 3 and not [l for l in art.launches if l.template == 0]
    assert all(l.inputs[0].name == "l_x_" for l in copies)
    assert sorted(l.view_offset for l in copies) == [0, E, 2 * E]
    assert all(l.view_strides == (S * 3 * E, E // H, 3 * E, 1) for l in copies)

    art = compile_with_dynamo(lambda x: (x[:, 1:].t() + 1.0, x[:, 1:] * 2.0), [torch.randn(6, 9)])
    copies = [l for l in art.launches if l.template == Template.COPY]
    assert sorted(l.view_strides for l in copies) == [(1, 9), (9, 1)] and all(l.view_offset == 1 for l in copies)


def test_pointwise_losses_lower_to_one_full_reduce_launch():
    F = torch.nn.functional
    x, y = torch.randn(8, 16), torch.randn(8, 16)
    (launch,) = compile_with_dynamo(lambda a, b: F.mse_loss(a, b), [x, y]).launches
    assert launch.template == Template.FULL_REDUCE and launch.params.reduce_op == ReduceOp.MEAN
    assert [launch.params.chain.instr[i].op for i in range(launch.params.chain.n_instr)] == [EwOp.SUB, EwOp.MUL]
    (launch,) = compile_with_dynamo(lambda a, b: F.l1_loss(a, b, reduction="sum"), [x, y]).launches
    assert launch.params.reduce_op == ReduceOp.SUM and launch.params.chain.instr[1].op == EwOp.ABS


def test_normalize_and_norm_lower_to_a_row_statistic_and_a_chain():
    F = torch.nn.functional
    x = torch.randn(8, 16)
    art = compile_with_dynamo(lambda a: F.normalize(a, dim=-1), [x])
    assert [l.template for l in art.launches] == [Template.ROW_REDUCE, Template.ELEMENTWISE]
    ops = [art.launches[1].params.instr[i].op for i in range(art.launches[1].params.n_instr)]
    assert ops == [EwOp.SQRT, EwOp.CONST, EwOp.MAX, EwOp.DIV]
    assert_unsupported(lambda a: F.normalize(a, dim=0), [x])
    assert_unsupported(lambda a: a.norm(p=1, dim=-1), [x])
