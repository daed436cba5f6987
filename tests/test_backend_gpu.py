"""End-to-end through the plugin surface: `torch.compile(fn, backend='gcu')` on CUDA tensors and
on CPU tensors (the reference's calling convention), compared with the reference's executed path
(eager on CPU) on identical seeded inputs."""
import pytest
import torch

import conductor  # noqa: F401
from conftest import assert_close
from examples import workloads as wl
from oracle import reference_path as rp

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def compiled(fn):
    torch._dynamo.reset()
    return torch.compile(fn, backend="gcu")


def run_both(fn, inputs):
    """(result with CUDA inputs, result with CPU inputs, reference result)."""
    want = rp.run_reference(fn, inputs)
    f = compiled(fn)
    with torch.no_grad():
        on_gpu = f(*[t.to(DEV) for t in inputs])
        assert on_gpu.device.type == "cuda"
        on_cpu = f(*inputs)
        assert on_cpu.device.type == "cpu"
    return on_gpu, on_cpu, want


def test_mul_add_bit_exact_both_conventions():
    on_gpu, on_cpu, want = run_both(wl.mul_add, wl.inputs_mul_add(300, 257, seed=41))
    assert torch.equal(on_gpu.cpu(), want) and torch.equal(on_cpu, want)


def test_reduce_mean_fusion():
    on_gpu, on_cpu, want = run_both(wl.reduce_mean_fusion, wl.inputs_reduce_mean(100, 4096, seed=42))
    assert_close(on_gpu, want, 1e-5, "reduce_mean gpu")
    assert_close(on_cpu, want, 1e-5, "reduce_mean host")


def test_softmax_forward_and_both_backward_forms():
    logits, grad = wl.inputs_softmax(64, 8192, seed=43)
    y_gpu, y_cpu, y_want = run_both(wl.softmax_forward, [logits])
    assert_close(y_gpu, y_want, 1e-5, "softmax fwd")
    assert_close(y_cpu, y_want, 1e-5, "softmax fwd host")
    for fn in (wl.softmax_backward, wl.softmax_backward_written_out):
        dx_gpu, _, dx_want = run_both(fn, [grad, y_want])
        assert_close(dx_gpu, dx_want, 1e-5, fn.__name__)


def test_unfused_graph_matches_fused():
    from conductor_b200.utils.config import get_config

    a, b, c = wl.inputs_mul_add(64, 128, seed=44)
    cfg = get_config()
    cfg.compilation.enable_fusion = False
    try:
        out = compiled(wl.mul_add)(a.to(DEV), b.to(DEV), c.to(DEV))
    finally:
        cfg.compilation.enable_fusion = True
    assert torch.equal(out.cpu(), a * b + c)


def test_multi_cluster_graph_with_shared_temporary():
    def model(x, y):
        t = x + y
        s = t.sum(-1, keepdim=True)
        return (t - s) * x, torch.relu(t)

    gen = torch.Generator().manual_seed(47)
    x, y = torch.randn(33, 200, generator=gen), torch.randn(33, 200, generator=gen)
    want = rp.run_reference(model, [x, y])
    got = compiled(model)(x.to(DEV), y.to(DEV))
    assert isinstance(got, tuple) and len(got) == 2
    # the fp32 row sum (|s| ~ 20, summation-order error ~ 2e-6) is subtracted and rescaled, so the
    # 1e-5 bound of a single fp32 reduction becomes 5e-5 for this composite
    assert_close(got[0], want[0], 5e-5, "diamond")
    assert torch.equal(got[1].cpu(), want[1])


def test_graph_capture_replays_the_plan():
    from conductor_b200.compiler.gcu_backend import get_gcu_backend

    x, w, b = (t.to(DEV) for t in wl.inputs_reduce_mean(256, 4096, seed=45))
    f = compiled(wl.reduce_mean_fusion)
    want = f(x, w, b).clone()
    plan = list(get_gcu_backend()._compiled_functions.values())[-1]
    g = plan.capture(x, w, b)
    (out,) = g.replay()
    torch.cuda.synchronize()
    assert torch.equal(out, want)
    x.mul_(2)                                   # same buffer, new contents: replay sees them
    (out2,) = g.replay()
    torch.cuda.synchronize()
    assert torch.equal(out2, f(x, w, b))
    seq = plan.capture_sequence([(x, w, b), (x, w, b)])
    seq.replay()
    torch.cuda.synchronize()
    assert torch.equal(seq.all_outputs[1][0], seq.all_outputs[0][0]) and seq.n_kernels == 2


@pytest.mark.parametrize("lanes", [2, 3])
def test_captured_sequence_with_runs_in_flight_matches_single_calls(lanes):
    """Runs recorded on several branches of one graph overlap in time; each must still produce what a
    call by itself produces (the attention launches of different branches need their own tile counters)."""
    from conductor_b200.compiler.gcu_backend import get_gcu_backend

    get_gcu_backend().clear_cache()            # the plans looked up below are the ones compiled here
    sets = [tuple(t.to(DEV) for t in wl.inputs_attention(2, 4, 512, 128, seed=300 + i)) for i in range(5)]
    f = compiled(wl.causal_attention)
    with torch.no_grad():
        want = [f(*s).clone() for s in sets]
    plan = list(get_gcu_backend()._compiled_functions.values())[-1]
    seq = plan.capture_sequence(sets, lanes=lanes)
    assert seq.lanes == lanes and seq.runs == 5
    for _ in range(3):
        seq.replay()
    torch.cuda.synchronize()
    for got, w in zip(seq.all_outputs, want):
        assert torch.equal(got[0], w)
    first = plan.capture_sequence(sets, keep_outputs="first", lanes=lanes)
    (out,) = first.replay()
    torch.cuda.synchronize()
    assert torch.equal(out, want[0])
    # a reduction with its inputs replaced between replays
    xs = [tuple(t.to(DEV) for t in wl.inputs_reduce_mean(512, 4096, seed=310 + i)) for i in range(4)]
    g = compiled(wl.reduce_mean_fusion)
    with torch.no_grad():
        g(*xs[0])
    plan = list(get_gcu_backend()._compiled_functions.values())[-1]
    seq = plan.capture_sequence(xs, lanes=lanes)
    seq.replay()
    xs[1][0].mul_(3)
    seq.replay()
    torch.cuda.synchronize()
    with torch.no_grad():
        for got, x in zip(seq.all_outputs, xs):
            assert torch.equal(got[0], g(*x))


def test_wrong_shape_at_call_time_raises():
    from conductor.utils.exceptions import ExecutionError
    from conductor_b200.compiler.gcu_backend import get_gcu_backend

    a, b, c = (t.to(DEV) for t in wl.inputs_mul_add(8, 8, seed=46))
    compiled(wl.mul_add)(a, b, c)
    plan = list(get_gcu_backend()._compiled_functions.values())[-1]
    with pytest.raises(ExecutionError):
        plan(a[:4], b[:4], c[:4])


def test_device_status_word_is_clean():
    import ctypes

    from conductor_b200.compiler.loader import load_library

    st = ctypes.c_int(-1)
    with torch.cuda.device(0):
        assert load_library().cdr_device_status(ctypes.byref(st), 1) == 0
    assert st.value == 0


def test_softmax_is_differentiable_through_the_backend():
    """loss.backward() through a gcu-compiled softmax runs the softmax-backward template."""
    logits, grad = wl.inputs_softmax(48, 1024, seed=48)
    x_ref = logits.clone().requires_grad_(True)
    y_ref = torch.softmax(x_ref, -1)
    y_ref.backward(grad)
    x = logits.to(DEV).requires_grad_(True)
    y = compiled(wl.softmax_forward)(x)
    assert y.requires_grad
    y.backward(grad.to(DEV))
    assert_close(y, y_ref, 1e-5, "softmax fwd under autograd")
    assert_close(x.grad, x_ref.grad, 1e-5, "softmax grad")


def test_wider_elementwise_and_reduction_coverage():
    gen = torch.Generator().manual_seed(49)
    x = torch.randn(64, 96, generator=gen)
    y = torch.rand(64, 96, generator=gen) + 0.5
    cases = {
        "sub_div": lambda a, b: (a - b) / b,
        "unary_math": lambda a, b: torch.tanh(a) + torch.sigmoid(a) * torch.exp(-b) - torch.sqrt(b) + torch.log(b),
        "abs_neg_trig": lambda a, b: torch.abs(a) - torch.neg(b) + torch.sin(a) * torch.cos(b),
        "max_min": lambda a, b: torch.maximum(a, b) - torch.minimum(a, b),
        "addcmul": lambda a, b: torch.addcmul(a, a, b, value=0.25),
        "row_sum": lambda a, b: (a * b).sum(-1),
        "row_amax": lambda a, b: torch.amax(a + b, dim=-1),
        "reduce_then_scale": lambda a, b: a / a.abs().sum(-1, keepdim=True),
        "full_mean": lambda a, b: (a * b).mean(),
    }
    for name, fn in cases.items():
        want = rp.run_reference(fn, [x, y])
        got = compiled(fn)(x.to(DEV), y.to(DEV))
        assert_close(got, want, 2e-5 if name in ("reduce_then_scale",) else 1e-5, name)


def test_comparison_select_and_activation_coverage():
    """Comparisons and `where` inside a fused chain (1.0 / 0.0 registers), clamp family, constant
    powers, rsqrt, silu, erf-gelu: selects and clamps exactly, transcendental ones within 1e-5."""
    F = torch.nn.functional
    gen = torch.Generator().manual_seed(50)
    x = torch.randn(72, 160, generator=gen)
    y = torch.randn(72, 160, generator=gen)
    x[0, 0], x[1, 1], y[2, 2] = float("nan"), 0.0, float("nan")
    exact = {
        "where_gt": lambda a, b: torch.where(a > 0, a, b * 0.5),
        "relu_backward_mask": lambda a, b: b * (a > 0),
        "compare_chain": lambda a, b: torch.where(a >= b, a - b, b - a) + (a == b) + (a != b) * 2.0 + (a < b) + (a <= b),
        "clamp_family": lambda a, b: torch.clamp(a, -1.0, 2.0) + b.clamp(min=0.5) + torch.clamp(a, max=0.25)
        + F.relu6(b) + F.hardtanh(a),
        "const_powers": lambda a, b: a ** 2 + b.pow(3) + torch.square(a),
    }
    close = {
        "rsqrt_recip": lambda a, b: torch.rsqrt(a * a + 1.0) + (b * b + 1.0).reciprocal() + (a * a + 0.5) ** 0.5,
        "silu_gelu_erf": lambda a, b: F.silu(a) + F.gelu(b) + torch.erf(a * b),
        "rms_norm": lambda a, b: a * torch.rsqrt((a * a).mean(-1, keepdim=True) + 1e-6) * b,
    }
    for name, fn in {**exact, **close}.items():
        want = rp.run_reference(fn, [x, y])
        got = compiled(fn)(x.to(DEV), y.to(DEV)).cpu()
        if name in exact:
            same = (got == want) | (torch.isnan(got) & torch.isnan(want))
            assert bool(same.all()), f"{name}: {int((~same).sum())} elements differ"
        else:
            assert_close(got, want, 1e-5, name)
    # bf16: the select runs in the chain's registers, results round per op like eager
    xb, yb = x.bfloat16(), y.bfloat16()
    fn = exact["where_gt"]
    got = compiled(fn)(xb.to(DEV), yb.to(DEV)).cpu()
    want = rp.run_reference(fn, [xb, yb])
    same = (got == want) | (torch.isnan(got) & torch.isnan(want))
    assert got.dtype == torch.bfloat16 and bool(same.all())
    with pytest.raises(Exception):
        compiled(lambda a: F.gelu(a, approximate="tanh"))(x.to(DEV))


def test_layer_norm_fused_and_decomposed():
    """layer_norm over the last dimension: the fused one-pass template (affine, plain, bf16, long rows)
    and the three-launch decomposition (ragged rows)."""
    F = torch.nn.functional
    gen = torch.Generator().manual_seed(54)
    x = torch.randn(6, 50, 256, generator=gen) * 3 + 1
    w, b = torch.randn(256, generator=gen), torch.randn(256, generator=gen)
    cases = {
        "affine": (lambda x_, w_, b_: F.layer_norm(x_, (256,), w_, b_, 1e-5), [x, w, b], 1e-5),
        "plain": (lambda x_: F.layer_norm(x_, (256,)), [x], 1e-5),
        "bf16": (lambda x_, w_, b_: F.layer_norm(x_, (256,), w_, b_), [x.bfloat16(), w.bfloat16(), b.bfloat16()], 2e-2),
        "ragged": (lambda x_: F.layer_norm(x_, (250,), eps=1e-3) + 1.0, [x[..., :250].contiguous()], 1e-5),
        "long_rows": (lambda x_, w_: F.layer_norm(x_, (8192,), w_), [torch.randn(5, 8192, generator=gen) - 2, torch.randn(8192, generator=gen)], 1e-5),
        "short_rows": (lambda x_, w_, b_: F.layer_norm(x_, (16,), w_, b_), [x[..., :16].contiguous(), w[:16].contiguous(), b[:16].contiguous()], 1e-5),
    }
    for name, (fn, inputs, tol) in cases.items():
        want = rp.run_reference(fn, inputs)
        got = compiled(fn)(*[t.to(DEV) for t in inputs])
        assert got.dtype == want.dtype
        assert_close(got.float(), want.float(), tol * 4 if tol < 1e-4 else tol, name)
    with pytest.raises(Exception):
        compiled(lambda x_: F.layer_norm(x_, (50, 256)))(x.to(DEV))


def test_layout_changes_and_multi_head_attention():
    """transpose / permute / t move data with the strided-copy template; with them a multi-head
    self-attention block (view -> transpose -> attention -> transpose -> reshape) compiles."""
    F = torch.nn.functional
    gen = torch.Generator().manual_seed(55)
    a = torch.randn(12, 40, generator=gen)
    t4 = torch.randn(2, 3, 8, 16, generator=gen)
    exact = {"t_add": (lambda x: x.t() + 1.0, [a]), "permute": (lambda x: x.permute(0, 2, 1, 3).contiguous() * 2.0, [t4]),
             "transpose_sum": (lambda x: x.transpose(-1, -2).sum(-1), [t4])}
    for name, (fn, inputs) in exact.items():
        want = rp.run_reference(fn, inputs)
        got = compiled(fn)(*[t.to(DEV) for t in inputs]).cpu()
        assert got.shape == want.shape, name
        assert_close(got, want, 1e-5, name)

    def mha(x):
        B, S, E = x.shape
        H, D = 4, E // 4
        q = x.view(B, S, H, D).transpose(1, 2)
        o = F.scaled_dot_product_attention(q, q * 0.5, q + 1.0, is_causal=True)
        return o.transpose(1, 2).reshape(B, S, E)

    x = torch.randn(2, 256, 256, generator=gen).bfloat16()
    want = rp.run_reference(mha, [x])
    got = compiled(mha)(x.to(DEV))
    assert got.shape == want.shape
    assert_close(got.float(), want.float(), 2e-2, "multi-head attention block")


def test_composite_activations_and_selections():
    """leaky_relu / elu / softplus / hardswish / hardsigmoid / masked_fill / lerp / inference-mode
    dropout are written out over the elementwise opcodes: selections exact, the rest within 1e-5
    in fp32 and 2e-2 in bf16 (intermediates stay fp32, one rounding at the end)."""
    F = torch.nn.functional
    gen = torch.Generator().manual_seed(59)
    x = 4.0 * torch.randn(72, 160, generator=gen)
    y = torch.randn(72, 160, generator=gen)
    mask = torch.rand(72, 160, generator=gen) > 0.5
    x[0, :4] = torch.tensor([0.0, 25.0, -30.0, 3.0])
    exact = {"masked_fill": (lambda a, m: a.masked_fill(m, -1e9) * 1.0, [x, mask]),
             "dropout_eval": (lambda a: F.dropout(a, 0.3, training=False) + 1.0, [x])}
    close = {"leaky_relu": (lambda a: F.leaky_relu(a, 0.1), [x]), "elu": (lambda a: F.elu(a, 1.5), [x]),
             "softplus": (lambda a: F.softplus(a, beta=2.0, threshold=10.0), [x]), "hardswish": (lambda a: F.hardswish(a), [x]),
             "hardsigmoid": (lambda a: F.hardsigmoid(a), [x]), "lerp": (lambda a, b: torch.lerp(a, b, 0.3), [x, y]),
             "lerp_tensor": (lambda a, b: torch.lerp(a, b, torch.sigmoid(b)), [x, y]),
             "masked_softmax": (lambda a, m: torch.softmax(a.masked_fill(m, float("-inf")), -1), [x, mask & (torch.arange(160) > 0)])}
    for name, (fn, inputs) in {**exact, **close}.items():
        want = rp.run_reference(fn, inputs)
        got = compiled(fn)(*[t.to(DEV) for t in inputs]).cpu()
        if name in exact:
            assert torch.equal(got, want), name
        else:
            assert_close(got, want, 1e-5, name)
    for name in ("leaky_relu", "elu", "softplus", "hardswish"):
        fn, inputs = close[name]
        xb = inputs[0].bfloat16()
        want = rp.run_reference(fn, [xb])
        got = compiled(fn)(xb.to(DEV)).cpu()
        assert got.dtype == torch.bfloat16
        assert_close(got.float(), want.float(), 2e-2, name + " bf16")


def test_reductions_over_inner_dimensions():
    """sum / mean / amax / amin over dimensions other than the last: reduced dimensions are moved to
    the back by the strided copy, then one row reduction; amax / amin exact, sums within 1e-5.
    Their results broadcast back along a middle or leading dimension, which the elementwise kernels
    do not index directly: the operand is expanded by a stride-0 copy first (as is `expand`)."""
    gen = torch.Generator().manual_seed(60)
    x = torch.randn(6, 40, 72, generator=gen)
    cases = {"sum0": lambda a: a.sum(0), "mean1_keepdim": lambda a: a.mean(1, keepdim=True), "amax01": lambda a: a.amax((0, 1)),
             "amin_neg2": lambda a: a.amin(-2), "sum12": lambda a: a.sum((1, 2)), "chain_sum02": lambda a: (a * 2.0 + 1.0).sum((0, 2)),
             "column_norm": lambda a: a / a.abs().sum(1, keepdim=True), "centre_over_batch": lambda a: a - a.mean(0),
             "expand_first_column": lambda a: a[:, :1].expand(6, 40, 72) + a,
             "broadcast_to": lambda a: torch.broadcast_to(a[:, :, :1], (6, 40, 72)) - a}
    for name, fn in cases.items():
        want = rp.run_reference(fn, [x])
        got = compiled(fn)(x.to(DEV)).cpu()
        assert got.shape == want.shape, name
        if name.startswith("am"):
            assert torch.equal(got, want), name
        else:
            assert_close(got, want, 1e-5, name)
    xb = x.bfloat16()
    want = rp.run_reference(cases["sum0"], [xb])
    got = compiled(cases["sum0"])(xb.to(DEV)).cpu()
    assert got.dtype == want.dtype
    assert_close(got.float(), want.float(), 2e-2, "sum0 bf16")


def test_row_statistics_lowered_to_several_launches():
    """rms_norm, log_softmax, logsumexp, var, std over the last dimension: row reductions with fp32
    statistics and a finishing elementwise launch; 1e-5 in fp32, 2e-2 in bf16."""
    F = torch.nn.functional
    gen = torch.Generator().manual_seed(61)
    x = 3.0 * torch.randn(96, 200, generator=gen) + 1.0
    x[0] += 80.0                                   # a row where the unshifted exp would overflow
    w = torch.rand(200, generator=gen) + 0.5
    cases = {"rms_norm_w": (lambda a, g: F.rms_norm(a, (200,), g, 1e-6), [x, w]), "rms_norm": (lambda a: F.rms_norm(a, (200,)), [x]),
             "log_softmax": (lambda a: F.log_softmax(a, -1), [x]), "logsumexp": (lambda a: torch.logsumexp(a, -1), [x]),
             "logsumexp_keepdim": (lambda a: a.logsumexp(1, keepdim=True), [x]), "var": (lambda a: a.var(-1), [x]),
             "std_keepdim": (lambda a: a.std(-1, keepdim=True), [x]), "var_biased": (lambda a: torch.var(a, dim=-1, correction=0), [x]),
             "nll_of_log_softmax": (lambda a: -(F.log_softmax(a * 0.5, -1) * torch.softmax(a, -1)).sum(-1), [x])}
    for name, (fn, inputs) in cases.items():
        want = rp.run_reference(fn, inputs)
        got = compiled(fn)(*[t.to(DEV) for t in inputs]).cpu()
        assert got.shape == want.shape and got.dtype == want.dtype, name
        assert_close(got, want, 1e-5, name)
    for name in ("rms_norm_w", "log_softmax", "var"):
        fn, inputs = cases[name]
        inputs = [t.bfloat16() for t in inputs]
        want = rp.run_reference(fn, inputs)
        got = compiled(fn)(*[t.to(DEV) for t in inputs]).cpu()
        assert got.dtype == torch.bfloat16
        assert_close(got.float(), want.float(), 2e-2, name + " bf16")


def test_pointwise_losses():
    """mse_loss / l1_loss: difference chain in fp32 + mean or sum over everything in one launch."""
    F = torch.nn.functional
    gen = torch.Generator().manual_seed(65)
    x, y = torch.randn(300, 257, generator=gen), torch.randn(300, 257, generator=gen)
    cases = {"mse": lambda a, b: F.mse_loss(a, b), "mse_sum": lambda a, b: F.mse_loss(a, b, reduction="sum"),
             "l1": lambda a, b: F.l1_loss(a * 2.0, b), "l1_none": lambda a, b: F.l1_loss(a, b, reduction="none") * 2.0}
    for name, fn in cases.items():
        want = rp.run_reference(fn, [x, y])
        got = compiled(fn)(x.to(DEV), y.to(DEV)).cpu()
        assert got.shape == want.shape and got.dtype == want.dtype, name
        assert_close(got, want, 1e-5, name)
    xb, yb = x.bfloat16(), y.bfloat16()
    want = rp.run_reference(cases["mse"], [xb, yb])
    got = compiled(cases["mse"])(xb.to(DEV), yb.to(DEV)).cpu()
    assert got.dtype == torch.bfloat16
    assert_close(got.float(), want.float(), 2e-2, "mse bf16")


def test_vector_norm_normalize_and_one_sided_clamps():
    """x.norm(dim=-1), linalg.vector_norm, F.normalize (row 2-norm in fp32, then sqrt / divide),
    clamp_min / clamp_max and expand_as."""
    F = torch.nn.functional
    gen = torch.Generator().manual_seed(66)
    x = torch.randn(96, 200, generator=gen)
    x[3] = 0.0                                     # a zero row: normalize divides by eps, not by 0
    close = {"norm": lambda a: a.norm(dim=-1), "vector_norm": lambda a: torch.linalg.vector_norm(a, dim=-1, keepdim=True),
             "normalize": lambda a: F.normalize(a, dim=-1), "normalize_default_dim": lambda a: F.normalize(a) * 2.0}
    exact = {"one_sided": lambda a: a.clamp_min(0.5) + a.clamp_max(-0.5), "expand_as": lambda a: a[:, :1].expand_as(a) + a}
    for name, fn in {**close, **exact}.items():
        want = rp.run_reference(fn, [x])
        got = compiled(fn)(x.to(DEV)).cpu()
        assert got.shape == want.shape, name
        if name in exact:
            assert torch.equal(got, want), name
        else:
            assert_close(got, want, 1e-5, name)
    xb = x.bfloat16()
    want = rp.run_reference(close["normalize"], [xb])
    assert_close(compiled(close["normalize"])(xb.to(DEV)).cpu().float(), want.float(), 2e-2, "normalize bf16")


def test_softmax_over_an_inner_dimension():
    """softmax over a dimension other than the last: transposing copy, row kernel, transposing copy."""
    gen = torch.Generator().manual_seed(62)
    x = 2.0 * torch.randn(5, 48, 72, generator=gen)
    for name, fn in {"dim1": lambda a: torch.softmax(a, 1), "dim0_scaled": lambda a: torch.softmax(a, 0) * 2.0,
                     "neg2": lambda a: a.softmax(-2)}.items():
        want = rp.run_reference(fn, [x])
        got = compiled(fn)(x.to(DEV)).cpu()
        assert got.shape == want.shape, name
        assert_close(got, want, 1e-5, name)


def test_concatenation_writes_parts_into_slices_of_the_result():
    """torch.cat: one strided copy per part into its slice of the result; exact.  The rotate-half
    form used by rotary embeddings (cat of a negated half and the other half) compiles with it."""
    gen = torch.Generator().manual_seed(63)
    a = torch.randn(4, 24, 64, generator=gen)
    b = torch.randn(4, 24, 64, generator=gen)
    cos = torch.cos(torch.randn(24, 64, generator=gen))
    cases = {"last": lambda p, q: torch.cat([p, q], -1) * 2.0, "middle_ragged": lambda p, q: torch.cat((p, q[:, :5], p[:, 3:4]), dim=1),
             "first": lambda p, q: torch.cat([p, q, p], 0), "odd_columns": lambda p, q: torch.cat([p[..., :3], q[..., 3:]], -1) + 1.0}
    for name, fn in cases.items():
        want = rp.run_reference(fn, [a, b])
        got = compiled(fn)(a.to(DEV), b.to(DEV)).cpu()
        assert got.shape == want.shape and torch.equal(got, want), name
    rope = lambda p, c: p * c + torch.cat([-p[..., 32:], p[..., :32]], -1) * (1.0 - c)  # noqa: E731
    assert_close(compiled(rope)(a.to(DEV), cos.to(DEV)).cpu(), rp.run_reference(rope, [a, cos]), 1e-5, "rotate half")
    ab = a.bfloat16()
    fn = cases["last"]
    assert torch.equal(compiled(fn)(ab.to(DEV), ab.to(DEV)).cpu(), rp.run_reference(fn, [ab, ab]))


def test_basic_slicing_goes_through_the_strided_copy():
    """x[a:b], x[..., ::2], narrow, select: a view with an offset and strides, gathered by the
    strided-copy template; results are bit-identical to eager (no arithmetic on the copied part)."""
    gen = torch.Generator().manual_seed(57)
    a = torch.randn(64, 96, generator=gen)
    t3 = torch.randn(4, 33, 50, generator=gen).bfloat16()
    ids = torch.randint(-50, 50, (16, 40), generator=gen)
    cases = {"columns": (lambda x: x[:, :32] * 2.0, [a]), "rows": (lambda x: x[5:37] + 1.0, [a]),
             "odd_offset": (lambda x: x[:, 3:51] * 1.0, [a]), "even_odd": (lambda x: x[..., 1::2] - x[..., 0::2], [a]),
             "narrow": (lambda x: x.narrow(1, 7, 20) + 0.5, [a]), "select_row": (lambda x: x[3] * 3.0, [a]),
             "select_mid": (lambda x: x.select(1, 5) + x.select(1, 6), [t3]),
             "qkv_split": (lambda x: x[..., :16] + x[..., 16:32] * x[..., 32:48], [t3]),
             "int_slice": (lambda x: x[2:10, ::4] + 1, [ids])}
    for name, (fn, inputs) in cases.items():
        want = rp.run_reference(fn, inputs)
        got = compiled(fn)(*[t.to(DEV) for t in inputs]).cpu()
        assert got.shape == want.shape and got.dtype == want.dtype, name
        assert torch.equal(got, want), name


def test_fused_qkv_projection_split_into_heads():
    """One [E, 3E] projection, chunk(3) into q / k / v, heads via view + transpose, causal attention:
    the members of the chunk are gathered straight from the projection's output."""
    F = torch.nn.functional
    gen = torch.Generator().manual_seed(58)
    B, S, E, H = 2, 128, 256, 4
    x = (0.5 * torch.randn(B, S, E, generator=gen)).bfloat16()
    w = (torch.randn(3 * E, E, generator=gen) / 16).bfloat16()
    b = (0.1 * torch.randn(3 * E, generator=gen)).bfloat16()

    def attn(x_, w_, b_):
        q, k, v = F.linear(x_, w_, b_).chunk(3, dim=-1)
        q, k, v = (t.view(B, S, H, E // H).transpose(1, 2) for t in (q, k, v))
        return F.scaled_dot_product_attention(q, k, v, is_causal=True).transpose(1, 2).reshape(B, S, E)

    want = rp.run_reference(attn, [x, w, b])
    got = compiled(attn)(x.to(DEV), w.to(DEV), b.to(DEV))
    assert got.shape == want.shape
    assert_close(got.float(), want.float(), 2e-2, "fused qkv attention")
    for name, fn in {"split": lambda t: (lambda a, c: a - c)(*t.split(E // 2, dim=-1)),
                     "unbind": lambda t: t.unbind(0)[1] * 2.0}.items():
        want = rp.run_reference(fn, [x])
        assert torch.equal(compiled(fn)(x.to(DEV)).cpu(), want), name


def test_transformer_block_compiles_and_matches_eager():
    """A pre-norm transformer block written with functional ops: layer norm, three projections,
    multi-head causal attention, output projection, residuals, GELU MLP -- every piece runs on a
    kernel template; the whole block is compared with eager bf16 on the CPU."""
    F = torch.nn.functional
    torch.manual_seed(56)
    B, S, E, H = 2, 128, 256, 4
    D = E // H

    def p(*shape, scale=0.05):
        return (torch.randn(*shape) * scale).bfloat16()

    params = [p(E) + 1, p(E), p(E, E), p(E), p(E, E), p(E), p(E, E), p(E), p(E, E), p(E), p(E) + 1, p(E), p(4 * E, E), p(4 * E),
              p(E, 4 * E), p(E)]

    def block(x, g1, b1, wq, bq, wk, bk, wv, bv, wo, bo, g2, b2, w1, c1, w2, c2):
        h = F.layer_norm(x, (E,), g1, b1)
        q = F.linear(h, wq, bq).view(B, S, H, D).transpose(1, 2)
        k = F.linear(h, wk, bk).view(B, S, H, D).transpose(1, 2)
        v = F.linear(h, wv, bv).view(B, S, H, D).transpose(1, 2)
        a = F.scaled_dot_product_attention(q, k, v, is_causal=True).transpose(1, 2).reshape(B, S, E)
        x = x + F.linear(a, wo, bo)
        h = F.layer_norm(x, (E,), g2, b2)
        return x + F.linear(F.gelu(F.linear(h, w1, c1)), w2, c2)

    x = torch.randn(B, S, E).bfloat16()
    want = rp.run_reference(block, [x] + params)
    f = compiled(block)
    got = f(*[t.to(DEV) for t in [x] + params])
    assert got.shape == want.shape and got.dtype == torch.bfloat16
    assert_close(got.float(), want.float(), 3e-2, "transformer block")


def test_llama_style_block_compiles_and_matches_eager():
    """RMS norm, fused QKV projection split by chunk, rotary embedding in the rotate-half form
    (slices, negation, cat, broadcast cos / sin), causal attention, SwiGLU MLP, residuals: every
    piece on a kernel template, compared with eager bf16 on the CPU."""
    F = torch.nn.functional
    B, S, E, H = 2, 128, 256, 4
    D = E // H
    gen = torch.Generator().manual_seed(64)

    def r(*shape, scale=1.0):
        return (scale * torch.randn(*shape, generator=gen)).bfloat16()

    def rotate_half(t):
        return torch.cat([-t[..., D // 2:], t[..., :D // 2]], -1)

    def block(x, g1, wqkv, wo, g2, wgate, wup, wdown, cos, sin):
        h = F.rms_norm(x, (E,), g1, 1e-6)
        q, k, v = F.linear(h, wqkv).chunk(3, dim=-1)
        q, k, v = (t.view(B, S, H, D).transpose(1, 2) for t in (q, k, v))
        q = q * cos + rotate_half(q) * sin
        k = k * cos + rotate_half(k) * sin
        a = F.scaled_dot_product_attention(q, k, v, is_causal=True).transpose(1, 2).reshape(B, S, E)
        x = x + F.linear(a, wo)
        h = F.rms_norm(x, (E,), g2, 1e-6)
        return x + F.linear(F.silu(F.linear(h, wgate)) * F.linear(h, wup), wdown)

    pos = torch.arange(S).float()[:, None] * (10000.0 ** (-torch.arange(0, D, 2).float() / D))[None, :]
    ang = torch.cat([pos, pos], -1)
    inputs = [r(B, S, E, scale=0.5), (torch.rand(E, generator=gen) + 0.5).bfloat16(), r(3 * E, E, scale=1 / 16),
              r(E, E, scale=1 / 16), (torch.rand(E, generator=gen) + 0.5).bfloat16(), r(2 * E, E, scale=1 / 16),
              r(2 * E, E, scale=1 / 16), r(E, 2 * E, scale=1 / 22), ang.cos().bfloat16(), ang.sin().bfloat16()]
    want = rp.run_reference(block, inputs)
    got = compiled(block)(*[t.to(DEV) for t in inputs])
    assert got.shape == want.shape and got.dtype == torch.bfloat16
    assert_close(got.float(), want.float(), 3e-2, "llama-style block")


def test_mixed_dtype_clusters():
    """A bool mask input, a comparison that leaves the graph as bool, an integer tensor scaling a
    float one: exact against eager."""
    gen = torch.Generator().manual_seed(53)
    a, b = torch.randn(33, 70, generator=gen), torch.randn(33, 70, generator=gen)
    m = torch.rand(33, 70, generator=gen) > 0.5
    i = torch.randint(-5, 6, (33, 70), generator=gen)
    cases = {
        "where_mask": (lambda m_, a_, b_: torch.where(m_, a_, b_ * 2.0), [m, a, b]),
        "compare_out": (lambda a_, b_: a_ > b_, [a, b]),
        "int_times_float": (lambda i_, a_: i_ * a_ + 1.0, [i, a]),
        "int_compare": (lambda i_: torch.where(i_ > 0, i_, -i_), [i]),
    }
    for name, (fn, inputs) in cases.items():
        want = rp.run_reference(fn, inputs)
        got = compiled(fn)(*[t.to(DEV) for t in inputs]).cpu()
        assert got.dtype == want.dtype and got.shape == want.shape, name
        assert torch.equal(got, want), name


def test_mlp_is_differentiable_through_the_backend():
    """loss.backward() through a gcu-compiled Linear -> ReLU -> Linear: every gradient is a launch of
    the GEMM template with transposed-operand layouts (plus one elementwise launch for the ReLU mask)."""
    torch.manual_seed(52)
    ref = torch.nn.Sequential(torch.nn.Linear(256, 512), torch.nn.ReLU(), torch.nn.Linear(512, 128)).bfloat16()
    import copy

    dev = copy.deepcopy(ref).to(DEV)
    x = torch.randn(4, 96, 256).bfloat16()
    xr = x.clone().requires_grad_(True)
    out_ref = ref(xr)
    gout = torch.randn(out_ref.shape).bfloat16()
    out_ref.backward(gout)

    xd = x.to(DEV).requires_grad_(True)
    f = compiled(dev)
    out = f(xd)
    assert out.requires_grad and out.grad_fn is not None
    assert_close(out.float(), out_ref.float(), 2e-2, "mlp forward")
    out.backward(gout.to(DEV))
    assert_close(xd.grad.float(), xr.grad.float(), 2e-2, "d/dx")
    for (name, p_ref), p_dev in zip(ref.named_parameters(), dev.parameters()):
        assert p_dev.grad is not None, name
        scale = float(p_ref.grad.float().abs().max())
        assert float((p_dev.grad.float().cpu() - p_ref.grad.float()).abs().max()) <= 2e-2 * max(scale, 1.0), name


def test_matmul_operator_forms():
    """`x @ w`, torch.mm and torch.matmul with a 2-D right operand lower to the GEMM template with the
    weight read in place; a relu behind it joins as the GEMM's epilogue."""
    gen = torch.Generator().manual_seed(51)
    x = torch.randn(3, 200, 256, generator=gen).bfloat16()
    w = (torch.randn(256, 384, generator=gen) / 16).bfloat16()
    for name, fn in {"matmul_relu": lambda a, b: torch.relu(a @ b), "matmul_scale": lambda a, b: torch.matmul(a, b) * 0.5}.items():
        want = rp.run_reference(fn, [x, w])
        got = compiled(fn)(x.to(DEV), w.to(DEV))
        assert got.shape == want.shape
        assert_close(got.float(), want.float(), 2e-2, name)
    x2 = x[0].contiguous()
    assert_close(compiled(lambda a, b: torch.mm(a, b))(x2.to(DEV), w.to(DEV)).float(),
                 rp.run_reference(lambda a, b: torch.mm(a, b), [x2, w]).float(), 2e-2, "mm")
    bias = (0.5 * torch.randn(384, generator=gen)).bfloat16()
    addmm = lambda c, a, b: torch.relu(torch.addmm(c, a, b))  # noqa: E731  bias row + x @ W in the GEMM's epilogue
    assert_close(compiled(addmm)(bias.to(DEV), x2.to(DEV), w.to(DEV)).float(),
                 rp.run_reference(addmm, [bias, x2, w]).float(), 2e-2, "addmm")


def test_integer_graph_is_bit_exact():
    a = torch.randint(-1000, 1000, (33, 65), dtype=torch.int32)
    b = torch.randint(-2**31, 2**31 - 1, (33, 65), dtype=torch.int32)
    fn = lambda p, q: (p + q) * p - q  # noqa: E731
    got = compiled(fn)(a.to(DEV), b.to(DEV))
    assert got.dtype == torch.int32 and torch.equal(got.cpu(), fn(a, b))


def test_bf16_chain_with_cast_is_bit_exact():
    x, w, b = wl.inputs_reduce_mean(40, 512, seed=50)
    fn = lambda x, w, b: torch.relu(x * w + b).float() * 2.0  # noqa: E731
    want = rp.run_reference(fn, [x, w, b])
    got = compiled(fn)(x.to(DEV), w.to(DEV), b.to(DEV))
    assert got.dtype == torch.float32 and torch.equal(got.cpu(), want)


# ---------------------------------------------------------------- strided graph inputs feeding layout changes
@pytest.mark.parametrize("make_input", [lambda base: base.t(), lambda base: base[:, ::2], lambda base: base[3:40, 5:61]],
                         ids=["transposed", "every_other_column", "window"])
@pytest.mark.parametrize("fn", [
    lambda x: x.t() + 1.0,
    lambda x: x.permute(1, 0).contiguous() * 2.0,
    lambda x: x[1:, 2:] - 3.0,
    lambda x: x.sum(dim=0),
    lambda x: torch.softmax(x, dim=0),
    lambda x: x.reshape(-1) * 0.5,
], ids=["t", "permute", "slice", "sum_dim0", "softmax_dim0", "reshape"])
def test_strided_input_followed_by_a_layout_change(fn, make_input):
    """A plan's layout-change launches describe views of CONTIGUOUS buffers; a caller's strided
    tensor (a transpose, a column subset, a window of a larger tensor) must be gathered first, not
    re-interpreted with those strides."""
    gen = torch.Generator().manual_seed(123)
    base = torch.randn(48, 64, generator=gen)
    want = fn(make_input(base))
    x = make_input(base.to(DEV))
    assert not x.is_contiguous()
    with torch.no_grad():
        got = compiled(fn)(x)
    assert got.shape == want.shape
    assert_close(got.cpu(), want, 1e-5, "strided input")


# ---------------------------------------------------------------- compile cache and debug dump on the GPU
def test_compile_cache_hit_and_misses_on_gpu():
    """A second compile of the same graph returns the cached plan and the identical result; a change
    of dtype or of input strides is a different key (reference: utils/cache.py, jit_compiler.py:443-470,
    whose hash covers names and shapes only)."""
    from conductor_b200.compiler.gcu_backend import get_gcu_backend

    backend = get_gcu_backend()
    backend.clear_cache()
    a, b, c = (t.to(DEV) for t in wl.inputs_mul_add(128, 256, seed=71))
    first = compiled(wl.mul_add)(a, b, c)
    assert len(backend._compiled_functions) == 1
    plan = next(iter(backend._compiled_functions.values()))
    calls = plan.calls
    again = compiled(wl.mul_add)(a, b, c)                       # Dynamo retraces; the backend must not recompile
    assert len(backend._compiled_functions) == 1 and next(iter(backend._compiled_functions.values())) is plan
    assert plan.calls == calls + 1 and torch.equal(first, again)
    half = compiled(wl.mul_add)(a.bfloat16(), b.bfloat16(), c.bfloat16())
    assert len(backend._compiled_functions) == 2 and half.dtype == torch.bfloat16
    at = a.t().contiguous().t()                                  # same shape and dtype, other strides
    strided = compiled(wl.mul_add)(at, b, c)
    assert len(backend._compiled_functions) == 3 and torch.equal(strided, first)
    backend.clear_cache()


def test_debug_dump_of_a_gpu_compiled_graph_holds_the_source_that_ran(tmp_path):
    """With a dump directory set, compiling and running a graph whose cluster has no ahead-of-time
    kernel instance leaves the CUDA source of its run-time instance beside the plan -- the same
    text the library hands out for that launch -- and the result matches eager
    (reference: utils/artifacts.py:18-237 keeps the generated DSL and the compiled objects)."""
    import ctypes

    from conductor_b200.compiler.executor import make_descriptors
    from conductor_b200.compiler.gcu_backend import get_gcu_backend
    from conductor_b200.compiler.loader import load_library
    from conductor_b200.utils.artifacts import get_debug_manager
    from conductor_b200.utils.config import ConductorConfig, reset_config, set_config
    from conductor_b200.utils.tracer import reset_tracer

    def chain(x, y):
        return torch.tanh(x - y) * y

    cfg = ConductorConfig.load()
    cfg.debug.enabled = True
    cfg.debug.dump_dir = str(tmp_path / "dump")
    set_config(cfg)
    reset_tracer()
    backend = get_gcu_backend()
    backend.clear_cache()
    backend.jit_compiler.clear_cache()
    try:
        gen = torch.Generator().manual_seed(72)
        x, y = torch.randn(256, 512, generator=gen), torch.randn(256, 512, generator=gen)
        got = compiled(chain)(x.to(DEV), y.to(DEV))
        assert_close(got.cpu(), chain(x, y), 1e-5, "dumped graph")
        plan = next(iter(backend._compiled_functions.values()))
        name = plan.artifact.entry_point
        mgr = get_debug_manager()
        names = {p.name for p in mgr.list_artifacts(name)}
        assert {f"{name}.fx.txt", f"{name}.dag.txt", f"{name}.clusters.json", f"{name}.plan.txt", f"{name}.source0.cu"} <= names, names
        dumped = mgr.get_instance_source_path(name, 0).read_text()
        assert "tanh" in dumped and "__global__" in dumped
        # the library's own answer for the launch that ran
        launch = plan.launches[0]
        lib = load_library()
        ins = make_descriptors([torch.empty(b.shape, dtype=b.dtype) for b in launch.inputs])
        outs = make_descriptors([torch.empty(s, dtype=d) for s, d in zip(launch.out_shapes, launch.out_dtypes)])
        buf = ctypes.create_string_buffer(1 << 17)
        rc = lib.cdr_template_source(launch.template, ins, len(launch.inputs), outs, len(launch.outputs),
                                     ctypes.cast(ctypes.byref(launch.params), ctypes.c_void_p), ctypes.sizeof(launch.params),
                                     buf, len(buf), 0)
        assert rc == 0 and buf.value.decode() == dumped
    finally:
        reset_config()
        reset_tracer()
        backend.clear_cache()
        backend.jit_compiler.clear_cache()


# ---------------------------------------------------------------- host calls in overlapped row chunks
@pytest.mark.parametrize("case", ["mul_add", "reduce_mean", "softmax", "mlp", "attention"])
def test_host_call_in_row_chunks_matches_one_piece(case):
    """A host-tensor call of a row-parallel graph runs in row chunks on three streams (copy in,
    kernels, copy out overlapped); the result must be the one-piece result bit for bit, for
    pinned and for pageable inputs, with a ragged last chunk."""
    from conductor_b200.utils.config import get_config

    if case == "mul_add":
        fn, inputs = wl.mul_add, wl.inputs_mul_add(1000, 512, seed=81)
    elif case == "reduce_mean":
        fn, inputs = wl.reduce_mean_fusion, wl.inputs_reduce_mean(1000, 1024, seed=82)
    elif case == "softmax":
        fn, inputs = wl.softmax_forward, wl.inputs_softmax(777, 2048, seed=83)[:1]
    elif case == "mlp":
        fn, inputs = wl.make_mlp(256, 512, 256, seed=84), wl.inputs_mlp(1000, 256, seed=84)
    else:
        fn, inputs = wl.causal_attention, wl.inputs_attention(6, 2, 256, 64, seed=85)
    cfg = get_config().runtime
    old = cfg.host_chunk_bytes
    try:
        cfg.host_chunk_bytes = 0
        with torch.no_grad():
            whole = compiled(fn)(*inputs)
        nbytes = inputs[0].numel() * inputs[0].element_size()
        cfg.host_chunk_bytes = max(1, nbytes // 5)                  # five chunks, the last one shorter
        with torch.no_grad():
            f = compiled(fn)
            chunked = f(*inputs)
            pinned = f(*[t.pin_memory() for t in inputs])
        assert chunked.device.type == "cpu" and torch.equal(chunked, whole) and torch.equal(pinned, whole)
        from conductor_b200.compiler.gcu_backend import get_gcu_backend

        plan = list(get_gcu_backend()._compiled_functions.values())[-1]
        assert plan.chunked_calls == 2, (case, plan.chunked_calls)
    finally:
        cfg.host_chunk_bytes = old
