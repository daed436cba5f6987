"""GPU parity: the CUDA kernel templates, called through the C ABI, against the golden
vectors, the C oracle and the reference's executed path (eager on CPU) on identical seeded
inputs.  Tolerances are the benchmark's: bit-exact for integer work and for the fp32/bf16
+,-,*,/ chains, max-abs/rel <= 1e-5 for fp32 transcendental/reduction results, <= 2e-2 bf16."""
import ctypes
import math

import numpy as np
import pytest
import torch

import abi_util as abi
from abi_util import COL, FULL, ROW, SCALAR
from conftest import assert_close, bf16_bits_to_tensor, load_golden, tensor_to_bf16_bits
from conductor_b200.codegen.kernel_templates import CdrReduceParams
from conductor_b200.codegen.operator_registry import EwOp, ReduceOp, Template
from conductor_b200.compiler.loader import load_library
from oracle import reference_path as rp
from oracle import scalar

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
F32_TOL, BF16_TOL = 1e-5, 2e-2


def bits_equal(a: torch.Tensor, b: torch.Tensor) -> bool:
    a, b = a.detach().cpu().contiguous(), b.detach().cpu().contiguous()
    if a.dtype != b.dtype or a.shape != b.shape:
        return False
    return torch.equal(a.view(torch.uint8), b.view(torch.uint8))


def cuda(*ts):
    return [t.to(DEV) for t in ts]


# ---------------------------------------------------------------- K1 elementwise
def test_mul_add_golden_bit_exact(executor):
    g = load_golden("c1_mul_add")
    a, b, c = cuda(g["a"], g["b"], g["c"])
    out = torch.empty_like(a)
    abi.launch(Template.ELEMENTWISE, [a, b, c], [out], abi.mul_add_program())
    assert bits_equal(out, g["out"])


@pytest.mark.parametrize("shape", [(1,), (3,), (4,), (257,), (1000, 3), (129, 1024), (7, 5, 33)])
def test_mul_add_ragged_sizes_bit_exact(executor, shape):
    gen = torch.Generator().manual_seed(11)
    a, b, c = (torch.randn(shape, generator=gen) for _ in range(3))
    want = torch.from_numpy(scalar.mul_add_f32(a.numpy(), b.numpy(), c.numpy()))
    assert torch.equal(want, a * b + c)                      # oracle == eager, bit for bit
    da, db, dc = cuda(a, b, c)
    out = torch.empty_like(da)
    abi.launch(Template.ELEMENTWISE, [da, db, dc], [out], abi.mul_add_program())
    assert bits_equal(out, want)


def test_mul_add_misaligned_pointers(executor):
    gen = torch.Generator().manual_seed(12)
    base = [torch.randn(4099, generator=gen).to(DEV) for _ in range(3)]
    a, b, c = (t[1:4098] for t in base)                      # data_ptr is 4 bytes off 16-byte alignment
    out_base = torch.zeros(4101, device=DEV)
    out = out_base[3:4100]
    abi.launch(Template.ELEMENTWISE, [a, b, c], [out], abi.mul_add_program())
    assert bits_equal(out, (a.cpu() * b.cpu() + c.cpu()))
    assert out_base[:3].abs().sum().item() == 0               # nothing written before the view


def test_elementwise_empty(executor):
    a = torch.empty(0, 16, device=DEV)
    out = torch.empty_like(a)
    abi.launch(Template.ELEMENTWISE, [a, a, a], [out], abi.mul_add_program())


def test_mul_add_bf16_bit_exact(executor):
    gen = torch.Generator().manual_seed(13)
    a, b, c = (torch.randn(333, 264, generator=gen).bfloat16() for _ in range(3))
    want = bf16_bits_to_tensor(scalar.mul_add_bf16(*(tensor_to_bf16_bits(t) for t in (a, b, c))))
    assert bits_equal(want, a * b + c)
    da, db, dc = cuda(a, b, c)
    out = torch.empty_like(da)
    abi.launch(Template.ELEMENTWISE, [da, db, dc], [out], abi.mul_add_program(torch.bfloat16))
    assert bits_equal(out, want)


def test_addcdiv_and_relu_named_chains(executor):
    gen = torch.Generator().manual_seed(14)
    a, b = torch.randn(64, 300, generator=gen), torch.randn(64, 300, generator=gen)
    c = torch.rand(64, 300, generator=gen) + 0.5
    da, db, dc = cuda(a, b, c)
    out = torch.empty_like(da)
    prog = abi.ew_program(3, [(EwOp.ADDCDIV, 0, 1, 2, 1.0, torch.float32)], [3])
    abi.launch(Template.ELEMENTWISE, [da, db, dc], [out], prog)
    assert bits_equal(out, torch.from_numpy(scalar.addcdiv_f32(a.numpy(), b.numpy(), c.numpy(), 1.0)))
    assert bits_equal(out, torch.addcdiv(a, b, c, value=1.0))
    x = torch.randn(128, 256, generator=gen)
    x[0, :4] = torch.tensor([float("nan"), -0.0, float("inf"), -float("inf")])
    dx = x.to(DEV)
    out = torch.empty_like(dx)
    abi.launch(Template.ELEMENTWISE, [dx], [out], abi.ew_program(1, [(EwOp.RELU, 0, 0, 0, 0, torch.float32)], [1]))
    assert_close(out, torch.relu(x), 0.0, "relu")
    assert torch.equal(out.cpu()[1:], torch.from_numpy(scalar.relu_f32(x.numpy()))[1:])


def test_interpreted_program_with_broadcasts(executor):
    # (sigmoid(x * w + 1.5) - col) / s : row, column and scalar broadcasts, unary math
    gen = torch.Generator().manual_seed(15)
    x = torch.randn(37, 64, generator=gen)
    w = torch.randn(64, generator=gen)
    col = torch.randn(37, 1, generator=gen)
    s = torch.tensor(3.0)
    want = (torch.sigmoid(x * w + 1.5) - col) / s
    prog = abi.ew_program(4, [
        (EwOp.MUL, 0, 1, 0, 0, torch.float32), (EwOp.ADD_IMM, 4, 0, 0, 1.5, torch.float32),
        (EwOp.SIGMOID, 5, 0, 0, 0, torch.float32), (EwOp.SUB, 6, 2, 0, 0, torch.float32),
        (EwOp.DIV, 7, 3, 0, 0, torch.float32)], [8], [FULL, ROW, COL, SCALAR])
    dx, dw, dcol, ds = cuda(x, w, col, s)
    out = torch.empty_like(dx)
    abi.launch(Template.ELEMENTWISE, [dx, dw, dcol, ds], [out], prog)
    assert_close(out, want, F32_TOL, "interpreted chain")
    # same program, ragged row length -> scalar path
    x2, w2 = torch.randn(37, 63, generator=gen), torch.randn(63, generator=gen)
    want2 = (torch.sigmoid(x2 * w2 + 1.5) - col) / s
    dx2, dw2 = cuda(x2, w2)
    out2 = torch.empty_like(dx2)
    abi.launch(Template.ELEMENTWISE, [dx2, dw2, dcol, ds], [out2], prog)
    assert_close(out2, want2, F32_TOL, "interpreted chain, scalar path")


def test_runtime_instance_mixed_dtypes_and_tail(executor):
    """A program with no ahead-of-time instance, on shapes the vector skeleton takes (aligned rows)
    plus a tail that is not a whole vector: mixed fp32 / bf16 / fp16 inputs, per-op rounding."""
    gen = torch.Generator().manual_seed(17)
    rows, cols = 257, 1032
    x = torch.randn(rows, cols, generator=gen)
    w = torch.randn(cols, generator=gen).bfloat16()
    col = torch.randn(rows, 1, generator=gen).half()
    s = torch.tensor(0.75)
    # eager semantics: every op rounds to its own result type
    t1 = x * w.float()                                   # fp32
    t2 = torch.tanh(t1)                                  # fp32
    t3 = (t2 + 0.5 * col.float() * s).bfloat16()         # addcmul, rounded to bf16
    want_a = (2.0 - t3.float()).bfloat16()               # bf16 output
    want_b = torch.maximum(t2, x)                        # fp32 output
    prog = abi.ew_program(4, [
        (EwOp.MUL, 0, 1, 0, 0, torch.float32), (EwOp.TANH, 4, 0, 0, 0, torch.float32),
        (EwOp.ADDCMUL, 5, 2, 3, 0.5, torch.bfloat16), (EwOp.RSUB_IMM, 6, 0, 0, 2.0, torch.bfloat16),
        (EwOp.MAX, 5, 0, 0, 0, torch.float32)], [7, 8], [FULL, ROW, COL, SCALAR])
    dx, dw, dcol, ds = cuda(x, w, col, s)
    oa = torch.empty(rows, cols, dtype=torch.bfloat16, device=DEV)
    ob = torch.empty(rows, cols, dtype=torch.float32, device=DEV)
    abi.launch(Template.ELEMENTWISE, [dx, dw, dcol, ds], [oa, ob], prog)
    assert_close(oa.float(), want_a.float(), BF16_TOL, "run-time instance, bf16 output")
    assert_close(ob, want_b, F32_TOL, "run-time instance, fp32 output")
    # +,-,*,/ only: bit-exact against eager, on a flat length that leaves a scalar tail
    n = 8 * 4096 + 5
    a, b = torch.randn(n, generator=gen), torch.randn(n, generator=gen) + 3.0
    prog2 = abi.ew_program(2, [(EwOp.SUB, 0, 1, 0, 0, torch.float32), (EwOp.DIV, 2, 1, 0, 0, torch.float32),
                               (EwOp.MUL_IMM, 3, 0, 0, 1.25, torch.float32)], [4])
    da, db = cuda(a, b)
    out = torch.empty_like(da)
    abi.launch(Template.ELEMENTWISE, [da, db], [out], prog2)
    assert bits_equal(out, ((a - b) / b) * 1.25)


def test_packed_bf16_chain_bit_exact(executor):
    """All-bf16 chains of +,-,*,relu,neg,abs,max,min run on bf16x2 instructions in their run-time
    instance; every op must round exactly like eager (fp32 op, then round to bf16), NaN included."""
    gen = torch.Generator().manual_seed(18)
    rows, cols = 129, 520
    x = (torch.randn(rows, cols, generator=gen) * 3).bfloat16()
    w = torch.randn(cols, generator=gen).bfloat16()
    b = torch.randn(cols, generator=gen).bfloat16()
    col = torch.randn(rows, 1, generator=gen).bfloat16()
    x[3, 7] = float("nan")
    x[5, 9] = float("inf")
    x[6, 11] = 1e-39        # bf16 subnormal
    t = torch.relu(x * w - b) + 1.5                      # eager bf16: each op rounds
    want1 = torch.minimum(torch.maximum(-t, col), torch.abs(x))
    want2 = 2.0 - t * 0.5
    bf = torch.bfloat16
    prog = abi.ew_program(4, [
        (EwOp.MUL, 0, 1, 0, 0, bf), (EwOp.SUB, 4, 2, 0, 0, bf), (EwOp.RELU, 5, 0, 0, 0, bf), (EwOp.ADD_IMM, 6, 0, 0, 1.5, bf),
        (EwOp.NEG, 7, 0, 0, 0, bf), (EwOp.MAX, 8, 3, 0, 0, bf), (EwOp.ABS, 0, 0, 0, 0, bf), (EwOp.MIN, 9, 10, 0, 0, bf),
        (EwOp.MUL_IMM, 7, 0, 0, 0.5, bf), (EwOp.RSUB_IMM, 12, 0, 0, 2.0, bf)], [11, 13], [FULL, ROW, ROW, COL])
    dx, dw, db, dcol = cuda(x, w, b, col)
    o1, o2 = torch.empty_like(dx), torch.empty_like(dx)
    abi.launch(Template.ELEMENTWISE, [dx, dw, db, dcol], [o1, o2], prog)
    for got, want, name in ((o1, want1, "min/max/abs"), (o2, want2, "imm ops")):
        g, e = got.cpu(), want
        same = (g.view(torch.int16) == e.view(torch.int16)) | (torch.isnan(g) & torch.isnan(e))
        assert bool(same.all()), f"{name}: {int((~same).sum())} elements differ from eager"
    # the same chain reduced over the last dimension: fp32 accumulation of the bf16 chain values
    chain = abi.ew_program(3, [(EwOp.MUL, 0, 1, 0, 0, bf), (EwOp.SUB, 3, 2, 0, 0, bf), (EwOp.RELU, 4, 0, 0, 0, bf)], [5],
                           [FULL, ROW, ROW])
    xc = x.clone()
    xc[3, 7] = 0.25
    xc[5, 9] = -2.0
    val = torch.relu(xc * w - b).float()
    for op, want in ((ReduceOp.SUM, val.double().sum(-1).float()), (ReduceOp.MEAN, val.double().mean(-1).float()),
                     (ReduceOp.MAX, val.amax(-1)), (ReduceOp.MIN, val.amin(-1))):
        out = torch.empty(rows, device=DEV)
        abi.launch(Template.ROW_REDUCE, [xc.to(DEV), dw, db], [out], reduce_params(chain, op))
        assert_close(out, want, F32_TOL, f"packed chain reduce op {op}")


def test_two_outputs(executor):
    gen = torch.Generator().manual_seed(16)
    a, b = torch.randn(50, 40, generator=gen), torch.randn(50, 40, generator=gen)
    prog = abi.ew_program(2, [(EwOp.ADD, 0, 1, 0, 0, torch.float32), (EwOp.MUL, 2, 0, 0, 0, torch.float32)], [2, 3])
    da, db = cuda(a, b)
    o1, o2 = torch.empty_like(da), torch.empty_like(da)
    abi.launch(Template.ELEMENTWISE, [da, db], [o1, o2], prog)
    assert bits_equal(o1, a + b) and bits_equal(o2, (a + b) * a)


def test_integer_chain_bit_exact(executor):
    rng = np.random.default_rng(2)
    a = rng.integers(-10, 11, (6, 17, 64), dtype=np.int32)
    b = rng.integers(-2**31, 2**31 - 1, (6, 17, 64), dtype=np.int32)        # wraps
    da, db = torch.from_numpy(a).to(DEV), torch.from_numpy(b).to(DEV)
    out = torch.empty_like(da)
    abi.launch(Template.ELEMENTWISE, [da, db], [out], abi.ew_program(2, [(EwOp.ADD, 0, 1, 0, 0, torch.int32)], [2]))
    assert np.array_equal(out.cpu().numpy(), scalar.add_i32(a, b))
    assert np.array_equal(out.cpu().numpy(), (torch.from_numpy(a) + torch.from_numpy(b)).numpy())
    a64 = torch.from_numpy(rng.integers(-2**40, 2**40, (1000,), dtype=np.int64))
    d64 = a64.to(DEV)
    out64 = torch.empty_like(d64)
    prog = abi.ew_program(1, [(EwOp.MUL, 0, 0, 0, 0, torch.int64), (EwOp.ADD_IMM, 1, 0, 0, 7, torch.int64)], [2])
    abi.launch(Template.ELEMENTWISE, [d64], [out64], prog)
    assert torch.equal(out64.cpu(), a64 * a64 + 7)


def test_bad_arguments_return_status_not_crash(executor):
    a = torch.randn(8, 8, device=DEV)
    out = torch.empty(8, 9, device=DEV)
    assert abi.launch(Template.ELEMENTWISE, [a, a, a], [out], abi.mul_add_program(), check=False) == -1
    assert abi.launch(99, [a], [a], abi.mul_add_program(), check=False) == -2
    bad = abi.ew_program(3, [(EwOp.MUL, 0, 7, 0, 0, torch.float32)], [3])     # reads an undefined register
    assert abi.launch(Template.ELEMENTWISE, [a, a, a], [torch.empty_like(a)], bad, check=False) == -1
    assert b"register" in executor.lib.cdr_last_error()


# ---------------------------------------------------------------- K2 row reduce
def reduce_params(chain, op):
    p = CdrReduceParams()
    p.chain = chain
    p.reduce_op = op
    return p


def mar_chain(dtype):
    return abi.ew_program(3, [(EwOp.MUL, 0, 1, 0, 0, dtype), (EwOp.ADD, 3, 2, 0, 0, dtype),
                              (EwOp.RELU, 4, 0, 0, 0, dtype)], [5], [FULL, ROW, ROW])


def test_reduce_mean_golden(executor):
    g = load_golden("c2_reduce_mean")
    x, w, b = cuda(g["x"], g["w"], g["b"])
    out = torch.empty(x.shape[0], device=DEV)
    abi.launch(Template.ROW_REDUCE, [x, w, b], [out], reduce_params(mar_chain(torch.bfloat16), ReduceOp.MEAN))
    assert_close(out, g["out"], F32_TOL, "reduce_mean golden")


@pytest.mark.parametrize("rows,cols", [(1, 8), (5, 256), (33, 512), (64, 4096), (7, 2048), (19, 8200), (3, 16384),
                                       (9, 100), (4, 20000)])
def test_reduce_mean_shapes(executor, rows, cols):
    x, w, b = rp.inputs_reduce_mean(rows, cols, seed=21)
    want = torch.from_numpy(scalar.mean_relu_mul_add_bf16(*(tensor_to_bf16_bits(t) for t in (x, w, b))))
    assert_close(rp.run_reference(rp.reduce_mean_fusion, [x, w, b]), want, F32_TOL, "oracle vs reference path")
    dx, dw, db = cuda(x, w, b)
    out = torch.empty(rows, device=DEV)
    abi.launch(Template.ROW_REDUCE, [dx, dw, db], [out], reduce_params(mar_chain(torch.bfloat16), ReduceOp.MEAN))
    assert_close(out, want, F32_TOL, f"reduce_mean {rows}x{cols}")


def test_row_sum_max_fp32(executor):
    gen = torch.Generator().manual_seed(22)
    x = torch.randn(45, 1000, generator=gen)
    dx = x.to(DEV)
    ident = abi.ew_program(1, [], [0])
    for op, want in ((ReduceOp.SUM, torch.from_numpy(scalar.row_sum_f32(x.numpy()))),
                     (ReduceOp.MEAN, torch.from_numpy(scalar.row_sum_f32(x.numpy(), mean=True))),
                     (ReduceOp.MAX, x.amax(-1)), (ReduceOp.MIN, x.amin(-1))):
        out = torch.empty(45, device=DEV)
        abi.launch(Template.ROW_REDUCE, [dx], [out], reduce_params(ident, op))
        assert_close(out, want, F32_TOL, f"row reduce op {op}")


@pytest.mark.parametrize("rows,cols", [(37, 64), (9, 1024), (5, 4104), (3, 70000)])
def test_row_reduce_runtime_instance(executor, rows, cols):
    """Chains with no ahead-of-time reduce instance on vector-shaped rows (warp-per-row and
    CTA-per-row skeletons): mixed dtypes, every reduce op, NaN propagation through max."""
    gen = torch.Generator().manual_seed(24)
    x = torch.randn(rows, cols, generator=gen).bfloat16()
    w = torch.randn(cols, generator=gen)
    col = torch.randn(rows, 1, generator=gen)
    val = torch.sigmoid(x.float() * w) - col                       # fp32 chain over a bf16 input
    chain = abi.ew_program(3, [(EwOp.MUL, 0, 1, 0, 0, torch.float32), (EwOp.SIGMOID, 3, 0, 0, 0, torch.float32),
                               (EwOp.SUB, 4, 2, 0, 0, torch.float32)], [5], [FULL, ROW, COL])
    dx, dw, dcol = cuda(x, w, col)
    for op, want in ((ReduceOp.SUM, val.double().sum(-1).float()), (ReduceOp.MEAN, val.double().mean(-1).float()),
                     (ReduceOp.MAX, val.amax(-1)), (ReduceOp.MIN, val.amin(-1))):
        out = torch.empty(rows, device=DEV)
        abi.launch(Template.ROW_REDUCE, [dx, dw, dcol], [out], reduce_params(chain, op))
        tol = F32_TOL * max(1.0, float(want.abs().max())) if op == ReduceOp.SUM else F32_TOL
        assert_close(out, want, tol, f"row reduce run-time instance op {op} {rows}x{cols}")
    # NaN in one row poisons that row's max only; bf16 output rounds once at the end
    xn = x.clone()
    xn[rows // 2, cols - 3] = float("nan")
    out = torch.empty(rows, dtype=torch.bfloat16, device=DEV)
    abi.launch(Template.ROW_REDUCE, [xn.to(DEV), dw, dcol], [out], reduce_params(chain, ReduceOp.MAX))
    got = out.cpu().float()
    assert torch.isnan(got[rows // 2]) and int(torch.isnan(got).sum()) == 1
    keep = torch.arange(rows) != rows // 2
    assert_close(got[keep], val.amax(-1).bfloat16().float()[keep], BF16_TOL, "bf16 row max")


def test_full_reduce_with_workspace(executor):
    gen = torch.Generator().manual_seed(23)
    x = torch.randn(300, 517, generator=gen)
    dx = x.to(DEV)
    out = torch.empty((), device=DEV)
    p = reduce_params(abi.ew_program(1, [(EwOp.MUL, 0, 0, 0, 0, torch.float32)], [1]), ReduceOp.SUM)
    n = abi.workspace_bytes(Template.FULL_REDUCE, [dx], [out], p)
    assert n > 0
    assert abi.launch(Template.FULL_REDUCE, [dx], [out], p, check=False) == -6        # no workspace
    ws = torch.empty(n, dtype=torch.uint8, device=DEV)
    for _ in range(2):                                                               # reusable scratch
        abi.launch(Template.FULL_REDUCE, [dx], [out], p, workspace=ws)
        assert_close(out, (x.double() * x.double()).sum().float(), F32_TOL, "sum of squares")


@pytest.mark.parametrize("M,N,dtype", [(8192, 4096, torch.bfloat16), (777, 1031, torch.float32), (5, 8, torch.float16),
                                       (1, 300, torch.bfloat16), (4096, 256, torch.float32), (33, 7, torch.bfloat16),
                                       (0, 64, torch.float32)])
def test_col_sum_against_fp64_host_sum(executor, M, N, dtype):
    """out[n] = sum_m x[m, n] (the bias gradient of a linear layer): fp32 accumulation in a fixed
    order, compared with a double-precision sum on the host; two runs are bit-identical."""
    gen = torch.Generator().manual_seed(M * 131 + N)
    x = torch.randn(M, N, generator=gen).to(dtype)
    want = x.double().sum(0)
    xd = x.to(DEV)
    outs = []
    for _ in range(2):
        out = torch.full((N,), float("nan"), dtype=dtype, device=DEV)
        ws = torch.full((abi.workspace_bytes(Template.COL_SUM, [xd], [out]),), 0xCD, dtype=torch.uint8, device=DEV)
        abi.launch(Template.COL_SUM, [xd], [out], workspace=ws)
        outs.append(out.cpu())
    assert torch.equal(outs[0], outs[1])
    tol = 1e-5 if dtype == torch.float32 else BF16_TOL
    scale = max(1.0, float(want.abs().max())) if M else 1.0
    assert float((outs[0].double() - want).abs().max()) <= tol * scale
    # shape checks: an output whose size does not divide the input, a missing workspace
    bad = torch.empty(N + 1, dtype=dtype, device=DEV)
    if M:
        assert abi.launch(Template.COL_SUM, [xd], [bad], workspace=ws, check=False) == -1
    assert abi.launch(Template.COL_SUM, [xd], [out], check=False) == -6


# ---------------------------------------------------------------- K3 softmax
def test_softmax_golden(executor):
    g = load_golden("c3_softmax")
    logits, grad, y = cuda(g["logits"], g["grad"], g["y"])
    out = torch.empty_like(logits)
    abi.launch(Template.SOFTMAX_FWD, [logits], [out])
    assert_close(out, g["y"], F32_TOL, "softmax fwd golden")
    dx = torch.empty_like(logits)
    abi.launch(Template.SOFTMAX_BWD, [grad, y], [dx])
    assert_close(dx, g["dx"], F32_TOL, "softmax bwd golden")


def test_softmax_known_answers(executor):
    ones = torch.ones(256, 512, device=DEV)
    out = torch.empty_like(ones)
    abi.launch(Template.SOFTMAX_FWD, [ones], [out])
    assert (out - 1.0 / 512).abs().max().item() <= 1e-6
    y = torch.full((16, 128), 0.5, device=DEV)
    dy = torch.ones(16, 128, device=DEV)
    dx = torch.empty_like(y)
    abi.launch(Template.SOFTMAX_BWD, [dy, y], [dx])
    assert (dx + 31.5).abs().max().item() <= 1e-6


@pytest.mark.parametrize("rows,cols", [(1, 4), (3, 32), (17, 100), (5, 1000), (33, 1024), (9, 8192), (2, 16384),
                                       (2, 32768), (2, 40000), (4, 8191)])
def test_softmax_shapes(executor, rows, cols):
    logits, grad = rp.inputs_softmax(rows, cols, seed=31)
    want = torch.from_numpy(scalar.softmax_f32(logits.numpy()))
    assert_close(torch.softmax(logits, -1), want, F32_TOL, "oracle vs eager")
    dl, dg = cuda(logits, grad)
    out = torch.empty_like(dl)
    abi.launch(Template.SOFTMAX_FWD, [dl], [out])
    assert_close(out, want, F32_TOL, f"softmax fwd {rows}x{cols}")
    assert (out.sum(-1) - 1).abs().max().item() < 1e-4
    dx = torch.empty_like(dl)
    abi.launch(Template.SOFTMAX_BWD, [dg, out], [dx])
    want_dx = torch.from_numpy(scalar.softmax_backward_f32(out.cpu().numpy(), grad.numpy()))
    assert_close(dx, want_dx, F32_TOL, f"softmax bwd {rows}x{cols}")


def test_softmax_bwd_matches_jacobian_form(executor):
    logits, grad = rp.inputs_softmax(8, 256, seed=32)
    y = torch.softmax(logits, -1)
    want = torch.from_numpy(scalar.softmax_backward_f32(y.numpy(), grad.numpy(), jacobian=True))
    dg, dy = cuda(grad, y)
    dx = torch.empty_like(dy)
    abi.launch(Template.SOFTMAX_BWD, [dg, dy], [dx])
    assert_close(dx, want, F32_TOL, "softmax bwd vs O(n^2) Jacobian")


def test_softmax_special_values(executor):
    x = torch.randn(6, 512)
    x[0, :] = -float("inf")                    # all -inf -> NaN row, as eager
    x[1, 5:] = -float("inf")                   # partly masked
    x[2, 7] = float("inf")                     # inf - inf -> NaN row
    x[3, 9] = float("nan")
    x[4] = 1e30
    want = torch.softmax(x, -1)
    dx = x.to(DEV)
    out = torch.empty_like(dx)
    abi.launch(Template.SOFTMAX_FWD, [dx], [out])
    assert_close(out, want, F32_TOL, "softmax special values")


def test_softmax_bf16(executor):
    gen = torch.Generator().manual_seed(33)
    x = (3 * torch.randn(40, 1024, generator=gen)).bfloat16()
    g = torch.randn(40, 1024, generator=gen).bfloat16()
    y = torch.softmax(x, -1)
    dxr = torch._softmax_backward_data(g, y, -1, torch.bfloat16)
    dx_, dg_, dy_ = cuda(x, g, y)
    out = torch.empty_like(dx_)
    abi.launch(Template.SOFTMAX_FWD, [dx_], [out])
    assert_close(out.float(), y.float(), BF16_TOL, "softmax fwd bf16")
    dx = torch.empty_like(dx_)
    abi.launch(Template.SOFTMAX_BWD, [dg_, dy_], [dx])
    assert_close(dx.float(), dxr.float(), BF16_TOL, "softmax bwd bf16")


# ---------------------------------------------------------------- host-pointer entry point
def test_execute_host_round_trip(executor):
    g = load_golden("c1_mul_add")
    out = torch.empty_like(g["a"])
    rc = abi.execute_host(Template.ELEMENTWISE, [g["a"], g["b"], g["c"]], [out], abi.mul_add_program())
    assert rc == 0, executor.lib.cdr_last_error()
    assert bits_equal(out, g["out"])
    g3 = load_golden("c3_softmax")
    y = torch.empty_like(g3["logits"])
    assert abi.execute_host(Template.SOFTMAX_FWD, [g3["logits"]], [y]) == 0
    assert_close(y, g3["y"], F32_TOL, "host softmax")
    assert executor.lib.cdr_release_host_arena(-1) == 0


# ---------------------------------------------------------------- full benchmark sizes
def test_full_size_mul_add_bit_exact(executor):
    a, b, c = rp.inputs_mul_add()
    want = rp.run_reference(rp.mul_add, [a, b, c])
    da, db, dc = cuda(a, b, c)
    out = torch.empty_like(da)
    abi.launch(Template.ELEMENTWISE, [da, db, dc], [out], abi.mul_add_program())
    assert bits_equal(out, want)


def test_full_size_reduce_mean(executor):
    x, w, b = rp.inputs_reduce_mean()
    want = rp.run_reference(rp.reduce_mean_fusion, [x, w, b])
    dx, dw, db = cuda(x, w, b)
    out = torch.empty(x.shape[0], device=DEV)
    abi.launch(Template.ROW_REDUCE, [dx, dw, db], [out], reduce_params(mar_chain(torch.bfloat16), ReduceOp.MEAN))
    assert_close(out, want, F32_TOL, "full-size reduce_mean")


def test_full_size_softmax(executor):
    logits, grad = rp.inputs_softmax()
    y_ref = rp.run_reference(rp.softmax_forward, [logits])
    dl = logits.to(DEV)
    y = torch.empty_like(dl)
    abi.launch(Template.SOFTMAX_FWD, [dl], [y])
    assert_close(y, y_ref, F32_TOL, "full-size softmax fwd")
    assert (y.sum(-1) - 1).abs().max().item() < 1e-4          # rows are distributions
    del dl
    dx_ref = rp.run_reference(rp.softmax_backward, [grad, y_ref])
    dg = grad.to(DEV)
    dx = torch.empty_like(dg)
    abi.launch(Template.SOFTMAX_BWD, [dg, y], [dx])
    assert_close(dx, dx_ref, F32_TOL, "full-size softmax bwd")
    assert dx.sum(-1).abs().max().item() < 1e-3               # softmax gradients sum to zero per row


def test_strided_copy_template(executor):
    """CDR_T_COPY gathers a strided view into a contiguous tensor, bit-exactly: vector path (inner
    dimension contiguous), scalar path (transposes of the inner dimension), every element size."""
    gen = torch.Generator().manual_seed(92)
    views = []
    x = torch.randn(2, 24, 4, 64, generator=gen).bfloat16().to(DEV)
    views += [x.transpose(1, 2), x.permute(2, 0, 1, 3), x.permute(0, 1, 3, 2), x[:, ::2], x[..., 8:40]]
    y = torch.randn(37, 53, generator=gen).to(DEV)
    views += [y.t(), y[3:, 5:], y.t()[::3]]
    views += [torch.arange(3 * 5 * 7, device=DEV).reshape(3, 5, 7).permute(2, 0, 1),
              (torch.rand(9, 11, generator=gen) > 0.5).to(DEV).t(),
              torch.arange(60, dtype=torch.int64, device=DEV).reshape(6, 10).t()]
    for v in views:
        out = torch.empty(v.shape, dtype=v.dtype, device=DEV)
        abi.launch(Template.COPY, [v], [out])
        assert torch.equal(out, v), (tuple(v.shape), v.stride(), v.dtype)
    out = torch.empty(5, 4, device=DEV)
    assert abi.launch(Template.COPY, [y[:4, :5]], [out], check=False) == -1          # shapes differ
    # a strided output view: parts written into slices of one result (concatenation), vector and
    # scalar paths, neighbours untouched
    whole = torch.full((2, 24, 4, 96), -7.0, device=DEV).bfloat16()
    abi.launch(Template.COPY, [x], [whole[..., 16:80]])
    assert torch.equal(whole[..., 16:80], x) and bool((whole[..., :16] == -7).all()) and bool((whole[..., 80:] == -7).all())
    wide = torch.zeros(37, 60, device=DEV)
    abi.launch(Template.COPY, [y], [wide[:, 3:56]])
    assert torch.equal(wide[:, 3:56], y) and bool((wide[:, :3] == 0).all()) and bool((wide[:, 56:] == 0).all())
    square = torch.zeros(9, 9, device=DEV)
    abi.launch(Template.COPY, [y[:7, :7].t()], [square.t()[2:, 1:8]])                 # both sides strided
    assert torch.equal(square[1:8, 2:], y[:7, :7]) and float(square[0].abs().sum() + square[:, :2].abs().sum()) == 0.0
    assert abi.launch(Template.COPY, [y[:, :1]], [wide[:, :1].expand(37, 1)], check=False) == 0
    assert abi.launch(Template.COPY, [y], [torch.zeros(37, 1, device=DEV).expand(37, 53)], check=False) != 0   # stride-0 output


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32, torch.int64, torch.bool])
def test_transposing_copies_take_the_tiled_paths(executor, dtype):
    """Views whose unit-stride dimension is not the innermost one go through a shared-memory tile:
    the 16-byte form when every extent and stride allows it, the element form otherwise (ragged
    extents, odd strides, 1-byte types), with batch dimensions around the transposed pair and with
    a strided output.  All bit-exact."""
    gen = torch.Generator().manual_seed(93)

    def rnd(*shape):
        t = torch.randn(*shape, generator=gen) * 50
        return (t > 0).to(DEV) if dtype == torch.bool else t.to(dtype).to(DEV)

    big = rnd(320, 448)
    views = [big.t(),                                     # whole-vector extents: 16-byte form
             rnd(3, 136, 264).transpose(1, 2),            # batched
             rnd(2, 72, 3, 40).permute(0, 2, 3, 1),       # [B, S, H, D] -> [B, H, D, S]
             rnd(129, 67).t(),                            # ragged: element form
             rnd(5, 33, 130).transpose(0, 2),             # unit-stride dimension lands first
             big[8:, 16:].t(),                            # offset base, still aligned for 2-byte and wider
             big[1:, 3:].t()]                             # misaligned base: element form
    for v in views:
        out = torch.empty(v.shape, dtype=v.dtype, device=DEV)
        abi.launch(Template.COPY, [v], [out])
        assert torch.equal(out, v), (tuple(v.shape), v.stride(), v.dtype)
    # transposed read into a slice of a wider result
    wide = torch.zeros(448, 400, dtype=dtype, device=DEV)
    abi.launch(Template.COPY, [big.t()], [wide[:, 40:360]])
    assert torch.equal(wide[:, 40:360], big.t()) and bool((wide[:, :40] == 0).all()) and bool((wide[:, 360:] == 0).all())


def test_layer_norm_template(executor):
    """CDR_T_LAYER_NORM through the C ABI against a float64 evaluation: row lengths from one vector
    to the 1024-thread variant, with and without scale / shift, bf16, and the refusals."""
    from conductor_b200.codegen.kernel_templates import CdrNormParams

    gen = torch.Generator().manual_seed(91)
    for rows, cols in ((3, 4), (17, 96), (64, 1024), (9, 4096), (5, 16384)):
        x = torch.randn(rows, cols, generator=gen) * 2 + 0.5
        w, b = torch.randn(cols, generator=gen), torch.randn(cols, generator=gen)
        xd = x.double()
        norm = (xd - xd.mean(-1, keepdim=True)) / torch.sqrt(xd.var(-1, unbiased=False, keepdim=True) + 1e-5)
        dx, dw, db = cuda(x, w, b)
        out = torch.empty_like(dx)
        abi.launch(Template.LAYER_NORM, [dx, dw, db], [out], CdrNormParams(1e-5, 1, 1, 0))
        assert_close(out, (norm * w.double() + b.double()).float(), 4e-5, f"layer_norm {rows}x{cols}")
        abi.launch(Template.LAYER_NORM, [dx], [out], CdrNormParams(1e-5, 0, 0, 0))
        assert_close(out, norm.float(), 4e-5, f"layer_norm plain {rows}x{cols}")
        abi.launch(Template.LAYER_NORM, [dx, db], [out], CdrNormParams(1e-5, 0, 1, 0))
        assert_close(out, (norm + b.double()).float(), 4e-5, f"layer_norm shift only {rows}x{cols}")
    xb = (torch.randn(33, 512, generator=gen) * 3).bfloat16()
    outb = torch.empty(33, 512, dtype=torch.bfloat16, device=DEV)
    abi.launch(Template.LAYER_NORM, [xb.to(DEV)], [outb], CdrNormParams(1e-5, 0, 0, 0))
    assert_close(outb.float(), torch.nn.functional.layer_norm(xb.float(), (512,)), BF16_TOL, "layer_norm bf16")
    ragged = torch.randn(4, 30, device=DEV)
    assert abi.launch(Template.LAYER_NORM, [ragged], [torch.empty_like(ragged)], CdrNormParams(1e-5, 0, 0, 0), check=False) == -2
    assert abi.launch(Template.LAYER_NORM, [dx, dw], [out], CdrNormParams(1e-5, 1, 1, 0), check=False) == -1   # bias missing


# ---------------------------------------------------------------- K4 GEMM + bias + ReLU
from conductor_b200.codegen.kernel_templates import CdrAttnParams, CdrGemmParams  # noqa: E402


def gemm(x, w, bias=None, relu=False):
    ins = [x, w] + ([bias] if bias is not None else [])
    out = torch.empty(*x.shape[:-1], w.shape[0], dtype=x.dtype, device=x.device)
    abi.launch(Template.GEMM_EPILOGUE, ins, [out], CdrGemmParams(1 if relu else 0, 1 if bias is not None else 0))
    return out


def test_mlp_golden(executor):
    g = load_golden("c4_mlp")
    x, w1, b1, w2, b2 = cuda(g["x"], g["w1"], g["b1"], g["w2"], g["b2"])
    h = gemm(x, w1, b1, relu=True)
    out = gemm(h, w2, b2)
    assert_close(out.float(), g["out"].float(), BF16_TOL, "mlp golden")


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (128, 256, 512), (1, 8, 8), (33, 40, 72), (200, 520, 136),
                                   (384, 768, 1024), (130, 257, 64), (1024, 1024, 4096)])
@pytest.mark.parametrize("relu", [False, True])
def test_gemm_shapes_against_oracle(executor, M, N, K, relu):
    gen = torch.Generator().manual_seed(M * 7 + N * 3 + K)
    x = torch.randn(M, K, generator=gen).bfloat16()
    w = (torch.randn(N, K, generator=gen) / K ** 0.5).bfloat16()
    b = torch.randn(N, generator=gen).bfloat16()
    if M * N * K <= 1 << 26:
        want = bf16_bits_to_tensor(scalar.linear_bf16(*(tensor_to_bf16_bits(t) for t in (x, w, b)), relu=relu)).float()
    else:                                     # the scalar oracle would take minutes: eager CPU instead
        want = torch.nn.functional.linear(x, w, b)
        want = (torch.relu(want) if relu else want).float()
    out = gemm(*cuda(x, w, b), relu=relu)
    assert_close(out.float(), want, BF16_TOL, f"gemm {M}x{N}x{K}")


@pytest.mark.parametrize("M,N,K,dtype", [(512, 768, 256, torch.bfloat16), (300, 520, 136, torch.bfloat16), (130, 257, 64, torch.float16),
                                         (1024, 1024, 512, torch.bfloat16)])
def test_gemm_with_gated_output(executor, M, N, K, dtype):
    """`gate_input`: out = (gate > 0) ? x @ W^T : 0 -- the backward of a ReLU fused into the product that
    makes its incoming gradient.  Vector path (whole 16-byte rows), scalar path (ragged N) and the special
    gate values: -0.0, +inf (positive), -inf, NaN (not positive)."""
    gen = torch.Generator().manual_seed(M + 3 * N + K)
    x = torch.randn(M, K, generator=gen).to(dtype)
    w = (torch.randn(N, K, generator=gen) / K ** 0.5).to(dtype)
    gate = torch.relu(torch.randn(M, N, generator=gen)).to(dtype)           # about half zeros, like a ReLU output
    gate[0, :6] = torch.tensor([-0.0, float("inf"), float("-inf"), float("nan"), 1e-30, -1.0]).to(dtype)
    want = torch.nn.functional.linear(x.float(), w.float()) * (gate.float() > 0)
    xd, wd, gd = cuda(x, w, gate)
    out = torch.full((M, N), float("nan"), dtype=dtype, device=DEV)
    abi.launch(Template.GEMM_EPILOGUE, [xd, wd, gd], [out], CdrGemmParams(0, 0, 0, 0, 1))
    assert_close(out.float(), want, BF16_TOL, f"gated gemm {M}x{N}x{K}")
    zeros_expected = ~(gate.float() > 0)
    assert bool((out.cpu()[zeros_expected] == 0).all())                      # exact zeros where the gate is closed
    # the gate must match the output's shape and dtype
    bad = torch.zeros(M, N + 1, dtype=dtype, device=DEV)
    assert abi.launch(Template.GEMM_EPILOGUE, [xd, wd, bad], [out], CdrGemmParams(0, 0, 0, 0, 1), check=False) == -1


def test_gemm_without_bias_fp16_and_3d_input(executor):
    gen = torch.Generator().manual_seed(77)
    x = torch.randn(4, 50, 96, generator=gen).half()
    w = (torch.randn(72, 96, generator=gen) / 10).half()
    out = gemm(*cuda(x, w))
    assert out.shape == (4, 50, 72)
    assert_close(out.float(), (x.float() @ w.float().T), BF16_TOL, "fp16 gemm")


@pytest.mark.parametrize("M,N,K,relu", [(128, 256, 64, False), (300, 520, 200, True), (1024, 1024, 512, False),
                                        (77, 72, 96, False), (2048, 256, 4096, True)])
def test_gemm_with_k_by_n_weights(executor, M, N, K, relu):
    """out = x @ W with W stored [K, N] (torch.matmul): the weight is read in place as an MN-major
    operand; same numbers as the [N, K] form on the transposed weight, and as the oracle."""
    gen = torch.Generator().manual_seed(M + N + K)
    x = torch.randn(M, K, generator=gen).bfloat16()
    w_kn = (torch.randn(K, N, generator=gen) / K ** 0.5).bfloat16()
    b = torch.randn(N, generator=gen).bfloat16()
    dx, dw, db = cuda(x, w_kn, b)
    out = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
    abi.launch(Template.GEMM_EPILOGUE, [dx, dw, db], [out], CdrGemmParams(1 if relu else 0, 1, 1, 0))
    same = gemm(dx, dw.t().contiguous(), db, relu=relu)
    assert bits_equal(out, same), "[K, N] and [N, K] forms differ"
    want = bf16_bits_to_tensor(scalar.linear_bf16(tensor_to_bf16_bits(x), tensor_to_bf16_bits(w_kn.t().contiguous()),
                                                  tensor_to_bf16_bits(b), relu=relu)).float()
    assert_close(out.float(), want, BF16_TOL, f"x @ W[K,N] {M}x{N}x{K}")
    # N not a multiple of 8 has no 16-byte row pitch in this layout
    bad = torch.randn(64, 12, device=DEV).bfloat16()
    assert abi.launch(Template.GEMM_EPILOGUE, [torch.randn(8, 64, device=DEV).bfloat16(), bad],
                      [torch.empty(8, 12, device=DEV, dtype=torch.bfloat16)], CdrGemmParams(0, 0, 1, 0), check=False) == -2


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (296, 520, 200), (1024, 512, 2048), (72, 80, 100)])
def test_gemm_with_transposed_x(executor, M, N, K):
    """x stored [K, M] (MN-major A operand), alone and together with [K, N] weights -- the form a
    weight gradient dW = dY^T @ x takes.  Bit-identical to the plain form on explicit transposes."""
    gen = torch.Generator().manual_seed(2 * M + N + K)
    x_km = torch.randn(K, M, generator=gen).bfloat16()
    w_nk = (torch.randn(N, K, generator=gen) / K ** 0.5).bfloat16()
    dx, dw = cuda(x_km, w_nk)
    plain = gemm(dx.t().contiguous(), dw) if K % 8 == 0 else None    # the plain form needs a 16-byte K pitch
    out = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
    if K % 8 == 0:
        abi.launch(Template.GEMM_EPILOGUE, [dx, dw], [out], CdrGemmParams(0, 0, 0, 1))
        assert bits_equal(out, plain), "[K, M] x with [N, K] weights"
    out2 = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
    abi.launch(Template.GEMM_EPILOGUE, [dx, dw.t().contiguous()], [out2], CdrGemmParams(0, 0, 1, 1))
    if K % 8 == 0:
        assert bits_equal(out2, plain), "[K, M] x with [K, N] weights"
    assert_close(out2.float(), x_km.float().t() @ w_nk.float().t(), BF16_TOL, "x^T @ W")


def test_gemm_rejects_what_it_cannot_run(executor):
    x = torch.randn(8, 12, device=DEV).bfloat16()         # K=12: row pitch not a multiple of 16 bytes
    w = torch.randn(8, 12, device=DEV).bfloat16()
    out = torch.empty(8, 8, device=DEV, dtype=torch.bfloat16)
    assert abi.launch(Template.GEMM_EPILOGUE, [x, w], [out], CdrGemmParams(0, 0), check=False) == -2
    xf = torch.randn(8, 16, device=DEV)
    assert abi.launch(Template.GEMM_EPILOGUE, [xf, xf], [torch.empty(8, 8, device=DEV)], CdrGemmParams(0, 0),
                      check=False) == -2


def test_full_size_mlp_through_backend(executor):
    import conductor  # noqa: F401

    mlp = rp.make_mlp()
    (x,) = rp.inputs_mlp()
    want = rp.run_reference(mlp, [x])
    torch._dynamo.reset()
    with torch.no_grad():
        out = torch.compile(mlp.to(DEV), backend="gcu")(x.to(DEV))
    assert_close(out.float(), want.float(), BF16_TOL, "full-size MLP")
    mlp.cpu()


# ---------------------------------------------------------------- K5 attention
def attention(q, k, v, causal, scale=None):
    out = torch.empty_like(q)
    scale = scale if scale is not None else q.shape[-1] ** -0.5
    p = CdrAttnParams(scale, 1 if causal else 0)
    # scratch: the counter the CTAs draw their tiles from.  Filled with garbage on purpose -- every
    # launch clears it itself
    ws = torch.full((abi.workspace_bytes(Template.ATTENTION, [q, k, v], [out], p),), 0xAB, dtype=torch.uint8, device=q.device)
    abi.launch(Template.ATTENTION, [q, k, v], [out], p, workspace=ws)
    return out


def test_attention_golden(executor):
    g = load_golden("c5_attention")
    out = attention(*cuda(g["q"], g["k"], g["v"]), causal=True)
    assert_close(out.float(), g["out"].float(), BF16_TOL, "attention golden")


@pytest.mark.parametrize("B,H,S,D,causal", [(1, 1, 128, 128, True), (1, 2, 256, 128, True), (2, 3, 384, 128, False),
                                            (1, 2, 200, 128, True), (1, 1, 77, 64, False), (2, 2, 512, 64, True),
                                            (1, 1, 1, 128, True), (1, 4, 1024, 128, True)])
def test_attention_shapes_against_oracle(executor, B, H, S, D, causal):
    q, k, v = rp.inputs_attention(B, H, S, D, seed=S + D)
    want = bf16_bits_to_tensor(scalar.attention_bf16(*(tensor_to_bf16_bits(t) for t in (q, k, v)), scale=D ** -0.5,
                                                     causal=causal)).float()
    ref = torch.nn.functional.scaled_dot_product_attention(q, k, v, is_causal=causal).float()
    assert_close(ref, want, BF16_TOL, "oracle vs eager")
    out = attention(*cuda(q, k, v), causal=causal)
    assert_close(out.float(), want, BF16_TOL, f"attention {B}x{H}x{S}x{D} causal={causal}")


@pytest.mark.parametrize("B,H,S,D,causal", [(3, 20, 600, 64, True), (2, 40, 520, 128, False), (1, 150, 300, 128, True)])
def test_attention_more_tiles_than_sms(executor, B, H, S, D, causal):
    """More (batch*head, query tile) pairs than the GPU has SMs: every persistent CTA walks several
    tiles, with ragged sequence lengths (partial key blocks, a last query tile with an empty half)."""
    q, k, v = rp.inputs_attention(B, H, S, D, seed=3 * S + D)
    ref = torch.nn.functional.scaled_dot_product_attention(q.float(), k.float(), v.float(), is_causal=causal)
    out = attention(*cuda(q, k, v), causal=causal)
    assert_close(out.float(), ref, BF16_TOL, f"attention {B}x{H}x{S}x{D} causal={causal}")
    # one head against the C oracle as well
    want = bf16_bits_to_tensor(scalar.attention_bf16(*(tensor_to_bf16_bits(t[:1, :1]) for t in (q, k, v)), scale=D ** -0.5,
                                                     causal=causal)).float()
    assert_close(out[:1, :1].float(), want, BF16_TOL, "first head vs oracle")


def test_attention_fp16_custom_scale_and_large_logits(executor):
    gen = torch.Generator().manual_seed(55)
    q = (4 * torch.randn(1, 2, 320, 64, generator=gen)).half()      # large logits: the running max keeps growing
    k = (4 * torch.randn(1, 2, 320, 64, generator=gen)).half()
    v = torch.randn(1, 2, 320, 64, generator=gen).half()
    want = scalar.attention_f32(q.float().numpy(), k.float().numpy(), v.float().numpy(), 0.3, causal=True)
    out = attention(*cuda(q, k, v), causal=True, scale=0.3)
    assert_close(out.float(), torch.from_numpy(want), BF16_TOL, "fp16 attention")


def test_attention_rejects_unsupported(executor):
    q = torch.randn(1, 1, 64, 96, device=DEV).bfloat16()            # head dim 96
    assert abi.launch(Template.ATTENTION, [q, q, q], [torch.empty_like(q)], CdrAttnParams(0.1, 0), check=False) == -2
    qf = torch.randn(1, 1, 64, 64, device=DEV)
    assert abi.launch(Template.ATTENTION, [qf, qf, qf], [torch.empty_like(qf)], CdrAttnParams(0.1, 0), check=False) == -2
    qb = torch.randn(1, 1, 64, 64, device=DEV).bfloat16()           # supported shape, but no scratch given
    assert abi.launch(Template.ATTENTION, [qb, qb, qb], [torch.empty_like(qb)], CdrAttnParams(0.1, 0), check=False) == -6


def test_attention_rescale_path_after_the_first_block(executor):
    """Scores that keep growing along the key axis: every later block's maximum exceeds the reference
    the softmax warps hold by far more than the 2^8 slack, so P is recomputed and the accumulator
    rescaled block after block (the path ordinary data takes only in a tile's first blocks)."""
    S, D = 640, 64
    gen = torch.Generator().manual_seed(77)
    q = torch.ones(1, 1, S, D).bfloat16()
    ramp = torch.arange(S, dtype=torch.float32).div(8).unsqueeze(-1)              # key i scores about i/8 * D * scale
    k = (ramp * torch.ones(1, 1, S, D) / D ** 0.5).bfloat16()
    v = torch.randn(1, 1, S, D, generator=gen).bfloat16()
    for causal in (True, False):
        want = scalar.attention_f32(q.float().numpy(), k.float().numpy(), v.float().numpy(), 1.0, causal=causal)
        out = attention(*cuda(q, k, v), causal=causal, scale=1.0)
        assert_close(out.float(), torch.from_numpy(want), BF16_TOL, f"growing scores causal={causal}")


def test_full_size_attention_through_backend(executor):
    import conductor  # noqa: F401

    q, k, v = rp.inputs_attention()
    want = rp.run_reference(rp.causal_attention, [q, k, v])
    torch._dynamo.reset()
    out = torch.compile(rp.causal_attention, backend="gcu")(*cuda(q, k, v))
    assert_close(out.float(), want.float(), BF16_TOL, "full-size causal attention")
    # rows are convex combinations of V rows: every output lies inside V's range
    assert out.float().abs().max().item() <= v.float().abs().max().item() + 1e-2
