"""Pin the C oracle: known-answer cases of the reference's kernel programs and golden vectors
produced by running the reference package (tests/golden/make_golden.py)."""
import math

import numpy as np
import torch

from conftest import assert_close, bf16_bits_to_tensor, load_golden, tensor_to_bf16_bits
from oracle import reference_path as rp
from oracle import scalar


# ---- known answers the reference's .co test programs check themselves with ----------
def test_softmax_all_ones_gives_uniform():
    # choreo-op/softmax-gcu-only-test.co:80-81,98: ones[256,512] -> 1/512, tol 1e-6
    y = scalar.softmax_f32(np.ones((256, 512), np.float32))
    assert np.abs(y - 1.0 / 512).max() <= 1e-6
    y2 = scalar.softmax_f32(np.ones((256, 512), np.float32), online=True)
    assert np.abs(y2 - 1.0 / 512).max() <= 1e-6


def test_softmax_backward_known_answer():
    # choreo-op/softmaxbw-gcu-only-test.co:69-70,88: Y=0.5, dY=1 on [16,128]; the Jacobian sum is
    # 0.5*(1-0.5) + 127*(0.5*(0-0.5)) = -31.5, tol 1e-6
    y = np.full((16, 128), 0.5, np.float32)
    dy = np.ones((16, 128), np.float32)
    assert np.abs(scalar.softmax_backward_f32(y, dy, jacobian=True) + 31.5).max() <= 1e-6
    assert np.abs(scalar.softmax_backward_f32(y, dy) + 31.5).max() <= 1e-6


def test_addcdiv_all_ones():
    # choreo-op/addcdiv-dynamic.co:476-497: 1 + 1*(1/1) == 2 exactly
    one = np.ones(8192, np.float32)
    assert (scalar.addcdiv_f32(one, one, one) == 2.0).all()


def test_relu_exact():
    # choreo-op/activation-relu-fp32-templated-kernel.co:57,75-78: U(-1,1), exact equality
    x = np.random.default_rng(0).uniform(-1, 1, (128, 256)).astype(np.float32)
    assert (scalar.relu_f32(x) == np.where(x > 0, x, 0)).all()


def test_int_add_and_matmul_exact():
    # choreo-op/elemwise-gcu-only-test.co:36-54, matmul-gcu-only-test.co:44-63: U{-10..10}, exact
    rng = np.random.default_rng(1)
    a = rng.integers(-10, 11, (6, 17, 64), dtype=np.int32)
    b = rng.integers(-10, 11, (6, 17, 64), dtype=np.int32)
    assert (scalar.add_i32(a, b) == a + b).all()
    lhs = rng.integers(-10, 11, (128, 256), dtype=np.int32)
    rhs = rng.integers(-10, 11, (256, 256), dtype=np.int32)
    assert (scalar.matmul_i32(lhs, rhs) == lhs @ rhs).all()


def test_attention_matches_reference_formula_on_ramp():
    # choreo-op/attention-gcu-only-test.co:210-216: Q=K=V=i+j (scaled down here so exp stays
    # finite in float), non-causal, tol 1e-4 against softmax(QK^T/sqrt(d))V in torch double
    i = np.arange(32)[:, None]
    j = np.arange(64)[None, :]
    m = ((i + j) / 64.0).astype(np.float32)
    out = scalar.attention_f32(m, m, m, 1.0 / math.sqrt(64), causal=False)
    t = torch.from_numpy(m).double()
    ref = torch.softmax(t @ t.T / math.sqrt(64), -1) @ t
    assert np.abs(out - ref.numpy()).max() <= 1e-4


# ---- golden vectors from the reference's own execution ---------------------------
def test_golden_mul_add_bit_exact():
    g = load_golden("c1_mul_add")
    out = scalar.mul_add_f32(g["a"].numpy(), g["b"].numpy(), g["c"].numpy())
    assert (out.view(np.uint32) == g["out"].numpy().view(np.uint32)).all()


def test_golden_reduce_mean():
    g = load_golden("c2_reduce_mean")
    out = scalar.mean_relu_mul_add_bf16(*(tensor_to_bf16_bits(g[k]) for k in ("x", "w", "b")))
    assert_close(torch.from_numpy(out), g["out"], 1e-5, "reduce_mean")


def test_golden_softmax_forward_and_backward():
    g = load_golden("c3_softmax")
    y = scalar.softmax_f32(g["logits"].numpy())
    assert_close(torch.from_numpy(y), g["y"], 1e-5, "softmax fwd")
    y_online = scalar.softmax_f32(g["logits"].numpy(), online=True)
    assert_close(torch.from_numpy(y_online), g["y"], 1e-5, "online softmax fwd")
    for jac in (False, True):
        dx = scalar.softmax_backward_f32(g["y"].numpy(), g["grad"].numpy(), jacobian=jac)
        assert np.abs(dx - g["dx"].numpy()).max() <= 1e-5
        assert np.abs(dx - g["dx_written_out"].numpy()).max() <= 1e-5


def test_golden_mlp():
    g = load_golden("c4_mlp")
    h = scalar.linear_bf16(tensor_to_bf16_bits(g["x"]), tensor_to_bf16_bits(g["w1"]), tensor_to_bf16_bits(g["b1"]),
                           relu=True)
    out = scalar.linear_bf16(h, tensor_to_bf16_bits(g["w2"]), tensor_to_bf16_bits(g["b2"]))
    assert_close(bf16_bits_to_tensor(out).float(), g["out"].float(), 2e-2, "mlp")


def test_golden_attention():
    g = load_golden("c5_attention")
    out = scalar.attention_bf16(*(tensor_to_bf16_bits(g[k]) for k in ("q", "k", "v")),
                                scale=1.0 / math.sqrt(g["q"].shape[-1]), causal=True)
    assert_close(bf16_bits_to_tensor(out).float(), g["out"].float(), 2e-2, "attention")


# ---- the restated reference path equals plain eager ------------------------------
def test_reference_path_is_eager():
    a, b, c = rp.inputs_mul_add(8, 16, seed=7)
    out = rp.run_reference(rp.mul_add, [a, b, c])
    assert torch.equal(out, a * b + c)
    g = load_golden("c1_mul_add")
    assert torch.equal(rp.run_reference(rp.mul_add, [g["a"], g["b"], g["c"]]), g["out"])
    g2 = load_golden("c2_reduce_mean")
    assert torch.equal(rp.run_reference(rp.reduce_mean_fusion, [g2["x"], g2["w"], g2["b"]]), g2["out"])
