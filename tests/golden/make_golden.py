"""Generate tests/golden/*.npz by running the REFERENCE package itself.

Run in the build container, where the reference checkout is mounted read-only:

    python tests/golden/make_golden.py /path/to/reference

The reference is copied to a temporary directory first (its DebugArtifactManager creates
``debug_dir/`` next to the package on import, conductor/utils/artifacts.py:28-44), imported
from there in THIS process (so this script must not import the new ``conductor`` package),
and each of the five benchmark graphs is run at a small size through
``torch.compile(fn, backend='gcu')`` on CPU tensors -- the reference's own execution of the
graph (it falls back to eager: conductor/compiler/gcu_backend.py:70-89).  Inputs and outputs
are stored; bf16 tensors as uint16 bit patterns.
"""
from __future__ import annotations

import os
import shutil
import sys
import tempfile
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent


def bits(t):
    import torch

    if t.dtype == torch.bfloat16:
        return t.contiguous().view(torch.int16).numpy().view(np.uint16)
    return t.contiguous().numpy()


def main(ref_root: str) -> None:
    os.environ["PYTHONDONTWRITEBYTECODE"] = "1"
    os.environ["CONDUCTOR_LOG_LEVEL"] = "ERROR"
    os.environ["CONDUCTOR_DEBUG"] = "0"
    tmp = tempfile.mkdtemp(prefix="conductor_ref_")
    shutil.copytree(Path(ref_root) / "conductor", Path(tmp) / "conductor")
    sys.path.insert(0, tmp)
    sys.path.insert(1, str(HERE.parent.parent))  # for oracle.reference_path (graphs + inputs only)
    import logging

    logging.disable(logging.CRITICAL)
    import torch
    import conductor  # noqa: F401  -- the reference: registers 'gcu'

    assert Path(conductor.__file__).resolve().is_relative_to(Path(tmp).resolve()), conductor.__file__
    try:
        from conductor.utils.config import get_config

        get_config().debug.enabled = False
    except Exception:
        pass
    from oracle import reference_path as rp

    def run(fn, inputs):
        torch._dynamo.reset()
        with torch.no_grad():
            out = torch.compile(fn, backend="gcu")(*inputs)
        return out[0] if isinstance(out, (tuple, list)) else out

    cases = {}
    a, b, c = rp.inputs_mul_add(16, 64, seed=1)
    cases["c1_mul_add"] = dict(a=a, b=b, c=c, out=run(rp.mul_add, [a, b, c]))
    x, w, bb = rp.inputs_reduce_mean(32, 256, seed=2)
    cases["c2_reduce_mean"] = dict(x=x, w=w, b=bb, out=run(rp.reduce_mean_fusion, [x, w, bb]))
    logits, grad = rp.inputs_softmax(16, 512, seed=3)
    y = run(rp.softmax_forward, [logits])
    cases["c3_softmax"] = dict(logits=logits, grad=grad, y=y, dx=run(rp.softmax_backward, [grad, y]),
                               dx_written_out=run(rp.softmax_backward_written_out, [grad, y]))
    mlp = rp.make_mlp(64, 128, 64, seed=4)
    (xm,) = rp.inputs_mlp(32, 64, seed=4)
    cases["c4_mlp"] = dict(x=xm, w1=mlp[0].weight.detach(), b1=mlp[0].bias.detach(), w2=mlp[2].weight.detach(),
                           b2=mlp[2].bias.detach(), out=run(mlp, [xm]))
    q, k, v = rp.inputs_attention(1, 2, 96, 64, seed=5)
    cases["c5_attention"] = dict(q=q, k=k, v=v, out=run(rp.causal_attention, [q, k, v]))
    for name, tensors in cases.items():
        np.savez_compressed(HERE / f"{name}.npz", **{k: bits(t) for k, t in tensors.items()})
        print(name, {k: tuple(t.shape) for k, t in tensors.items()})
    shutil.rmtree(tmp, ignore_errors=True)


if __name__ == "__main__":
    if len(sys.argv) < 2 and "CONDUCTOR_REFERENCE_ROOT" not in os.environ:
        raise SystemExit("usage: make_golden.py <path to a checkout of the reference>")
    main(sys.argv[1] if len(sys.argv) > 1 else os.environ["CONDUCTOR_REFERENCE_ROOT"])
