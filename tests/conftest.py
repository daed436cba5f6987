"""Shared pytest setup.

Markers: ``gpu`` -- needs a CUDA device (the parity tests proper; they call the kernels
through the C ABI).  Everything else runs on CPU: the oracle against golden vectors, the
FX->DAG analysis and clustering, and the ABI surface of the built library.
"""
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

GOLDEN = Path(__file__).resolve().parent / "golden"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: test needs a CUDA device")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def bf16_bits_to_tensor(a: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(a.view(np.int16).copy()).view(torch.bfloat16)


def tensor_to_bf16_bits(t: torch.Tensor) -> np.ndarray:
    return t.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16)


def load_golden(name: str) -> dict:
    """Golden case as torch tensors; uint16 arrays are bf16 bit patterns."""
    data = np.load(GOLDEN / f"{name}.npz")
    out = {}
    for k in data.files:
        a = data[k]
        out[k] = bf16_bits_to_tensor(a) if a.dtype == np.uint16 else torch.from_numpy(a.copy())
    return out


@pytest.fixture(scope="session")
def built_library():
    """Path of libconductor_b200.so, building it when the tree has none."""
    from conductor_b200.csrc.build import LIB_PATH, build

    if not LIB_PATH.exists():
        build()
    return LIB_PATH


@pytest.fixture(scope="session")
def executor(built_library):
    from conductor_b200.compiler.executor import get_executor

    return get_executor()


def max_abs_rel(actual: torch.Tensor, expected: torch.Tensor):
    a, e = actual.detach().double().cpu(), expected.detach().double().cpu()
    diff = (a - e).abs()
    max_abs = diff.max().item() if diff.numel() else 0.0
    denom = e.abs().clamp_min(1e-30)
    max_rel = (diff / denom).max().item() if diff.numel() else 0.0
    return max_abs, max_rel


def assert_close(actual, expected, tol, what=""):
    """The acceptance rule of the benchmark spec: every element within `tol` in absolute OR
    relative terms (max-abs/rel error <= 1e-5 for fp32, <= 2e-2 for bf16)."""
    a, e = actual.detach().double().cpu(), expected.detach().double().cpu()
    assert a.shape == e.shape, f"{what}: shape {tuple(a.shape)} vs {tuple(e.shape)}"
    nan_mismatch = torch.isnan(a) != torch.isnan(e)
    assert not nan_mismatch.any(), f"{what}: NaN pattern differs"
    mask = ~torch.isnan(e)
    diff = (a[mask] - e[mask]).abs()
    ok = (a[mask] == e[mask]) | (diff <= tol) | (diff <= tol * e[mask].abs())
    if not ok.all():
        bad = (~ok).nonzero()
        i = bad[0].item()
        raise AssertionError(
            f"{what}: {int((~ok).sum())} of {ok.numel()} elements outside tol={tol}; "
            f"first: got {a[mask][i].item()!r}, want {e[mask][i].item()!r}; max abs {diff[~torch.isnan(diff)].max().item():.3e}")
