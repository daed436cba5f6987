"""The allocation-free full reduction, `cdr_full_reduce_noalloc`.

Some callers of this library may not allocate device memory while they run: a serving process or
a framework memory pool that took all of HBM at start-up, or a latency-critical loop that cannot
tolerate the device-wide synchronisation of an allocation.  For them the library offers a variant
of the full reduction whose scratch lives in a fixed array inside the library instead of in a
workspace the caller would have to allocate.  This test calls that variant through the C ABI, twice
in a row (every call shares the one array, so the second call runs on whatever the first left
behind), and compares each result with the ordinary workspace-taking entry point and with a
double-precision sum computed on the host (the two entry points may run different kernels: the
allocation-free one never compiles or loads a run-time instance, because that would allocate).

The file name sorts last on purpose: a run that stops at the first failure has already run every
other test."""
import ctypes

import pytest
import torch

import abi_util as abi
from conductor_b200.codegen.kernel_templates import CdrReduceParams
from conductor_b200.codegen.operator_registry import EwOp, ReduceOp, Template
from conductor_b200.compiler.executor import make_descriptors
from conductor_b200.compiler.loader import load_library

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
F32_TOL = 1e-5


def params(chain, op):
    p = CdrReduceParams()
    p.chain = chain
    p.reduce_op = op
    return p


def noalloc(inputs, out, p):
    lib = load_library()
    ind, outd = make_descriptors(inputs), make_descriptors([out])
    stream = torch.cuda.current_stream(out.device).cuda_stream
    with torch.cuda.device(out.device):
        rc = lib.cdr_full_reduce_noalloc(ind, len(inputs), outd, 1, ctypes.cast(ctypes.byref(p), ctypes.c_void_p),
                                         ctypes.sizeof(p), stream)
    return rc, lib.cdr_last_error().decode()


def with_workspace(inputs, out, p):
    n = abi.workspace_bytes(Template.FULL_REDUCE, inputs, [out], p)
    ws = torch.empty(n, dtype=torch.uint8, device=out.device)
    abi.launch(Template.FULL_REDUCE, inputs, [out], p, workspace=ws)


def test_noalloc_matches_workspace_entry_point_twice_in_a_row():
    gen = torch.Generator().manual_seed(91)
    x1 = torch.randn(777, 1031, generator=gen).to(DEV)
    x2 = (torch.randn(64, 50, generator=gen) * 3).to(DEV)          # different size: fewer CTAs, stale partials
    sum_sq = params(abi.ew_program(1, [(EwOp.MUL, 0, 0, 0, 0, torch.float32)], [1]), ReduceOp.SUM)
    mean = params(abi.ew_program(1, [], [0]), ReduceOp.MEAN)
    exact = {id(sum_sq): lambda t: (t.double() ** 2).sum().item(), id(mean): lambda t: t.double().mean().item()}
    for x, p in ((x1, sum_sq), (x2, mean), (x1, mean)):
        want = torch.empty((), device=DEV)
        with_workspace([x], want, p)
        got = torch.full((), float("nan"), device=DEV)
        rc, msg = noalloc([x], got, p)
        assert rc == 0, msg
        torch.cuda.synchronize()
        w, g = want.item(), got.item()
        assert abs(g - w) <= F32_TOL * max(1.0, abs(w)), (g, w)
        host = exact[id(p)](x.cpu())
        assert abs(g - host) <= F32_TOL * max(1.0, abs(host)), (g, host)


def test_noalloc_leaves_the_device_allocation_untouched():
    """The call must not allocate: the driver's free-memory figure is the same before and after
    calls on a program and a shape this process has not run before (the ordinary entry point would
    compile and load a run-time kernel instance for it)."""
    x = torch.randn(512, 264, device=DEV)                    # vector-shaped: the ordinary path would specialise it
    p = params(abi.ew_program(1, [(EwOp.ABS, 0, 0, 0, 0, torch.float32)], [1]), ReduceOp.SUM)
    got = torch.empty((), device=DEV)
    rc, msg = noalloc([x], got, p)                            # first call on the device resolves the array's address
    assert rc == 0, msg
    torch.cuda.synchronize()
    q = params(abi.ew_program(1, [(EwOp.NEG, 0, 0, 0, 0, torch.float32), (EwOp.ABS, 1, 0, 0, 0, torch.float32)], [2]),
               ReduceOp.SUM)
    free_before, _ = torch.cuda.mem_get_info()
    for _ in range(2):
        rc, msg = noalloc([x], got, q)
        assert rc == 0, msg
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before
    host = x.cpu().double().abs().sum().item()
    assert abs(got.item() - host) <= F32_TOL * max(1.0, abs(host))


def test_noalloc_runs_inside_a_stream_capture_on_a_program_it_has_not_seen():
    """A caller that records its step in a CUDA graph may not compile, load a module or allocate while
    the capture is open.  After one call on the device (which resolves the scratch array's address)
    a program this process has never run is launched inside a capture and replayed twice."""
    x = torch.randn(300, 520, device=DEV)
    got = torch.full((), float("nan"), device=DEV)
    warm = params(abi.ew_program(1, [], [0]), ReduceOp.SUM)
    rc, msg = noalloc([x], got, warm)
    assert rc == 0, msg
    torch.cuda.synchronize()
    fresh = params(abi.ew_program(1, [(EwOp.SIGMOID, 0, 0, 0, 0, torch.float32), (EwOp.MUL, 1, 0, 0, 0, torch.float32)], [2]),
                   ReduceOp.SUM)                                # sum(x * sigmoid(x)): a chain no other test reduces
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            rc, msg = noalloc([x], got, fresh)
    torch.cuda.current_stream().wait_stream(side)
    assert rc == 0, msg
    host = (x.cpu().double() * torch.sigmoid(x.cpu().double())).sum().item()
    for _ in range(2):
        got.fill_(float("nan"))
        graph.replay()
        torch.cuda.synchronize()
        assert abs(got.item() - host) <= 1e-4 * max(1.0, abs(host)), (got.item(), host)


def test_noalloc_reports_bad_arguments():
    x = torch.randn(8, 8, device=DEV)
    out = torch.empty((), device=DEV)
    p = params(abi.ew_program(1, [], [0]), ReduceOp.SUM)
    lib = load_library()
    ind, outd = make_descriptors([x]), make_descriptors([out])
    rc = lib.cdr_full_reduce_noalloc(ind, 1, outd, 1, None, 0, None)
    assert rc == -1 and b"cdr_reduce_params" in lib.cdr_last_error()
    bad_out = torch.empty(2, device=DEV)
    rc, msg = noalloc([x], bad_out, p)
    assert rc == -1 and "one element" in msg
