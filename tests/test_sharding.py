"""Batch sharding: partition arithmetic, which inputs carry the batch, and the multi-process path
with a world of two `gloo` ranks on CPU (the shard runner is a CPU stand-in there; the kernels
themselves are covered by the GPU tests)."""
import os
import socket
import sys

import pytest
import torch
import torch.fx as fx
import torch.multiprocessing as mp

from conductor.optimization.graph_analyzer import GraphAnalyzer
from conductor_b200.compiler.sharding import ShardedCallable, batch_inputs, row_partition
from examples import workloads as wl


def test_row_partition():
    assert row_partition(16384, 8) == [(i * 2048, (i + 1) * 2048) for i in range(8)]
    assert row_partition(10, 4) == [(0, 3), (3, 6), (6, 9), (9, 10)]
    assert row_partition(2, 4) == [(0, 1), (1, 2), (2, 2), (2, 2)]
    assert row_partition(0, 2) == [(0, 0), (0, 0)]
    parts = row_partition(8, 8)
    assert all(e - s == 1 for s, e in parts)          # config 5 at 8 GPUs: one sequence each
    with pytest.raises(ValueError):
        row_partition(4, 0)


def dag_of(fn, inputs):
    box = {}

    def backend(gm, ex):
        box["dag"] = GraphAnalyzer().parse_fx_graph(gm, ex)
        return gm.forward

    torch._dynamo.reset()
    with torch.no_grad():
        torch.compile(fn, backend=backend)(*inputs)
    torch._dynamo.reset()
    return box["dag"]


def test_batch_inputs_of_the_benchmark_graphs():
    dag = dag_of(wl.mul_add, wl.inputs_mul_add(8, 8))          # square: w-like vectors must not be picked by size
    assert batch_inputs(dag) == (8, [0, 1, 2])
    dag = dag_of(wl.reduce_mean_fusion, wl.inputs_reduce_mean(64, 64))
    assert batch_inputs(dag) == (64, [0])                        # w, b are [64] too, but row-broadcast
    dag = dag_of(wl.softmax_forward, wl.inputs_softmax(8, 32)[:1])
    assert batch_inputs(dag) == (8, [0])
    dag = dag_of(wl.make_mlp(32, 32, 32), wl.inputs_mlp(32, 32))
    batch, idx = batch_inputs(dag)
    assert batch == 32 and [dag.inputs[i].name for i in idx] == ["l_args_0_"]
    dag = dag_of(wl.causal_attention, wl.inputs_attention(4, 2, 16, 32))
    assert batch_inputs(dag) == (4, [0, 1, 2])


def test_single_process_form_splits_and_reassembles():
    x, w, b = wl.inputs_reduce_mean(10, 64, seed=3)
    seen = []

    def run_shard(inputs, device_index):
        seen.append((device_index, inputs[0].shape[0]))
        return (wl.reduce_mean_fusion(*inputs),)

    sc = ShardedCallable(run_shard, 10, [0], devices=[0, 1, 2, 3])
    (out,) = sc(x, w, b)
    assert seen == [(0, 3), (1, 3), (2, 3), (3, 1)]
    assert torch.equal(out, wl.reduce_mean_fusion(x, w, b))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out_q):
    import torch.distributed as dist

    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from conductor_b200.compiler.sharding import ShardedCallable
        from examples import workloads

        x, w, b = workloads.inputs_reduce_mean(11, 64, seed=5)            # 11 rows over 2 ranks: 6 + 5
        rows = []

        def run_shard(inputs, r):
            rows.append(inputs[0].shape[0])
            return (workloads.reduce_mean_fusion(*inputs),)

        sc = ShardedCallable(run_shard, 11, [0], rank=rank, world_size=world, gather_outputs=True)
        (full,) = sc(x, w, b)
        local_only = ShardedCallable(run_shard, 11, [0], rank=rank, world_size=world, gather_outputs=False)(x, w, b)
        want = workloads.reduce_mean_fusion(x, w, b)
        out_q.put((rank, rows[0], bool(torch.equal(full, want)), tuple(local_only[0].shape)))
    finally:
        dist.destroy_process_group()


def test_two_gloo_ranks_shard_and_gather():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = sorted(q.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert results == [(0, 6, True, (6,)), (1, 5, True, (5,))]


def _worker_small_batch(rank, world, port, out_q):
    import torch.distributed as dist

    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from conductor_b200.compiler.sharding import ShardedCallable
        from examples import workloads

        x, w, b = workloads.inputs_reduce_mean(1, 64, seed=8)             # one row over two ranks: rank 1 has none
        ran = []

        def run_shard(inputs, r):
            ran.append(inputs[0].shape[0])
            return (workloads.reduce_mean_fusion(*inputs),)

        sc = ShardedCallable(run_shard, 1, [0], rank=rank, world_size=world, gather_outputs=True,
                             output_spec=[((1,), torch.float32)])
        (full,) = sc(x, w, b)
        even = ShardedCallable(run_shard, 4, [0], rank=rank, world_size=world, gather_outputs=True)
        x4 = workloads.inputs_reduce_mean(4, 64, seed=9)[0]
        (full4,) = even(x4, w, b)                                           # equal blocks: gathered in place
        out_q.put((rank, ran, bool(torch.equal(full, workloads.reduce_mean_fusion(x, w, b))),
                   bool(torch.equal(full4, workloads.reduce_mean_fusion(x4, w, b)))))
    finally:
        dist.destroy_process_group()


def test_rank_without_rows_still_joins_the_gather():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker_small_batch, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = sorted(q.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert results == [(0, [1, 2], True, True), (1, [2], True, True)]


def test_rank_without_rows_and_unknown_outputs_is_refused_before_any_collective():
    for rank in (0, 1):           # the rank that does have rows must refuse too, or it would wait alone
        sc = ShardedCallable(lambda inputs, r: (inputs[0],), 1, [0], rank=rank, world_size=2, gather_outputs=True)
        with pytest.raises(Exception, match="no rows"):
            sc(torch.zeros(1, 4))


@pytest.mark.gpu
def test_shard_polymorphic_plan_on_gpu():
    """A plan compiled for the full batch runs on a block of its rows (what every rank does)."""
    import conductor  # noqa: F401
    from conductor_b200.compiler.callable import Callable
    from conductor_b200.compiler.gcu_backend import get_gcu_backend

    x, w, b = wl.inputs_reduce_mean(64, 4096, seed=6)
    torch._dynamo.reset()
    f = torch.compile(wl.reduce_mean_fusion, backend="gcu")
    full = f(x.cuda(), w.cuda(), b.cuda())
    plan = list(get_gcu_backend()._compiled_functions.values())[-1]
    shard_plan = Callable(plan.artifact, batch_size=64)
    (part,) = shard_plan(x[16:40].cuda(), w.cuda(), b.cuda())
    assert part.shape == (24,) and torch.equal(part, full[16:40])
    sc = ShardedCallable.from_artifact(plan.artifact, n_devices=1)
    (again,) = sc(x.cuda(), w.cuda(), b.cuda())
    assert torch.equal(again, full)


# ---------------------------------------------------------------- row chunks of host-tensor calls (decision logic, CPU)
def _callable_for(fn, inputs):
    import conductor  # noqa: F401
    from conductor_b200.compiler.callable import Callable
    from conductor_b200.compiler.jit_compiler import ChoreoJITCompiler

    box = {}

    def backend(gm, ex):
        box["plan"] = Callable(ChoreoJITCompiler().compile_graph(gm, ex), gm)
        return gm.forward

    torch._dynamo.reset()
    with torch.no_grad():
        torch.compile(fn, backend=backend)(*inputs)
    torch._dynamo.reset()
    return box["plan"]


def test_host_calls_are_cut_into_row_chunks_only_for_row_parallel_plans():
    from conductor_b200.utils.config import get_config

    cfg = get_config().runtime
    old = (cfg.host_chunk_bytes, cfg.host_max_chunks)
    try:
        cfg.host_chunk_bytes, cfg.host_max_chunks = 1 << 20, 8
        a, b, c = wl.inputs_mul_add(1000, 512, seed=1)                     # 3 x 2,048,000 bytes of batch inputs: five chunks of at least 1 MiB
        plan = _callable_for(wl.mul_add, [a, b, c])
        chunks = plan._host_chunks([a, b, c])
        assert chunks is not None and chunks[0][0] == 0 and chunks[-1][1] == 1000 and len(chunks) == 5
        assert all(e0 == s1 for (_, e0), (s1, _) in zip(chunks, chunks[1:]))   # contiguous, no gaps
        assert plan._host_chunks([t[:4].contiguous() for t in (a, b, c)]) is None   # another batch size: one piece
        cfg.host_chunk_bytes = 0
        assert plan._host_chunks([a, b, c]) is None                           # switched off
        cfg.host_chunk_bytes = 1 << 20
        small = wl.inputs_mul_add(16, 64, seed=2)
        assert _callable_for(wl.mul_add, small)._host_chunks(small) is None     # too small to be worth it
        # a layout change ties the plan to the full shapes
        x = torch.randn(1024, 512)
        assert _callable_for(lambda t: t.t().contiguous() + 1.0, [x])._host_chunks([x]) is None
        # a reduction over the rows is not row-parallel
        assert _callable_for(lambda t: t.sum(), [x])._host_chunks([x]) is None
        # a product whose right operand has as many rows as the batch: the weight must stay whole
        y = torch.randn(1024, 512)
        p2 = _callable_for(lambda u, v: torch.nn.functional.linear(u, v), [x.bfloat16(), y.bfloat16()])
        assert p2._host_chunks([x.bfloat16(), y.bfloat16()]) is None or p2._chunk_plan[1] == [0]
        # row softmax and the mean-fusion graph are
        lg = wl.inputs_softmax(2048, 512, seed=3)[:1]
        assert _callable_for(wl.softmax_forward, lg)._host_chunks(lg) is not None
    finally:
        cfg.host_chunk_bytes, cfg.host_max_chunks = old
