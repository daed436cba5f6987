"""Config, compile cache, debug dump and exception surface (CPU only)."""
import json

import pytest
import torch
import torch.fx as fx

from conductor.compiler.jit_compiler import ChoreoJITCompiler
from conductor.utils.cache import CompilationCache
from conductor.utils.config import ConductorConfig, get_config, reset_config, set_config
from conductor.utils.exceptions import (CompilationError, ConductorError, DeviceError, ExecutionError,
                                        UnsupportedOperationError)


def traced(fn=lambda a, b, c: a * b + c):
    return fx.symbolic_trace(fn)


def test_config_defaults_env_and_file(monkeypatch, tmp_path):
    cfg = ConductorConfig.load()
    assert not cfg.debug.enabled and cfg.cache.enabled and cfg.compilation.enable_fusion
    assert cfg.runtime.device == "gcu" and cfg.runtime.devices == 1 and cfg.logging.level == "WARNING"
    monkeypatch.setenv("CONDUCTOR_DEBUG", "1")
    monkeypatch.setenv("CONDUCTOR_DISABLE_CACHE", "true")
    monkeypatch.setenv("CONDUCTOR_LOG_LEVEL", "info")
    monkeypatch.setenv("CONDUCTOR_DEVICES", "4")
    cfg = ConductorConfig.load()
    assert cfg.debug.enabled and not cfg.cache.enabled and cfg.logging.level == "INFO" and cfg.runtime.devices == 4
    for k in ("CONDUCTOR_DEBUG", "CONDUCTOR_DISABLE_CACHE", "CONDUCTOR_LOG_LEVEL", "CONDUCTOR_DEVICES"):
        monkeypatch.delenv(k)
    path = tmp_path / "conductor_config.json"
    path.write_text(json.dumps({"compilation": {"enable_fusion": False, "unknown_key": 1}, "cache": {"max_size_mb": 7}}))
    cfg = ConductorConfig.load(str(path))
    assert not cfg.compilation.enable_fusion and cfg.cache.max_size_mb == 7
    assert cfg.to_dict()["compilation"]["timeout_seconds"] == 300


def test_compilation_cache_lru():
    c = CompilationCache(max_entries=2)
    c.put("a", 1)
    c.put("b", 2)
    assert c.get("a") == 1                      # touch a: b becomes the eviction candidate
    c.put("c", 3)
    assert c.get("b") is None and c.get("a") == 1 and c.get("c") == 3 and len(c) == 2
    st = c.get_stats()
    assert st["hits"] == 3 and st["misses"] == 1 and st["evictions"] == 1
    off = CompilationCache(enabled=False)
    off.put("x", 1)
    assert off.get("x") is None and "x" not in off


def test_compile_cache_hits_and_key_covers_dtype():
    comp = ChoreoJITCompiler()
    gm = traced()
    f32 = [torch.randn(4, 4)] * 3
    a1 = comp.compile_graph(gm, f32)
    a2 = comp.compile_graph(gm, f32)
    assert a1 is a2 and comp.stats["cache_hits"] == 1 and comp.stats["compiled"] == 1
    bf16 = [t.bfloat16() for t in f32]
    a3 = comp.compile_graph(traced(), bf16)
    assert a3 is not a1 and a3.launches[0].params.instr[0].round_to == 1          # rounds to bf16
    assert comp._generate_graph_hash(gm, f32) != comp._generate_graph_hash(gm, bf16)
    assert comp._generate_graph_hash(gm, f32) != comp._generate_graph_hash(gm, [torch.randn(4, 8)] * 3)
    comp.clear_cache()
    assert comp.compile_graph(gm, f32) is not a1


def test_debug_dump_is_opt_in(tmp_path):
    """Artifacts and trace (reference: utils/artifacts.py, utils/tracer.py): nothing is written or
    traced by default; with a directory set, one compile leaves the FX graph, the DAG table, the
    cluster list with template parameters and the plan."""
    import json

    from conductor_b200.utils.artifacts import get_debug_manager
    from conductor_b200.utils.tracer import get_tracer, reset_tracer

    assert not get_debug_manager().enabled() and not get_tracer().is_enabled()
    cfg = ConductorConfig.load()
    cfg.debug.enabled = True
    cfg.debug.dump_dir = str(tmp_path / "dump")
    set_config(cfg)
    reset_tracer()
    try:
        art = ChoreoJITCompiler().compile_graph(traced(), [torch.randn(4, 4)] * 3)
        mgr = get_debug_manager()
        names = {p.name for p in mgr.list_artifacts(art.entry_point)}
        for kind in ("fx.txt", "dag.txt", "clusters.json", "plan.txt"):
            assert f"{art.entry_point}.{kind}" in names, names
        assert "elementwise<elementwise[mul,add]>" in mgr.get_plan_path(art.entry_point).read_text()
        assert "buffers:" in mgr.get_dag_path(art.entry_point).read_text()
        clusters = json.loads(mgr.get_clusters_path(art.entry_point).read_text())
        assert clusters[0]["template"] == "elementwise" and clusters[0]["nodes"] == ["mul", "add"]
        assert [i["op"] for i in clusters[0]["params"]["instr"]] == [3, 1]           # MUL then ADD
        assert len(clusters[0]["params"]["input_mode"]) == 3
        kinds = [r["kind"] for r in get_tracer().records]
        assert {"cache", "hash", "dag", "plan", "compilation"} <= set(kinds)
        assert mgr.get_artifact_summary(art.entry_point)["total_bytes"] > 0
        assert mgr.clean_artifacts(art.entry_point) == len(names) and not mgr.list_artifacts()
    finally:
        reset_config()
        reset_tracer()
    assert not get_config().debug.enabled and not get_debug_manager().enabled()


def test_artifact_metadata():
    art = ChoreoJITCompiler().compile_graph(traced(), [torch.randn(4, 4)] * 3)
    assert art.artifact_type == "kernel_plan" and art.entry_point.startswith("kernel_") and art.is_valid()
    assert art.metadata["n_clusters"] == 1 and art.metadata["n_nodes"] == 2
    assert art.path.endswith("libconductor_b200.so")
    assert "plan kernel_" in art.metadata["plan"]


def test_exception_hierarchy_and_fields():
    assert issubclass(CompilationError, ConductorError) and issubclass(DeviceError, ConductorError)
    e = UnsupportedOperationError("cumsum", "no template")
    assert e.operation == "cumsum" and "cumsum" in str(e) and "no template" in str(e)
    x = ExecutionError("boom", kernel_name="k", status=-5)
    assert x.status == -5 and x.kernel_name == "k" and "status=-5" in str(x)
    c = CompilationError("bad", dsl_code="plan", compiler_output="line1\nerror: x\n")
    assert c.get_compiler_errors() == ["error: x"]


def test_validation_failure_is_a_compilation_error():
    comp = ChoreoJITCompiler()
    with pytest.raises((CompilationError, ValueError)):
        comp.compile_graph(traced(), [torch.randn(4, 4)])            # wrong number of example inputs


def test_cache_key_covers_the_constants_a_plan_captures():
    """Two structurally identical modules (same graph text, same target names) hold different
    weights: the plan captures the weights by reference, so they must not share a cache entry."""
    import torch.nn as nn

    from conductor.compiler.gcu_backend import GCUBackend

    class Net(nn.Module):
        def __init__(self):
            super().__init__()
            self.fc = nn.Linear(16, 16)

        def forward(self, x):
            return self.fc(x)

    g1, g2 = fx.symbolic_trace(Net()), fx.symbolic_trace(Net())
    assert str(g1.graph) == str(g2.graph)
    x = [torch.randn(4, 16)]
    comp = ChoreoJITCompiler()
    assert comp._generate_graph_hash(g1, x) != comp._generate_graph_hash(g2, x)
    assert comp._generate_graph_hash(g1, x) == comp._generate_graph_hash(g1, x)
    be = GCUBackend()
    assert be._compute_graph_hash(g1, x) != be._compute_graph_hash(g2, x)
    a1, a2 = comp.compile_graph(g1, x), comp.compile_graph(g2, x)
    assert a1 is not a2
    w1 = [b.constant_value for b in a1.dag.buffers if getattr(b, "constant_value", None) is not None]
    w2 = [b.constant_value for b in a2.dag.buffers if getattr(b, "constant_value", None) is not None]
    assert w1 and w2 and w1[0] is not w2[0]


def test_scratch_lane_of_the_executor_is_per_thread():
    """Runs recorded on different branches of one CUDA graph are bound under different lanes (their
    scratch buffers must not be shared); the lane is state of the recording thread only."""
    import threading

    from conductor_b200.compiler.executor import get_executor

    ex = get_executor()
    assert ex.workspace_lane == 0
    ex.workspace_lane = 2
    seen = []
    t = threading.Thread(target=lambda: seen.append(ex.workspace_lane))
    t.start()
    t.join()
    try:
        assert seen == [0] and ex.workspace_lane == 2
    finally:
        ex.workspace_lane = 0


def test_reference_arm_of_the_bench_prints_the_contract_line():
    """`bench.py --impl reference` runs the reference's CPU path and prints one JSON line with the keys
    the measurement contract names (here on the smallest configuration, two steps)."""
    import json
    import os
    import subprocess
    import sys

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    run = subprocess.run([sys.executable, os.path.join(root, "bench.py"), "--impl", "reference", "--workload", "c1",
                          "--steps", "2", "--warmup", "1"], capture_output=True, text=True, timeout=600, cwd=root)
    assert run.returncode == 0, run.stderr[-2000:]
    line = json.loads(run.stdout.strip().splitlines()[-1])
    for key in ("metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling",
                "vs_baseline", "dtype", "data", "config", "impl", "cpu_baseline", "e2e"):
        assert key in line, key
    assert line["impl"] == "reference" and line["unit"] == "samples/s" and line["higher_is_better"] is True
    assert line["cpu_baseline"]["kind"] in ("reference", "port") and line["cpu_baseline"]["cores"] >= 1
    assert line["e2e"]["h2d_bytes_per_step"] == 0 and line["e2e"]["d2h_bytes_per_step"] == 0
    assert line["config"]["workload"].startswith("c1 ") and line["value"] > 0
