"""Opt-in debug artifacts of a compiled graph.

Counterpart of ``DebugArtifactManager`` (reference: ``conductor/utils/artifacts.py:18-244``), which
saves the generated DSL, the host wrapper, the object file and the shared library of every kernel
under ``debug_dir`` next to the package -- at construction, whether asked or not.  Nothing is
generated per graph here except a kernel plan, so the artifacts are the things a developer reads
beside a profile: the FX graph, the DAG table with buffer scopes, the cluster list with the chosen
template and its parameters, the readable plan, and -- for clusters that run a run-time instance --
the CUDA source of that instance (``cdr_template_source``).  Nothing is written unless a directory
is given (``debug.dump_dir`` in the configuration or ``CONDUCTOR_DEBUG_DIR``).
"""
from __future__ import annotations

import ctypes
import json
import os
from pathlib import Path
from typing import Any, Optional

import torch

from .logging import get_logger

logger = get_logger(__name__)

_TEMPLATE_NAMES = {0: "alias", 1: "elementwise", 2: "row_reduce", 3: "softmax_fwd", 4: "softmax_bwd",
                   5: "gemm_epilogue", 6: "attention", 7: "full_reduce", 8: "layer_norm"}
_KINDS = ("fx", "dag", "clusters", "plan", "source")


def _struct_to_dict(obj: Any) -> Any:
    """ctypes parameter block -> plain JSON-able values (arrays trimmed to their used length)."""
    if obj is None:
        return None
    if isinstance(obj, ctypes.Array):
        return [_struct_to_dict(v) for v in obj]
    if isinstance(obj, ctypes.Structure):
        out = {}
        for name, _ in obj._fields_:
            out[name] = _struct_to_dict(getattr(obj, name))
        n_instr = out.get("n_instr")
        if isinstance(n_instr, int) and isinstance(out.get("instr"), list):
            out["instr"] = out["instr"][:n_instr]
        n_in = out.get("n_inputs")
        if isinstance(n_in, int) and isinstance(out.get("input_mode"), list):
            out["input_mode"] = out["input_mode"][:n_in]
        n_out = out.get("n_outputs")
        if isinstance(n_out, int) and isinstance(out.get("out_reg"), list):
            out["out_reg"] = out["out_reg"][:n_out]
        return out
    return obj


class DebugArtifactManager:
    """Files of one artifact directory, named ``<kernel>.<kind>.<ext>``."""

    def __init__(self, root: Optional[str] = None):
        self.root: Optional[Path] = Path(root) if root else None

    # ------------------------------------------------------------------ paths
    def enabled(self) -> bool:
        return self.root is not None

    def _path(self, kernel_name: str, kind: str, ext: str) -> Path:
        if self.root is None:
            raise RuntimeError("no artifact directory configured")
        self.root.mkdir(parents=True, exist_ok=True)
        return self.root / f"{kernel_name}.{kind}.{ext}"

    def get_fx_graph_path(self, kernel_name: str) -> Path:
        return self._path(kernel_name, "fx", "txt")

    def get_dag_path(self, kernel_name: str) -> Path:
        return self._path(kernel_name, "dag", "txt")

    def get_clusters_path(self, kernel_name: str) -> Path:
        return self._path(kernel_name, "clusters", "json")

    def get_plan_path(self, kernel_name: str) -> Path:
        """The readable plan takes the place of the reference's DSL source file
        (``artifacts.py:60-62 get_dsl_source_path``)."""
        return self._path(kernel_name, "plan", "txt")

    get_dsl_source_path = get_plan_path

    def get_instance_source_path(self, kernel_name: str, index: int) -> Path:
        return self._path(kernel_name, f"source{index}", "cu")

    # ------------------------------------------------------------------ writers
    def _write(self, path: Path, text: str) -> Path:
        path.write_text(text if text.endswith("\n") else text + "\n")
        logger.debug("wrote %s", path)
        return path

    def save_fx_graph(self, kernel_name: str, graph_module: torch.fx.GraphModule) -> Path:
        return self._write(self.get_fx_graph_path(kernel_name), str(graph_module.graph))

    def save_dag(self, kernel_name: str, dag_text: str) -> Path:
        return self._write(self.get_dag_path(kernel_name), dag_text)

    def save_plan(self, kernel_name: str, plan_text: str) -> Path:
        return self._write(self.get_plan_path(kernel_name), plan_text)

    save_dsl_source = save_plan

    def save_clusters(self, kernel_name: str, launches: list) -> Path:
        """Cluster list with the chosen template, operands and the parameter block."""
        rows = []
        for i, l in enumerate(launches):
            rows.append({
                "index": i,
                "template": _TEMPLATE_NAMES.get(l.template, str(l.template)),
                "template_id": l.template,
                "name": l.name,
                "cluster_type": getattr(getattr(l.cluster, "cluster_type", None), "value", None),
                "nodes": [n.op_name for n in getattr(l.cluster, "nodes", [])],
                "inputs": [{"name": b.name, "shape": list(b.shape or ()), "dtype": str(b.dtype), "scope": b.scope.value}
                           for b in l.inputs],
                "outputs": [{"name": b.name, "shape": list(s), "dtype": str(d), "scope": b.scope.value}
                            for b, s, d in zip(l.outputs, l.out_shapes, l.out_dtypes)],
                "alias_of": l.alias_of.name if l.alias_of is not None else None,
                "needs_workspace": l.needs_workspace,
                "params": _struct_to_dict(l.params),
            })
        return self._write(self.get_clusters_path(kernel_name), json.dumps(rows, indent=2))

    def save_instance_sources(self, kernel_name: str, launches: list) -> list[Path]:
        """CUDA source of the run-time instance of every elementwise / row-reduce launch that has
        one.  Needs the kernel library but no GPU; launches the library cannot describe are skipped."""
        try:
            from ..compiler.loader import load_library
            from ..codegen.kernel_templates import CdrTensor
            from .type_mapping import to_cdr_dtype

            lib = load_library()
        except Exception as exc:  # library not built: the other artifacts are still useful
            logger.debug("instance sources skipped: %s", exc)
            return []

        def describe(shapes_dtypes):
            arr = (CdrTensor * max(len(shapes_dtypes), 1))()
            for d, (shape, dtype) in zip(arr, shapes_dtypes):
                shape = tuple(shape or ())
                d.data = None
                d.dtype = to_cdr_dtype(dtype)
                d.rank = len(shape)
                stride = 1
                for k in range(len(shape) - 1, -1, -1):
                    d.shape[k] = shape[k]
                    d.stride[k] = stride
                    stride *= max(shape[k], 1)
            return arr

        written = []
        buf = ctypes.create_string_buffer(1 << 17)
        for i, l in enumerate(launches):
            if l.template not in (1, 2) or l.params is None:
                continue
            try:
                ins = describe([(b.shape, b.dtype) for b in l.inputs])
                outs = describe(list(zip(l.out_shapes, l.out_dtypes)))
                rc = lib.cdr_template_source(l.template, ins, len(l.inputs), outs, len(l.outputs),
                                             ctypes.cast(ctypes.byref(l.params), ctypes.c_void_p), ctypes.sizeof(l.params),
                                             buf, len(buf), 0)
            except Exception as exc:
                logger.debug("instance source of launch %d skipped: %s", i, exc)
                continue
            if rc == 0:
                written.append(self._write(self.get_instance_source_path(kernel_name, i), buf.value.decode()))
        return written

    def save_compilation(self, kernel_name: str, graph_module, dag_text: str, plan_text: str, launches: list) -> list[Path]:
        """Everything for one compiled graph."""
        paths = [self.save_fx_graph(kernel_name, graph_module), self.save_dag(kernel_name, dag_text),
                 self.save_clusters(kernel_name, launches), self.save_plan(kernel_name, plan_text)]
        return paths + self.save_instance_sources(kernel_name, launches)

    # ------------------------------------------------------------------ queries (reference: artifacts.py:168-237)
    def list_artifacts(self, kernel_name: Optional[str] = None) -> list:
        if self.root is None or not self.root.exists():
            return []
        pattern = f"{kernel_name}.*" if kernel_name else "*"
        return sorted(p for p in self.root.glob(pattern) if p.is_file())

    def clean_artifacts(self, kernel_name: Optional[str] = None) -> int:
        n = 0
        for p in self.list_artifacts(kernel_name):
            p.unlink()
            n += 1
        return n

    def get_artifact_summary(self, kernel_name: str) -> dict:
        files = self.list_artifacts(kernel_name)
        return {"kernel_name": kernel_name, "directory": str(self.root) if self.root else None,
                "files": {p.name: p.stat().st_size for p in files}, "total_bytes": sum(p.stat().st_size for p in files)}


_manager: Optional[DebugArtifactManager] = None


def get_debug_manager() -> DebugArtifactManager:
    """Manager for the configured directory (``CONDUCTOR_DEBUG_DIR`` wins over ``debug.dump_dir``);
    disabled -- and writing nothing -- when neither is set."""
    global _manager
    from .config import get_config

    root = os.environ.get("CONDUCTOR_DEBUG_DIR") or get_config().debug.dump_dir
    if _manager is None or (str(_manager.root) if _manager.root else None) != (str(Path(root)) if root else None):
        _manager = DebugArtifactManager(root)
    return _manager
