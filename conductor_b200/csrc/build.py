"""Build libconductor_b200.so in-tree with nvcc for sm_100a.

Replaces the reference's per-graph compile-and-link step
(conductor/compiler/jit_compiler.py:260-343 runs `choreo -c -fpic` then `gcc -shared`;
conductor/compiler/host_wrapper.py:270-295 runs `g++ -shared` on the generated wrapper)
with one ahead-of-time build of the fixed kernel-template library.

Usage: python -m conductor_b200.csrc.build [--force] [--verbose]
"""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

CSRC = Path(__file__).resolve().parent
LIB_NAME = "libconductor_b200.so"
LIB_PATH = CSRC / LIB_NAME

# file -> extra flags.  The elementwise and reduction templates must not contract
# a*b+c into an fma: eager rounds the product and the sum separately.
SOURCES = {
    "cdr_api.cu": [],
    "cdr_elementwise.cu": ["--fmad=false"],
    "cdr_jit.cu": [],
    "cdr_reduce.cu": ["--fmad=false"],
    "cdr_softmax.cu": ["--fmad=false"],
    "cdr_layernorm.cu": [],
    "cdr_copy.cu": [],
    "cdr_gemm.cu": [],
    "cdr_attention.cu": [],
}

COMMON = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "-Xcompiler", "-fvisibility=hidden",
]


def _nvcc() -> str:
    cand = os.environ.get("NVCC") or "/usr/local/cuda/bin/nvcc"
    return cand if os.path.exists(cand) else "nvcc"


def _deps_mtime() -> float:
    paths = list(CSRC.glob("*.cuh")) + [CSRC.parent.parent / "include" / "conductor_b200.h"]
    return max(p.stat().st_mtime for p in paths if p.exists())


def _compile(src: str, flags: list[str], verbose: bool) -> Path:
    obj = CSRC / (Path(src).stem + ".o")
    cmd = [_nvcc(), *COMMON, *flags, "-c", str(CSRC / src), "-o", str(obj)]
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src}:\n{res.stdout}\n{res.stderr}")
    if verbose:
        sys.stderr.write(res.stderr)
    return obj


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile every kernel template and link the shared library; returns its path."""
    dep_time = _deps_mtime()
    todo = []
    for src, flags in SOURCES.items():
        obj = CSRC / (Path(src).stem + ".o")
        src_time = max((CSRC / src).stat().st_mtime, dep_time)
        if force or verbose or not obj.exists() or obj.stat().st_mtime < src_time:
            todo.append((src, flags))
    if todo:
        with ThreadPoolExecutor(max_workers=min(len(todo), os.cpu_count() or 1)) as pool:
            list(pool.map(lambda sf: _compile(sf[0], sf[1], verbose), todo))
    objs = [str(CSRC / (Path(s).stem + ".o")) for s in SOURCES]
    if todo or not LIB_PATH.exists():
        cmd = [_nvcc(), "-shared", "-o", str(LIB_PATH), *objs, "-cudart", "shared", "-ldl"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    return LIB_PATH


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(path)
