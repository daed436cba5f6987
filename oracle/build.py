"""Build the C oracle (oracle/libcdr_oracle.so) with gcc.

TEST INFRASTRUCTURE ONLY: tests, the smoke check and the benchmark's CPU-baseline leg use
it as the checker; the package never imports it.

The reference itself has nothing that compiles here: its device code is Choreo DSL (`.co`)
that needs the `choreo` compiler, and its only C++ is a header (choreo-headers/choreo.h), so
there is no `oracle/_ref` build.
"""
from __future__ import annotations

import subprocess
from pathlib import Path

HERE = Path(__file__).resolve().parent
SRC = HERE / "cdr_oracle.c"
LIB = HERE / "libcdr_oracle.so"


def build(force: bool = False) -> Path:
    if force or not LIB.exists() or LIB.stat().st_mtime < SRC.stat().st_mtime:
        cmd = ["gcc", "-O2", "-fPIC", "-shared", "-ffp-contract=off", "-fno-fast-math", "-std=c11",
               str(SRC), "-o", str(LIB), "-lm"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"gcc failed:\n{res.stderr}")
    return LIB


if __name__ == "__main__":
    print(build(force=True))
