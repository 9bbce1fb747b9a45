"""Builds oracle/_build/liboracle.so from oracle.c with gcc (no -ffast-math, no FMA contraction, so the scalar
expressions round exactly as written).  TEST INFRASTRUCTURE, see oracle/__init__.py."""
from __future__ import annotations

import subprocess
from pathlib import Path

HERE = Path(__file__).resolve().parent
OUT = HERE / "_build" / "liboracle.so"


def build(force: bool = False) -> Path:
    src = HERE / "oracle.c"
    if not force and OUT.exists() and OUT.stat().st_mtime >= src.stat().st_mtime:
        return OUT
    OUT.parent.mkdir(exist_ok=True)
    cmd = ["gcc", "-O2", "-std=c11", "-fPIC", "-shared", "-ffp-contract=off", "-fno-fast-math", "-fopenmp",
           "-Wall", "-o", str(OUT), str(src), "-lm"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"gcc failed:\n{r.stdout}\n{r.stderr}")
    return OUT


if __name__ == "__main__":
    print(build(force=True))
