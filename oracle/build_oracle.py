"""Build recipe for the oracle's native parts (test infrastructure only).

* ``oracle/_build/liboracle.so``  -- oracle/oracle_train.c (gcc, OpenMP).
* ``oracle/_ref/prune_input.so``  -- the REFERENCE's own window enumeration,
  compiled from ``<reference>/flyvec/src/prune_input.cpp`` where it lies; only
  attempted when a reference checkout is present.  Nothing is copied into this
  repository; the output directory is git-ignored.

The reference's trainer is CUDA-only and its build script needs cuBLAS/cuRAND
and a GPU to run, so only ``prune_input.cpp`` (plain C++/OpenMP) is built here.
"""
from __future__ import annotations

import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
BUILD = HERE / "_build"
REF_OUT = HERE / "_ref"
CUDA_INC = "/usr/local/cuda/include"  # prune_input.cpp includes <cuda.h> for nothing but the header


def build_oracle_lib(force: bool = False) -> Path:
    BUILD.mkdir(exist_ok=True)
    out = BUILD / "liboracle.so"
    src = HERE / "oracle_train.c"
    if force or not out.exists() or out.stat().st_mtime < src.stat().st_mtime:
        subprocess.run(["gcc", "-O2", "-fopenmp", "-fPIC", "-shared", "-std=c11", "-o", str(out), str(src), "-lm"],
                       check=True)
    return out


def build_reference_prune_input(reference_root: str = "/root/reference") -> Path | None:
    src = Path(reference_root) / "flyvec" / "src" / "prune_input.cpp"
    if not src.exists():
        return None
    REF_OUT.mkdir(exist_ok=True)
    out = REF_OUT / "prune_input.so"
    if not out.exists() or out.stat().st_mtime < src.stat().st_mtime:
        subprocess.run(["g++", "-O2", "-fopenmp", "-fPIC", "-shared", "-I", CUDA_INC, "-o", str(out), str(src)],
                       check=True)
    return out


if __name__ == "__main__":
    print(build_oracle_lib(force=True))
    print(build_reference_prune_input(sys.argv[1] if len(sys.argv) > 1 else "/root/reference"))
