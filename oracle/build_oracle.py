"""Build recipe for the oracle's native parts (test infrastructure only).

* ``oracle/_build/liboracle.so``      -- oracle/oracle_train.c (gcc, OpenMP).
* ``oracle/_ref/prune_input.so``      -- the REFERENCE's own window enumeration,
  compiled from ``<reference>/flyvec/src/prune_input.cpp`` where it lies.
* ``oracle/_ref/ref_kernels_host.so`` -- the REFERENCE's own training kernels,
  executed on the host: the text of its ``__global__`` functions is cut out of
  ``<reference>/flyvec/src/cuda_funcs.cu`` and ``cu_special_reduction.cu`` into
  the generated ``oracle/_ref/ref_kernels.inc`` and compiled by g++ against the
  CUDA-on-host model of ``oracle/cuda_on_host.h`` (``oracle/ref_kernels_host.cpp``
  restates only the host-side launch sequence).

The two ``_ref`` targets are only attempted when a reference checkout is
present (``FLYVEC_REFERENCE`` in the environment, or a ``reference`` directory
beside this repository).  Nothing of the reference is copied into this
repository: the output directory is git-ignored and holds generated files and
binaries only.  The reference's complete trainer (cuBLAS, cuRAND, managed
memory, five shared objects made by its own script) is not built.
"""
from __future__ import annotations

import os
import re
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
BUILD = HERE / "_build"
REF_OUT = HERE / "_ref"
CUDA_INC = "/usr/local/cuda/include"  # prune_input.cpp includes <cuda.h> for nothing but the header


def reference_root(explicit: str | os.PathLike | None = None) -> Path | None:
    """Where the reference checkout lies, or None."""
    cands = [explicit, os.environ.get("FLYVEC_REFERENCE"), HERE.parent.parent / "reference"]
    for c in cands:
        if c and (Path(c) / "flyvec" / "src").is_dir():
            return Path(c)
    return None


def _newer(out: Path, *srcs: Path) -> bool:
    return out.exists() and all(out.stat().st_mtime >= s.stat().st_mtime for s in srcs)


def build_oracle_lib(force: bool = False) -> Path:
    BUILD.mkdir(exist_ok=True)
    out = BUILD / "liboracle.so"
    src = HERE / "oracle_train.c"
    if force or not _newer(out, src):
        subprocess.run(["gcc", "-O2", "-fopenmp", "-fPIC", "-shared", "-std=c11", "-o", str(out), str(src), "-lm"],
                       check=True)
    return out


def build_reference_prune_input(root: str | os.PathLike | None = None) -> Path | None:
    ref = reference_root(root)
    out = REF_OUT / "prune_input.so"
    if ref is None:
        return out if out.exists() else None
    src = ref / "flyvec" / "src" / "prune_input.cpp"
    REF_OUT.mkdir(exist_ok=True)
    if not _newer(out, src):
        subprocess.run(["g++", "-O2", "-fopenmp", "-fPIC", "-shared", "-I", CUDA_INC, "-o", str(out), str(src)],
                       check=True)
    return out


# ---------------------------------------------------------------------------
# The reference's kernels, cut out of its sources by name
# ---------------------------------------------------------------------------
#: ``__global__`` functions of the live training path (every overload of a name is taken)
KERNELS = {
    "cuda_funcs.cu": [
        "cuda_func1_odd", "cuda_func1_even", "dense_sparse_matmul_special", "cuda_ds_xx_t_synapses_kernel",
        "get_max_and_m_max_kernel_2", "func_ds_eq_ds_input_kernel_sparse", "fill_func_kernel",
        "xx_atomic_update_kernel", "inflate_from_M_kernel_4",
    ],
    "cu_special_reduction.cu": [
        "reduce_by_chunks_and_absmax_kernel_sparse_2D", "max_of_AbsVal_kernel_finish",
        "update_model_multiGPU_kernel_sparse_2D",
    ],
}
#: plain host helpers taken the same way
HOST_FUNCS = {"cuda_funcs.cu": ["split_to_chuncks"]}
MACROS = {"cuda_funcs.cu": ["CACHE_LINE_SIZE"]}


def _skip_noncode(text: str, i: int) -> int:
    """If a comment or a literal starts at ``i`` return the index just past it, else ``i``."""
    if text.startswith("//", i):
        j = text.find("\n", i)
        return len(text) if j < 0 else j
    if text.startswith("/*", i):
        j = text.find("*/", i + 2)
        return len(text) if j < 0 else j + 2
    if text[i] in "\"'":
        q = text[i]
        j = i + 1
        while j < len(text) and text[j] != q:
            j += 2 if text[j] == "\\" else 1
        return j + 1
    return i


def _match(text: str, i: int, open_ch: str, close_ch: str) -> int:
    """``text[i]`` is ``open_ch``; index just past the matching ``close_ch``."""
    depth = 0
    while i < len(text):
        j = _skip_noncode(text, i)
        if j != i:
            i = j
            continue
        c = text[i]
        if c == open_ch:
            depth += 1
        elif c == close_ch:
            depth -= 1
            if depth == 0:
                return i + 1
        i += 1
    raise ValueError("unbalanced source text")


def extract_definitions(text: str, name: str, global_only: bool) -> list[str]:
    """Every *definition* (not declaration) of function ``name`` with its template header."""
    qual = r"__global__\s+" if global_only else r""
    pat = re.compile(r"(template\s*<[^>]*>\s*)?" + qual + r"void\s+" + re.escape(name) + r"\s*\(")
    out = []
    for mt in pat.finditer(text):
        # a match inside a comment is not code
        line_start = text.rfind("\n", 0, mt.start()) + 1
        if "//" in text[line_start:mt.start()]:
            continue
        close = _match(text, mt.end() - 1, "(", ")")
        k = close
        while k < len(text) and text[k].isspace():
            k += 1
        if k >= len(text) or text[k] != "{":
            continue  # a declaration
        end = _match(text, k, "{", "}")
        out.append(text[mt.start():end])
    return out


def generate_reference_kernels(ref: Path, out: Path) -> None:
    parts = ["// GENERATED from a reference checkout by oracle/build_oracle.py -- not part of this repository.\n"]
    for fname in sorted(set(KERNELS) | set(HOST_FUNCS) | set(MACROS)):
        text = (ref / "flyvec" / "src" / fname).read_text()
        for macro in MACROS.get(fname, []):
            mt = re.search(r"^#define\s+" + macro + r"\b.*$", text, re.M)
            if not mt:
                raise RuntimeError(f"{fname}: macro {macro} not found")
            parts.append(mt.group(0) + "\n")
        for name in KERNELS.get(fname, []):
            defs = extract_definitions(text, name, global_only=True)
            if not defs:
                raise RuntimeError(f"{fname}: no definition of __global__ {name} found")
            parts += [f"// ---- {fname}: {name}\n{d}\n" for d in defs]
        for name in HOST_FUNCS.get(fname, []):
            defs = extract_definitions(text, name, global_only=False)
            if not defs:
                raise RuntimeError(f"{fname}: no definition of {name} found")
            parts += [f"// ---- {fname}: {name}\n{d}\n" for d in defs]
    out.write_text("\n".join(parts))


def build_reference_kernels(root: str | os.PathLike | None = None, force: bool = False) -> Path | None:
    """``oracle/_ref/ref_kernels_host.so`` or None when it neither exists nor can be built."""
    out = REF_OUT / "ref_kernels_host.so"
    ref = reference_root(root)
    if ref is None:
        return out if out.exists() else None
    REF_OUT.mkdir(exist_ok=True)
    srcs = [HERE / "ref_kernels_host.cpp", HERE / "cuda_on_host.cpp", HERE / "cuda_on_host.h", Path(__file__)]
    refsrcs = [ref / "flyvec" / "src" / f for f in KERNELS]
    if force or not _newer(out, *srcs, *refsrcs):
        inc = REF_OUT / "ref_kernels.inc"
        generate_reference_kernels(ref, inc)
        # -O1 without contraction: every float operation rounds where the source text says
        subprocess.run(["g++", "-O1", "-ffp-contract=off", "-fno-fast-math", "-std=c++17", "-w", "-fPIC", "-shared",
                        "-I", str(HERE), "-I", str(REF_OUT), "-o", str(out),
                        str(HERE / "ref_kernels_host.cpp"), str(HERE / "cuda_on_host.cpp")], check=True)
    return out


if __name__ == "__main__":
    root = sys.argv[1] if len(sys.argv) > 1 else None
    print(build_oracle_lib(force=True))
    print(build_reference_prune_input(root))
    print(build_reference_kernels(root, force=True))
