"""Build recipes for the test oracle (never for the shipped library).

``build_oracle()`` compiles ``candy_oracle.c`` into ``liboracle.so`` next to it.

``build_ref()`` compiles the reference project's own CUDA source for the quantized
path (``tensor/internal/cuda/kernels/quantized.cu`` of a gocnn/candy checkout) into
``_ref/quantized_sm100a.cubin`` *from where it lies*; no reference source is copied.
The checkout is looked for in ``$CANDY_REFERENCE_DIR``, else in a directory named
``reference`` beside this repository.  The cubin is a test
fixture: GPU tests load it with the CUDA driver API to pin this oracle against code
the reference itself ships.  (The reference's Go CPU path cannot be built here: no Go
toolchain.  Its Metal shaders cannot be built either.)

Run as a script to build both:  ``python oracle/build_oracle.py``
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
ORACLE_SO = HERE / "liboracle.so"
REF_DIR = HERE / "_ref"
REF_CUBIN = REF_DIR / "quantized_sm100a.cubin"
REF_SOURCE_REL = Path("tensor/internal/cuda/kernels/quantized.cu")


def _newer(target: Path, *sources: Path) -> bool:
    if not target.exists():
        return False
    t = target.stat().st_mtime
    return all(s.stat().st_mtime <= t for s in sources)


def build_oracle(force: bool = False) -> Path:
    src = HERE / "candy_oracle.c"
    if not force and _newer(ORACLE_SO, src):
        return ORACLE_SO
    cmd = ["gcc", "-O2", "-ffp-contract=off", "-fno-fast-math", "-fopenmp", "-shared", "-fPIC",
           "-o", str(ORACLE_SO), str(src), "-lm"]
    subprocess.run(cmd, check=True)
    return ORACLE_SO


def reference_dir() -> Path | None:
    d = os.environ.get("CANDY_REFERENCE_DIR")
    p = Path(d) if d else HERE.parent.parent / "reference"
    return p if (p / REF_SOURCE_REL).exists() else None


def build_ref(force: bool = False) -> Path | None:
    """Returns the cubin path, or None when no reference checkout / nvcc is present."""
    ref = reference_dir()
    if ref is None or shutil.which("nvcc") is None:
        return REF_CUBIN if REF_CUBIN.exists() else None
    src = ref / REF_SOURCE_REL
    if not force and _newer(REF_CUBIN, src):
        return REF_CUBIN
    REF_DIR.mkdir(exist_ok=True)
    cmd = ["nvcc", "-cubin", "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo",
           "-I", str(src.parent), "-o", str(REF_CUBIN), str(src)]
    subprocess.run(cmd, check=True)
    return REF_CUBIN


if __name__ == "__main__":
    print(build_oracle(force="--force" in sys.argv))
    print(build_ref(force="--force" in sys.argv))
