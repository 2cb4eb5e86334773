"""Build ``libb200scan.so`` (the C-ABI CUDA library) in-tree with nvcc for sm_100a.

``python -m tsfast_b200.build`` compiles every ``csrc/*.cu`` into ``tsfast_b200/lib/`` and links
them into one shared library.  nvcc cross-compiles, so no GPU is needed to build.  Objects are
rebuilt only when a source or header is newer.
"""

from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
LIBDIR = PKG / "lib"
LIB = LIBDIR / "libb200scan.so"
INCLUDE = PKG.parent / "include"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-lineinfo", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "-ccbin", "/usr/bin/g++",
]
# Approximate division / flush-to-zero only where the reference's own GPU kernels use fast
# transcendentals (the Mamba section and its conv + SiLU); the diagonal, all-pole, projection and
# glue kernels keep IEEE arithmetic.
FAST_MATH_SOURCES = {"mamba_scan.cu", "conv_silu.cu"}


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(exe).exists():
        raise RuntimeError("nvcc not found: cannot build libb200scan.so")
    return exe


def _stale(target: Path, deps: list[Path]) -> bool:
    if not target.exists():
        return True
    mt = target.stat().st_mtime
    return any(d.stat().st_mtime > mt for d in deps)


def build(verbose: bool = False, force: bool = False, extra_flags: list[str] | None = None,
          out: Path | None = None) -> Path:
    """Compile the library; returns its path. ``extra_flags``/``out`` serve tuning builds."""
    LIBDIR.mkdir(exist_ok=True)
    out = Path(out) if out else LIB
    objdir = LIBDIR if out == LIB else out.parent / (out.stem + "_obj")
    objdir.mkdir(parents=True, exist_ok=True)
    headers = sorted(CSRC.glob("*.cuh")) + sorted(INCLUDE.glob("*.h"))
    sources = sorted(CSRC.glob("*.cu"))
    nvcc = _nvcc()
    flags = NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + (extra_flags or [])

    def compile_one(src: Path):
        obj = objdir / (src.stem + ".o")
        if force or _stale(obj, [src, *headers]):
            extra = ["--use_fast_math"] if src.name in FAST_MATH_SOURCES else []
            r = subprocess.run([nvcc, *flags, *extra, "-c", str(src), "-o", str(obj)], capture_output=True, text=True)
            if r.returncode != 0:
                raise RuntimeError(f"nvcc failed on {src.name}:\n{r.stdout}\n{r.stderr}")
            if verbose:
                sys.stderr.write(r.stderr)
            return obj, True
        return obj, False

    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as ex:
        results = list(ex.map(compile_one, sources))
    objs = [o for o, _ in results]
    if force or any(ch for _, ch in results) or _stale(out, objs):
        r = subprocess.run([nvcc, "-shared", "-o", str(out), *map(str, objs), "-ccbin", "/usr/bin/g++"],
                           capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    return out


if __name__ == "__main__":
    p = build(verbose="-v" in sys.argv, force="-f" in sys.argv)
    print(p)
