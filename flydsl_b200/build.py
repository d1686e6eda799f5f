"""In-tree nvcc build of libflymoe_sm100.so (sm_100a only).

``python -m flydsl_b200.build`` compiles every ``csrc/*.cu`` with
``-gencode arch=compute_100a,code=sm_100a -lineinfo`` and links one shared library
next to this file.  nvcc cross-compiles without a GPU.  Objects are rebuilt only
when a source or header is newer than them; the ``-Xptxas -v`` report of every
object (registers, spills, shared memory per kernel) is kept beside it as
``build/<name>.ptxas.txt`` and survives builds that recompile nothing.

``--prof`` builds a second library, ``libflymoe_sm100_prof.so``, from the same sources
with ``-DFLYMOE_PROF``: the grouped-GEMM kernels then add up the cycles their roles spend
waiting (``FLYMOE_LIB=<that file> python bench.py --wait-accounting`` prints them).
"""

from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
INCLUDE = PKG_DIR.parent / "include"
BUILD_DIR = PKG_DIR / "build"
LIB_PATH = PKG_DIR / "libflymoe_sm100.so"
PROF_LIB_PATH = PKG_DIR / "libflymoe_sm100_prof.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr", "-Xptxas", "-v",
]


def _nvcc() -> str:
    cand = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(cand):
        raise RuntimeError("nvcc not found: the flymoe library cannot be built")
    return cand


def _newest_header_mtime() -> float:
    hdrs = list(CSRC.glob("*.cuh")) + list(INCLUDE.glob("*.h"))
    return max(p.stat().st_mtime for p in hdrs)


def build(force: bool = False, verbose: bool = False, prof: bool = False) -> Path:
    """Compile (if stale) and return the path of the shared library."""
    nvcc = _nvcc()
    out_dir = BUILD_DIR / "prof" if prof else BUILD_DIR
    out_dir.mkdir(parents=True, exist_ok=True)
    lib_path = PROF_LIB_PATH if prof else LIB_PATH
    extra = ["-DFLYMOE_PROF"] if prof else []
    sources = sorted(CSRC.glob("*.cu"))
    hdr_m = _newest_header_mtime()

    def compile_one(src: Path) -> Path:
        obj = out_dir / (src.stem + ".o")
        stale = force or (not obj.exists()) or obj.stat().st_mtime < max(src.stat().st_mtime, hdr_m)
        if stale:
            cmd = [nvcc, *NVCC_FLAGS, *extra, "-c", str(src), "-o", str(obj)]
            r = subprocess.run(cmd, capture_output=True, text=True)
            if r.returncode != 0:
                raise RuntimeError(f"nvcc failed on {src.name}:\n{r.stdout}\n{r.stderr}")
            (out_dir / (src.stem + ".ptxas.txt")).write_text(r.stdout + r.stderr)
        return obj

    with ThreadPoolExecutor(max_workers=min(8, len(sources))) as ex:
        objs = list(ex.map(compile_one, sources))
    relink = force or (not lib_path.exists()) or any(o.stat().st_mtime > lib_path.stat().st_mtime for o in objs)
    if relink:
        cmd = [nvcc, "-shared", "-o", str(lib_path), *map(str, objs), "-gencode",
               "arch=compute_100a,code=sm_100a", "-cudart", "static"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    if verbose:
        print(ptxas_report(out_dir))
    return lib_path


def ptxas_report(out_dir: Path = BUILD_DIR) -> str:
    """The kept ``-Xptxas -v`` output of every object, one section per source file."""
    parts = []
    for p in sorted(out_dir.glob("*.ptxas.txt")):
        parts.append(f"==== {p.name[:-len('.ptxas.txt')]}.cu\n{p.read_text()}")
    return "\n".join(parts)


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose=True, prof="--prof" in sys.argv)
    print(path)
