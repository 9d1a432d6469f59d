"""In-tree nvcc build of the C-ABI library ``libmk_b200.so`` for sm_100a.

The reference builds one cubin and one host library per kernel image at run time, with a content-hash cache
(``sgl_muse_mega/common/jit.py:100-146``). Here one shared library carries every kernel; it is built once, in the source
tree (``sgl_muse_mega_b200/lib/``), and rebuilt only when a source under ``csrc/`` or ``include/`` is newer than it.
"""

from __future__ import annotations

import os
import shutil
import subprocess
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent.parent
CSRC = PKG / "csrc"
INCLUDE = PKG.parent / "include"
LIB_DIR = PKG / "lib"
LIB = LIB_DIR / "libmk_b200.so"
# The trace build: the same sources with the kernels' %globaltimer stamps compiled in (per-CTA milestones of the expert,
# dense, row and attention kernels, read back through mk_*_trace_read; ``bench.py --timeline`` prints a layer's timeline).
TRACE_LIB = LIB_DIR / "libmk_b200_trace.so"
TRACE_FLAGS = ["-DUMMA_TRACE", "-DDENSE_TRACE", "-DROWS_TRACE"]

DEVICE_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC",
]  # fmt: skip


def nvcc() -> str:
    home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    exe = Path(home) / "bin" / "nvcc"
    if exe.exists():
        return str(exe)
    found = shutil.which("nvcc")
    if not found:
        raise RuntimeError("nvcc not found (set CUDA_HOME)")
    return found


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def _stale(lib: Path = LIB) -> bool:
    if not lib.exists():
        return True
    t = lib.stat().st_mtime
    deps = list(CSRC.glob("*")) + list(INCLUDE.glob("*.h"))
    return any(p.stat().st_mtime > t for p in deps)


def build(force: bool = False, verbose: bool = False, trace: bool = False) -> Path:
    """Compiles every ``csrc/*.cu`` for sm_100a and links ``libmk_b200.so`` (``trace``: the trace build,
    ``libmk_b200_trace.so``); returns its path."""
    lib = TRACE_LIB if trace else LIB
    if not force and not _stale(lib):
        return lib
    LIB_DIR.mkdir(exist_ok=True)
    obj_dir = LIB_DIR / ("obj_trace" if trace else "obj")
    obj_dir.mkdir(exist_ok=True)
    flags = list(DEVICE_FLAGS) + (TRACE_FLAGS if trace else [])
    if verbose:
        flags += ["-Xptxas", "-v"]

    def compile_one(src: Path) -> Path:
        obj = obj_dir / (src.stem + ".o")
        cmd = [nvcc(), *flags, "-I", str(INCLUDE), "-c", str(src), "-o", str(obj)]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src.name}:\n{r.stdout}\n{r.stderr}")
        if verbose:
            print(r.stderr)
        return obj

    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as pool:
        objs = list(pool.map(compile_one, sources()))
    tmp = lib.with_suffix(".so.tmp")
    cmd = [nvcc(), "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "--cudart", "static",
           "-o", str(tmp), *map(str, objs)]  # fmt: skip
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    os.replace(tmp, lib)
    return lib


if __name__ == "__main__":
    import sys

    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv, trace="--trace" in sys.argv))
