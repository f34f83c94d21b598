"""Ahead-of-time build of the sm_100a kernel library.

``python -m coffin_b200._C.build`` compiles every ``.cu`` beside this file with
``nvcc -gencode arch=compute_100a,code=sm_100a`` into ``libcoffin_b200.so`` in this
directory (nvcc cross-compiles without a GPU).  The library exports plain C symbols and
links only the CUDA runtime, so it is built once, travels with the tree and is loaded
with ctypes; there is no JIT step at import (the reference JIT-builds its extensions on
first import behind a file lock, ``backends/corex/kernels/__init__.py:85-167``).
"""
from __future__ import annotations

import concurrent.futures as cf
import hashlib
import os
import shutil
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
LIB = HERE / "libcoffin_b200.so"
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
FLAGS = ["-O3", "-std=c++17", "-lineinfo", "--use_fast_math", "-Xcompiler", "-fPIC",
         "-Xcompiler", "-fvisibility=hidden", "--expt-relaxed-constexpr"]


def nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(exe).exists():
        raise RuntimeError("nvcc not found")
    return exe


def sources() -> list[Path]:
    return sorted(HERE.glob("*.cu"))


def _digest(src: Path) -> str:
    h = hashlib.sha256()
    h.update(src.read_bytes())
    for hdr in sorted(HERE.glob("*.cuh")) + sorted(HERE.glob("*.h")):
        h.update(hdr.read_bytes())
    h.update(" ".join(ARCH + FLAGS).encode())
    return h.hexdigest()


def _compile(src: Path, verbose: bool) -> tuple[Path, str]:
    obj = HERE / "build" / (src.stem + ".o")
    stamp = obj.with_suffix(".sha")
    dig = _digest(src)
    if obj.exists() and stamp.exists() and stamp.read_text() == dig:
        return obj, ""
    obj.parent.mkdir(exist_ok=True)
    cmd = [nvcc(), *ARCH, *FLAGS, "-c", str(src), "-o", str(obj)]
    if verbose:
        cmd[1:1] = ["-Xptxas", "-v"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src.name}:\n{r.stdout}\n{r.stderr}")
    stamp.write_text(dig)
    return obj, r.stderr


def build(verbose: bool = False, force: bool = False) -> Path:
    """Compile what changed and link the shared library. Returns its path."""
    if force and (HERE / "build").exists():
        shutil.rmtree(HERE / "build")
    srcs = sources()
    with cf.ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as ex:
        results = list(ex.map(lambda s: _compile(s, verbose), srcs))
    objs = [o for o, _ in results]
    if verbose:
        for (_, log), s in zip(results, srcs):
            if log:
                print(f"==== {s.name}\n{log}")
    newest = max(o.stat().st_mtime for o in objs)
    if not LIB.exists() or LIB.stat().st_mtime < newest:
        cmd = [nvcc(), *ARCH, "-shared", "-o", str(LIB), *map(str, objs)]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    return LIB


if __name__ == "__main__":
    path = build(verbose="-v" in sys.argv, force="--force" in sys.argv)
    print(path)
