"""ctypes binding of ``libcoffin_b200.so`` (the sm_100a kernel library).

``call("name", *args)`` launches ``cb_name`` on the current torch CUDA stream: tensors are
passed as device pointers, Python ints as 64-bit integers, floats as C floats, ``None`` as a
null pointer, and the stream is appended.  A non-zero status raises.  There is no fallback:
on a CUDA machine a missing library is an error, so that a silent PyTorch path can never
stand in for the kernels (the reference instead fills missing natives from its torch
backend, ``backends/reference/__init__.py:1243-1260``).
"""
from __future__ import annotations

import ctypes
import os
from pathlib import Path

import torch

_LIB_PATH = Path(__file__).resolve().parent.parent / "_C" / "libcoffin_b200.so"
_lib: ctypes.CDLL | None = None

ERRORS = {10001: "unsupported shape/alignment", 10002: "bad argument", 10003: "driver entry point",
          10004: "device-side wait timed out"}


class KernelError(RuntimeError):
    pass


def available() -> bool:
    return _LIB_PATH.exists()


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not _LIB_PATH.exists():
            if os.environ.get("COFFIN_B200_AUTOBUILD", "1") == "1":
                from .._C.build import build
                build()
            else:
                raise KernelError(f"{_LIB_PATH} is missing: run python -m coffin_b200._C.build")
        _lib = ctypes.CDLL(str(_LIB_PATH))
    return _lib


def _conv(a):
    if isinstance(a, torch.Tensor):
        return ctypes.c_void_p(a.data_ptr())
    if a is None:
        return ctypes.c_void_p(0)
    if isinstance(a, bool):
        return ctypes.c_int64(int(a))
    if isinstance(a, int):
        return ctypes.c_int64(a)
    if isinstance(a, float):
        return ctypes.c_float(a)
    if isinstance(a, (ctypes.c_void_p, ctypes.c_int64, ctypes.c_float)) or type(a).__name__ == "CArgObject":
        return a
    raise TypeError(f"cannot pass {type(a)} to a kernel")


_fn_cache: dict[str, object] = {}


def call(name: str, *args, stream: int | None = None) -> None:
    fn = _fn_cache.get(name)
    if fn is None:
        fn = getattr(lib(), "cb_" + name)
        fn.restype = ctypes.c_int
        _fn_cache[name] = fn
    if stream is None:
        stream = torch.cuda.current_stream().cuda_stream
    rc = fn(*[_conv(a) for a in args], ctypes.c_void_p(stream))
    if rc != 0:
        raise KernelError(f"cb_{name} failed: {ERRORS.get(rc, 'CUDA error')} ({rc})")


def call_nostream(name: str, *args) -> int:
    fn = getattr(lib(), "cb_" + name)
    fn.restype = ctypes.c_int
    return fn(*[_conv(a) for a in args])


_exports: list[str] | None = None


def exported() -> list[str]:
    """Names of the ``cb_*`` entry points that the loaded library resolves: every ``CB_EXPORT``
    declaration found in the sources beside it is looked up in the shared object, so the count
    reported by ``ping`` is what the binary really exports, not a constant."""
    global _exports
    if _exports is None:
        import re
        names: set[str] = set()
        for src in sorted(_LIB_PATH.parent.glob("*.cu")):
            names.update(re.findall(r"CB_EXPORT\s+[\w\s\*]+?\b(cb_\w+)\s*\(", src.read_text()))
        handle = lib()
        _exports = sorted(n for n in names if hasattr(handle, n))
    return _exports


def set_pdl(on: bool) -> None:
    """Launch kernels with programmatic dependent launch (the prologue of kernel n+1 overlaps
    the tail of kernel n)."""
    call_nostream("set_pdl", int(on))
