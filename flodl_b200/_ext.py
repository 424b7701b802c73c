"""Loader for the in-tree native library (`flodl_b200/_C.so`).

`C` is the pybind11 module holding the sm_100a kernels, the symmetric-memory collectives and the
C++ runtime. It is built in-tree by `flodl_b200._build` (or `__graft_entry__.build()`); if the
shared object is missing it is built on first import. Nothing in the package falls back silently
to a PyTorch implementation on a CUDA device: ops that need the library raise if it is absent.
"""
from __future__ import annotations

import importlib
import os

import torch  # noqa: F401  (libtorch must be loaded before the extension)

_C = None
_ERR = None


def load():
    global _C, _ERR
    if _C is not None:
        return _C
    try:
        from . import _build
        if _build.needs_build() and os.environ.get("FLODL_B200_NO_BUILD", "0") != "1":
            _build.build()
        # FLODL_B200_BOUNDS_CHECK=1 selects the debug library (`_C_dbg.so`: device-side index checks that
        # record a violation instead of faulting); it is a separate file, the regular library is untouched
        _C = importlib.import_module("flodl_b200._C_dbg" if _build.BOUNDS_CHECK else "flodl_b200._C")
    except Exception as e:  # pragma: no cover - surfaced by require()
        _ERR = e
        _C = None
    return _C


def require():
    c = load()
    if c is None:
        raise RuntimeError(f"flodl_b200 native library is not available: {_ERR!r}")
    return c


def available() -> bool:
    return load() is not None


def lib_path() -> str:
    from . import _build
    return str(_build.TARGET)
