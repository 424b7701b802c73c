"""Verbosity-gated logging (flodl/src/log.rs:1-110): five levels, `FLODL_VERBOSITY` env override,
Normal/Verbose to stdout, Debug/Trace to stderr."""
from __future__ import annotations

import os
import sys
from enum import IntEnum


class Verbosity(IntEnum):
    Quiet = 0
    Normal = 1
    Verbose = 2
    Debug = 3
    Trace = 4


def _from_env() -> Verbosity:
    v = os.environ.get("FLODL_VERBOSITY", "").strip().lower()
    names = {"quiet": 0, "normal": 1, "verbose": 2, "debug": 3, "trace": 4}
    if v in names:
        return Verbosity(names[v])
    if v.isdigit() and int(v) <= 4:
        return Verbosity(int(v))
    return Verbosity.Normal


_LEVEL = _from_env()


def verbosity() -> Verbosity:
    return _LEVEL


def set_verbosity(level) -> None:
    global _LEVEL
    _LEVEL = Verbosity(int(level))


def enabled(level: Verbosity) -> bool:
    return _LEVEL >= level


def msg(*args) -> None:
    if _LEVEL >= Verbosity.Normal:
        print(*args, file=sys.stdout, flush=True)


def verbose(*args) -> None:
    if _LEVEL >= Verbosity.Verbose:
        print(*args, file=sys.stdout, flush=True)


def debug(*args) -> None:
    if _LEVEL >= Verbosity.Debug:
        print(*args, file=sys.stderr, flush=True)


def trace(*args) -> None:
    if _LEVEL >= Verbosity.Trace:
        print(*args, file=sys.stderr, flush=True)
