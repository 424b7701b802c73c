"""Gradient-mode guards (flodl/src/autograd/context.rs:24-66)."""
from __future__ import annotations

import torch


class NoGradGuard:
    """RAII-style guard: gradient recording is off while the object is alive / inside `with`."""

    @classmethod
    def new(cls, *args, **kw):
        return cls(*args, **kw)

    def __init__(self):
        self._prev = torch.is_grad_enabled()
        torch.set_grad_enabled(False)
        self._active = True

    def release(self):
        if self._active:
            torch.set_grad_enabled(self._prev)
            self._active = False

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.release()
        return False

    def __del__(self):
        self.release()


def no_grad(f=None):
    """`no_grad(|| ...)`: run `f` without recording; with no argument, a context manager."""
    if f is None:
        return torch.no_grad()
    with torch.no_grad():
        return f()


def is_grad_enabled() -> bool:
    return torch.is_grad_enabled()
