"""Mixed precision (flodl/src/nn/amp.rs): `AutocastGuard`, `autocast`, `cast_parameters`, `GradScaler`.

Under an autocast guard the GEMM-shaped ops of `flodl_b200.ops` cast their inputs to the guard's
dtype and run on the tensor-core kernels (with the bf16 parameter shadows when present); the
guard also enters `torch.autocast` so the remaining PyTorch ops follow the same policy."""
from __future__ import annotations

from typing import Callable, Sequence

import torch

from .. import ops as _ops
from ..autograd import Variable
from ..tensor import Device, DType
from .module import Parameter


class AutocastGuard:
    def __init__(self, dtype=DType.BFloat16, device_type: str = "cuda"):
        self.dtype = dtype.torch if isinstance(dtype, DType) else dtype
        self.device_type = device_type
        self._prev = _ops.FLAGS.autocast
        _ops.FLAGS.autocast = self.dtype
        self._ctx = torch.autocast(device_type=device_type, dtype=self.dtype)
        self._ctx.__enter__()
        self._active = True

    @classmethod
    def new(cls, dtype): return cls(dtype)

    @classmethod
    def for_device(cls, device, dtype=DType.BFloat16):
        return cls(dtype, "cuda" if Device.of(device).is_cuda() else "cpu")

    def release(self):
        if self._active:
            self._ctx.__exit__(None, None, None)
            _ops.FLAGS.autocast = self._prev
            self._active = False

    def __enter__(self): return self
    def __exit__(self, *exc):
        self.release()
        return False
    def __del__(self):
        try:
            self.release()
        except Exception:
            pass


def autocast(dtype, f: Callable):
    g = AutocastGuard(dtype, "cuda" if torch.cuda.is_available() else "cpu")
    try:
        return f()
    finally:
        g.release()


def is_autocast_enabled() -> bool:
    return _ops.FLAGS.autocast is not None


def cast_parameters(params: Sequence[Parameter], dtype) -> None:
    """Cast parameter storage in place (e.g. to bf16 for inference); keeps `requires_grad`."""
    dt = dtype.torch if isinstance(dtype, DType) else dtype
    for p in params:
        t = p.t if isinstance(p, Parameter) else p
        if t.dtype != dt and t.is_floating_point():
            rg = t.requires_grad
            t.data = t.data.to(dt)
            t.grad = None
            t.requires_grad_(rg)


class GradScaler:
    """Dynamic loss scaling: scale 65536, x2 after 2000 clean steps, x0.5 (and the step is skipped)
    when any gradient is non-finite (flodl/src/nn/amp.rs:109-199)."""

    def __init__(self, init_scale: float = 65536.0, growth: float = 2.0, backoff: float = 0.5, interval: int = 2000):
        self._scale, self.growth, self.backoff, self.interval = init_scale, growth, backoff, interval
        self.steps_since_growth = 0
        self.found_inf = False

    @classmethod
    def new(cls): return cls()

    def scale(self, loss: Variable) -> Variable:
        return loss.mul_scalar(self._scale)

    def scale_factor(self) -> float:
        return self._scale

    def step(self, params: Sequence[Parameter], step_fn: Callable[[], None]) -> bool:
        inv = 1.0 / self._scale
        grads = [(p.t if isinstance(p, Parameter) else p) for p in params]
        grads = [t for t in grads if t.grad is not None]
        if grads:
            finite = torch.stack([torch.isfinite(t.grad).all() for t in grads]).all()
            if not bool(finite.item()):
                self.found_inf = True
                return False
            torch._foreach_mul_([t.grad for t in grads], inv)
        step_fn()
        return True

    def update(self) -> None:
        if self.found_inf:
            self._scale *= self.backoff
            self.steps_since_growth = 0
        else:
            self.steps_since_growth += 1
            if self.steps_since_growth >= self.interval:
                self._scale *= self.growth
                self.steps_since_growth = 0
        self.found_inf = False

    # Stateful
    def save_state(self, w) -> None:
        import struct
        w.write(struct.pack("<dq", self._scale, self.steps_since_growth))

    def load_state(self, r) -> None:
        import struct
        self._scale, self.steps_since_growth = struct.unpack("<dq", r.read(16))
