"""Learning-rate schedules (flodl/src/nn/scheduler.rs): pure functions of the step index."""
from __future__ import annotations

import math
from typing import Sequence


class Scheduler:
    @classmethod
    def new(cls, *args, **kw):
        return cls(*args, **kw)

    def lr(self, step: int) -> float:  # pragma: no cover - interface
        raise NotImplementedError


class StepDecay(Scheduler):
    def __init__(self, base_lr: float, step_size: int, gamma: float):
        self.base_lr, self.step_size, self.gamma = base_lr, max(1, step_size), gamma
    def lr(self, step): return self.base_lr * self.gamma ** (step // self.step_size)


class CosineScheduler(Scheduler):
    def __init__(self, base_lr: float, min_lr: float, total_steps: int):
        self.base_lr, self.min_lr, self.total = base_lr, min_lr, max(1, total_steps)
    def lr(self, step):
        s = min(step, self.total)
        return self.min_lr + 0.5 * (self.base_lr - self.min_lr) * (1 + math.cos(math.pi * s / self.total))


class WarmupScheduler(Scheduler):
    """Linear ramp `target * (s+1)/W` for the first W steps, then `inner.lr(s - W)`."""
    def __init__(self, inner: Scheduler, target_lr: float, warmup_steps: int):
        self.inner, self.target_lr, self.warmup = inner, target_lr, warmup_steps
    def lr(self, step):
        if step < self.warmup:
            return self.target_lr * (step + 1) / self.warmup
        return self.inner.lr(step - self.warmup)


class PlateauScheduler:
    """Lower-is-better metric; after `patience` non-improving observations lr *= factor (>= min_lr)."""
    @classmethod
    def new(cls, base_lr: float, patience: int, factor: float, min_lr: float) -> "PlateauScheduler":
        return cls(base_lr, patience, factor, min_lr)

    def __init__(self, base_lr: float, patience: int, factor: float, min_lr: float):
        self.patience, self.factor, self.min_lr = patience, factor, min_lr
        self.current_lr, self.best, self.wait = base_lr, math.inf, 0
    def observe(self, metric: float) -> float:
        if metric < self.best:
            self.best, self.wait = metric, 0
        else:
            self.wait += 1
            if self.wait >= self.patience:
                self.current_lr = max(self.current_lr * self.factor, self.min_lr)
                self.wait = 0
        return self.current_lr
    def lr(self, step: int = 0) -> float:
        return self.current_lr


class ExponentialLR(Scheduler):
    def __init__(self, base_lr: float, gamma: float): self.base_lr, self.gamma = base_lr, gamma
    def lr(self, step): return self.base_lr * self.gamma ** step


class MultiStepLR(Scheduler):
    def __init__(self, base_lr: float, milestones: Sequence[int], gamma: float):
        self.base_lr, self.milestones, self.gamma = base_lr, sorted(milestones), gamma
    def lr(self, step): return self.base_lr * self.gamma ** sum(1 for m in self.milestones if step >= m)


class OneCycleLR(Scheduler):
    def __init__(self, max_lr: float, total_steps: int, warmup_frac: float = 0.3):
        self.max_lr, self.total = max_lr, total_steps
        self.warmup = round(total_steps * min(max(warmup_frac, 0.0), 1.0))
    @classmethod
    def with_warmup_frac(cls, max_lr, total_steps, warmup_frac): return cls(max_lr, total_steps, warmup_frac)
    def lr(self, step):
        step = min(step, self.total)
        lo = self.max_lr / 25.0
        if step < self.warmup:
            return lo + (step / max(self.warmup, 1)) * (self.max_lr - lo)
        t = (step - self.warmup) / max(self.total - self.warmup, 1)
        return lo + 0.5 * (self.max_lr - lo) * (1 + math.cos(t * math.pi))


class CyclicLR(Scheduler):
    def __init__(self, base_lr: float, max_lr: float, step_size: int, step_size_down: int = None):
        self.base_lr, self.max_lr, self.up = base_lr, max_lr, step_size
        self.down = step_size if step_size_down is None else step_size_down
    @classmethod
    def asymmetric(cls, base_lr, max_lr, up, down): return cls(base_lr, max_lr, up, down)
    def lr(self, step):
        pos = step % (self.up + self.down)
        scale = pos / self.up if pos <= self.up else 1.0 - (pos - self.up) / self.down
        return self.base_lr + (self.max_lr - self.base_lr) * scale
