"""Epoch-history analysis (flodl/src/graph/trend.rs): OLS slope, stall / improvement / convergence."""
from __future__ import annotations

import math
from typing import List, Sequence


def ols_slope(data: Sequence[float]) -> float:
    n = len(data)
    if n < 2:
        return 0.0
    sx = n * (n - 1) / 2.0
    sy = float(sum(data))
    sxy = float(sum(i * y for i, y in enumerate(data)))
    sxx = float(sum(i * i for i in range(n)))
    denom = n * sxx - sx * sx
    if abs(denom) < 1e-15:
        return 0.0
    return (n * sxy - sx * sy) / denom


class Trend:
    def __init__(self, values: Sequence[float]):
        self._v = [float(x) for x in values]

    @classmethod
    def new(cls, values: Sequence[float]) -> "Trend": return cls(values)

    def __len__(self): return len(self._v)
    def len(self): return len(self._v)
    def is_empty(self): return not self._v
    def values(self) -> List[float]: return list(self._v)
    def last(self, n: int) -> List[float]: return self._v[max(0, len(self._v) - n):] if n > 0 else []
    def latest(self) -> float: return self._v[-1] if self._v else 0.0
    def mean(self) -> float: return sum(self._v) / len(self._v) if self._v else 0.0
    def min(self) -> float: return min(self._v) if self._v else math.inf
    def max(self) -> float: return max(self._v) if self._v else -math.inf
    def _window(self, w: int): return self.last(w) if w > 0 else self._v
    def slope(self, window: int = 0) -> float: return ols_slope(self._window(window))
    def stalled(self, window: int, tol: float) -> bool: return abs(self.slope(window)) < tol
    def improving(self, window: int = 0) -> bool: return self.slope(window) < 0.0

    def converged(self, window: int, tol: float) -> bool:
        d = self._window(window)
        if len(d) < 2:
            return False
        m = sum(d) / len(d)
        return sum((v - m) ** 2 for v in d) / len(d) < tol


class TrendGroup:
    def __init__(self, trends: Sequence[Trend]): self.trends = list(trends)
    def __len__(self): return len(self.trends)
    def len(self): return len(self.trends)
    def is_empty(self): return not self.trends
    def all_improving(self, w=0): return bool(self.trends) and all(t.improving(w) for t in self.trends)
    def any_improving(self, w=0): return any(t.improving(w) for t in self.trends)
    def all_stalled(self, w, tol): return bool(self.trends) and all(t.stalled(w, tol) for t in self.trends)
    def any_stalled(self, w, tol): return any(t.stalled(w, tol) for t in self.trends)
    def all_converged(self, w, tol): return bool(self.trends) and all(t.converged(w, tol) for t in self.trends)
    def any_converged(self, w, tol): return any(t.converged(w, tol) for t in self.trends)
    def mean_slope(self, w=0): return sum(t.slope(w) for t in self.trends) / len(self.trends) if self.trends else 0.0
    def slopes(self, w=0): return [t.slope(w) for t in self.trends]
