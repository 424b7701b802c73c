"""Weight-space divergence guard for periodic parameter averaging
(flodl/src/distributed/ddp_run/convergence.rs).

Signal: per rank, ||params_before_sync - params_after_sync|| / ||params_after_sync||. With the
norms before and after, the same three numbers also give the cosine between a replica and the
consensus and the magnitude shift.
"""
from __future__ import annotations

import math
from collections import deque
from dataclasses import dataclass
from typing import List, Optional

from ... import log
from .messages import ApplyPolicy


@dataclass
class DivergenceReport:
    deltas: List[float]
    pre_norms: Optional[List[float]] = None
    post_norm: Optional[float] = None

    def max_relative_delta(self) -> float:
        return max(self.deltas, default=0.0) if self.deltas else 0.0

    def cosine_similarities(self) -> Optional[List[float]]:
        if self.pre_norms is None or self.post_norm is None or self.post_norm < 1e-10:
            return None
        out = []
        for delta, pre in zip(self.deltas, self.pre_norms):
            if pre < 1e-10:
                out.append(0.0)
                continue
            diff_sq = (delta * self.post_norm) ** 2
            c = (pre * pre + self.post_norm ** 2 - diff_sq) / (2.0 * pre * self.post_norm)
            out.append(max(-1.0, min(1.0, c)))
        return out

    def magnitude_shifts(self) -> Optional[List[float]]:
        if self.pre_norms is None or self.post_norm is None:
            return None
        return [p - self.post_norm for p in self.pre_norms]


@dataclass(frozen=True)
class ConvergenceAction:
    """`kind`: Stable | SuppressGrowth | NudgeDown (with `factor`)."""
    kind: str
    factor: float = 1.0

    @staticmethod
    def Stable(): return ConvergenceAction("Stable")
    @staticmethod
    def SuppressGrowth(): return ConvergenceAction("SuppressGrowth")
    @staticmethod
    def NudgeDown(factor: float): return ConvergenceAction("NudgeDown", float(factor))


class ConvergenceGuard:
    """Keeps the last five divergences. `Sync` never acts; `Cadence`/`Async` suppress anchor growth
    when the last three values rise strictly and the newest exceeds `threshold`."""

    @classmethod
    def new(cls, *args, **kw):
        return cls(*args, **kw)

    def __init__(self, policy: ApplyPolicy, enabled: bool = True, threshold: float = 0.05):
        self.policy, self.enabled, self.threshold = policy, bool(enabled), float(threshold)
        self._history: deque = deque(maxlen=5)

    def report(self, report: DivergenceReport) -> ConvergenceAction:
        if not self.enabled:
            return ConvergenceAction.Stable()
        d = report.max_relative_delta()
        if math.isnan(d):
            d = 0.0
        self._history.append(d)
        if self.policy == ApplyPolicy.Sync:
            return ConvergenceAction.Stable()
        return self._check_trend()

    def _check_trend(self) -> ConvergenceAction:
        h = self._history
        if len(h) < 3:
            return ConvergenceAction.Stable()
        if h[-1] > h[-2] > h[-3] and h[-1] > self.threshold:
            log.verbose(f"  ddp: weight-space divergence trending up | history={[round(x, 4) for x in h]} | suppressing growth")
            return ConvergenceAction.SuppressGrowth()
        return ConvergenceAction.Stable()

    def history(self) -> List[float]:
        return list(self._history)
