"""El Che: the cadence controller for replicas of unequal speed.

The slowest replica anchors the cadence (`anchor` batches between two synchronisations); every
other replica runs `anchor * slow_ms / own_ms` batches in the same wall time. After each
synchronisation `report_timing` refines the per-rank milliseconds-per-batch estimate (adaptive
EMA), re-derives the batch counts (10 % dead zone) and tunes the anchor so that the
synchronisation costs about `overhead_target` of the compute time. Same behaviour as the
reference's `ElChe` (flodl/src/distributed/el_che.rs:35-384); the arithmetic lives in the C++
runtime (`csrc/runtime/runtime.cpp`), this class is the builder-style front.
"""
from __future__ import annotations

from typing import List, Optional, Sequence

from .. import _ext


class ElChe:
    def __init__(self, world_size: int, anchor: int):
        if world_size < 1:
            raise ValueError("ElChe: world_size must be >= 1")
        self._c = _ext.require().ElChe(int(world_size), max(1, int(anchor)))
        self.world_size = int(world_size)

    @classmethod
    def new(cls, world_size: int, anchor: int) -> "ElChe":
        return cls(world_size, anchor)

    # ---- builder ------------------------------------------------------------------------------
    def with_overhead_target(self, target: float) -> "ElChe":
        self._c.set_overhead_target(float(target))
        return self

    def with_max_anchor(self, max_anchor: int) -> "ElChe":
        self._c.set_max_anchor(int(max_anchor))
        return self

    def with_max_batch_diff(self, max_diff: int) -> "ElChe":
        self._c.set_max_batch_diff(int(max_diff))
        return self

    def with_speed_ratio(self, slow_rank: int, ratio: float) -> "ElChe":
        self._c.set_speed_ratio(int(slow_rank), float(ratio))
        return self

    # ---- queries ------------------------------------------------------------------------------
    def batches(self, rank: int) -> int:
        return self._c.batches(rank)

    def batch_counts(self) -> List[int]:
        return list(self._c.batch_counts())

    def total_batches(self) -> int:
        return self._c.total_batches()

    def anchor(self) -> int:
        return self._c.anchor()

    def anchor_wall_ms(self) -> float:
        return self._c.anchor_wall_ms()

    def is_calibrated(self) -> bool:
        return self._c.is_calibrated()

    def has_speed_hint(self) -> bool:
        return self._c.has_speed_hint()

    def ms_per_batch(self) -> List[float]:
        return list(self._c.ms_per_batch())

    def max_batch_diff(self) -> Optional[int]:
        return self._c.max_batch_diff()

    def clamp_total(self, max_total: int) -> List[int]:
        return list(self._c.clamp_total(int(max_total)))

    # ---- feedback -----------------------------------------------------------------------------
    def report_timing(self, wall_ms: Sequence[float], actual_batches: Sequence[int], sync_ms: float) -> None:
        self._c.report_timing([float(x) for x in wall_ms], [int(x) for x in actual_batches], float(sync_ms))

    def nudge_anchor_down(self, factor: float) -> None:
        self._c.nudge_anchor_down(float(factor))
