"""Per-node / per-level wall-clock profiling of `Graph.forward` (flodl/src/graph/profile.rs,
graph.rs:454-468, :538-549). Host timers, no device sync: this measures launch + blocking time,
exactly as the reference does; device time is what `flodl_b200.monitor.Timeline` and CUDA events
are for."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional

from .trend import Trend


@dataclass
class NodeTiming:
    id: str
    tag: str
    duration: float
    level: int


@dataclass
class LevelTiming:
    index: int
    wall_clock: float
    sum_nodes: float
    num_nodes: int

    def parallelism(self) -> float:
        return self.sum_nodes / self.wall_clock if self.wall_clock > 0 else 1.0


@dataclass
class Profile:
    total: float
    levels: List[LevelTiming] = field(default_factory=list)
    nodes: List[NodeTiming] = field(default_factory=list)

    def timing(self, tag_or_id: str) -> Optional[float]:
        for n in self.nodes:
            if n.tag == tag_or_id or n.id == tag_or_id:
                return n.duration
        return None

    def __str__(self) -> str:
        lines = [f"forward: {self.total * 1e3:.3f} ms"]
        for lv in self.levels:
            lines.append(f"  level {lv.index}: {lv.wall_clock * 1e3:.3f} ms ({lv.num_nodes} nodes)")
        for n in sorted(self.nodes, key=lambda n: -n.duration)[:10]:
            lines.append(f"    {n.tag or n.id}: {n.duration * 1e3:.3f} ms")
        return "\n".join(lines)


class ProfileMixin:
    def _init_profile(self) -> None:
        self._profiling = False
        self.last_profile: Optional[Profile] = None
        self.timing_buffer: Dict[str, List[float]] = {}
        self.timing_history: Dict[str, List[float]] = {}

    def enable_profiling(self) -> None: self._profiling = True
    def disable_profiling(self) -> None: self._profiling = False
    def profiling(self) -> bool: return self._profiling
    def profile(self) -> Optional[Profile]: return self.last_profile

    def _store_profile(self, total, levels, nodes) -> None:
        self.last_profile = Profile(total, [LevelTiming(*l) for l in levels], [NodeTiming(*n) for n in nodes])

    def timing(self, tag: str) -> Optional[float]:
        return self.last_profile.timing(tag) if self.last_profile else None

    def parallelism(self) -> float:
        p = self.last_profile
        if not p or not p.levels:
            return 1.0
        wall = sum(l.wall_clock for l in p.levels)
        return sum(l.sum_nodes for l in p.levels) / wall if wall > 0 else 1.0

    def collect_timings(self, tags=()) -> None:
        """Append the last profile's node durations (tagged nodes; all if `tags` is empty) to the timing buffers."""
        if not self.last_profile:
            return
        for n in self.last_profile.nodes:
            key = n.tag or n.id
            if tags and key not in tags:
                continue
            self.timing_buffer.setdefault(key, []).append(n.duration)

    def flush_timings(self, tags=()) -> None:
        keys = list(tags) if tags else list(self.timing_buffer.keys())
        for k in keys:
            vals = self.timing_buffer.pop(k, None)
            if vals:
                self.timing_history.setdefault(k, []).append(sum(vals) / len(vals))

    def timing_trend(self, tag: str) -> Trend:
        return Trend(self.timing_history.get(tag, []))

    def timing_trends(self, tags) -> List[Trend]:
        return [self.timing_trend(t) for t in tags]

    def reset_timing_trend(self, tags=()) -> None:
        if not tags:
            self.timing_history.clear()
        else:
            for t in tags:
                self.timing_history.pop(t, None)
