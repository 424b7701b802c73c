"""`Timeline`: a background sampler (CPU, RAM, per-GPU utilisation / memory) plus training events
on one clock, for finding idle gaps and synchronisation cost
(flodl/src/monitor/timeline.rs).

Events are injected by the DDP coordinator and workers (`SyncStart`, `SyncEnd{duration_ms}`,
`CpuAvgStart/End`, `AnchorChanged{from,to}`, `Throttle{rank}`, `EpochStart/End`) or by the user
(`Custom`). `subscribe()` returns a queue that receives batches of new samples/events.
"""
from __future__ import annotations

import csv
import json
import queue
import threading
import time
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

from .resources import ResourceSampler

EVENT_KINDS = ("EpochStart", "EpochEnd", "SyncStart", "SyncEnd", "CpuAvgStart", "CpuAvgEnd", "AnchorChanged", "Throttle", "Idle",
               "Custom")


class EventKind:
    """One of the event variants, with its fields: `EventKind.SyncEnd(duration_ms=3.1)`,
    `EventKind.AnchorChanged(8, 12)`, `EventKind.Custom("eval")` (flodl/src/monitor/timeline.rs:77-98).
    `Timeline.event` takes one of these, or the kind's name and the fields as keywords."""

    def __init__(self, kind: str, **fields):
        if kind not in EVENT_KINDS:
            raise ValueError(f"unknown timeline event kind {kind!r}")
        self.kind, self.fields = kind, fields

    def __repr__(self) -> str:
        return f"EventKind.{self.kind}({', '.join(f'{k}={v!r}' for k, v in self.fields.items())})"

    def __eq__(self, other) -> bool:
        return isinstance(other, EventKind) and (self.kind, self.fields) == (other.kind, other.fields)

    @classmethod
    def EpochStart(cls, epoch: int): return cls("EpochStart", epoch=int(epoch))
    @classmethod
    def EpochEnd(cls, epoch: int, loss: float): return cls("EpochEnd", epoch=int(epoch), loss=float(loss))
    @classmethod
    def SyncStart(cls): return cls("SyncStart")
    @classmethod
    def SyncEnd(cls, duration_ms: float): return cls("SyncEnd", duration_ms=float(duration_ms))
    @classmethod
    def CpuAvgStart(cls): return cls("CpuAvgStart")
    @classmethod
    def CpuAvgEnd(cls, duration_ms: float): return cls("CpuAvgEnd", duration_ms=float(duration_ms))
    @classmethod
    def AnchorChanged(cls, from_: int, to: int): return cls("AnchorChanged", **{"from": int(from_), "to": int(to)})
    @classmethod
    def Throttle(cls, rank: int): return cls("Throttle", rank=int(rank))
    @classmethod
    def Idle(cls, device: int, duration_ms: float): return cls("Idle", device=int(device), duration_ms=float(duration_ms))
    @classmethod
    def Custom(cls, label: str): return cls("Custom", label=str(label))


@dataclass
class GpuTimelineSample:
    """One GPU inside a `TimelineSample` (timeline.rs:36-49); `TimelineSample.gpu_samples()` gives these."""
    device: int
    compute_util: Optional[float]
    vram_used_bytes: Optional[int]
    vram_allocated_bytes: Optional[int]
    vram_total_bytes: Optional[int] = None
    sm_mhz: Optional[int] = None
    power_w: Optional[float] = None


@dataclass
class TimelineBroadcast:
    """What a subscriber's queue receives every broadcast interval: the samples and events since the last one,
    as dicts ready for JSON (timeline.rs:125-132). Indexable by "samples" / "events" as well."""
    samples: List[dict]
    events: List[dict]

    def __getitem__(self, key: str):
        return getattr(self, key)


@dataclass
class TimelineEvent:
    t_ms: int
    kind: str
    fields: Dict[str, object] = field(default_factory=dict)

    def to_dict(self) -> dict:
        return {"t_ms": self.t_ms, "kind": self.kind, **self.fields}


@dataclass
class TimelineSample:
    t_ms: int
    cpu_percent: Optional[float]
    ram_used_bytes: Optional[int]
    gpus: List[dict]

    def to_dict(self) -> dict:
        return {"t_ms": self.t_ms, "cpu_percent": self.cpu_percent, "ram_used_bytes": self.ram_used_bytes, "gpus": self.gpus}

    def gpu_samples(self) -> List[GpuTimelineSample]:
        return [GpuTimelineSample(g.get("index"), g.get("util"), g.get("vram_used"), g.get("vram_allocated"), g.get("vram_total"),
                                  g.get("sm_mhz"), g.get("power_w")) for g in self.gpus]


@dataclass
class TimelineSummary:
    duration_ms: int
    samples: int
    events: int
    sync_count: int
    sync_total_ms: float
    cpu_avg_count: int
    cpu_avg_total_ms: float
    throttle_count: int
    anchor_changes: int
    gpu_mean_util: Dict[int, float]
    gpu_idle_ms: Dict[int, int]

    def __str__(self) -> str:
        util = ", ".join(f"GPU{i} {u:.0f}%" for i, u in sorted(self.gpu_mean_util.items()))
        return (f"timeline: {self.duration_ms / 1000:.1f}s, {self.samples} samples, {self.sync_count} syncs "
                f"({self.sync_total_ms:.0f} ms), {self.throttle_count} throttles, {self.anchor_changes} anchor changes; {util}")


class Timeline:
    def __init__(self, poll_interval_ms: int = 100, broadcast_interval_ms: int = 1000, sampler: Optional[ResourceSampler] = None):
        self.poll_s = max(0.001, poll_interval_ms / 1000.0)
        self.broadcast_s = max(self.poll_s, broadcast_interval_ms / 1000.0)
        self._sampler = sampler
        self._t0 = time.monotonic()
        self._samples: List[TimelineSample] = []
        self._events: List[TimelineEvent] = []
        self._lock = threading.Lock()
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None
        self._subs: List[queue.Queue] = []
        self._sent = (0, 0)

    @classmethod
    def new(cls, poll_interval_ms: int = 100) -> "Timeline":
        return cls(poll_interval_ms)

    @classmethod
    def with_intervals(cls, poll_interval_ms: int, broadcast_interval_ms: int) -> "Timeline":
        return cls(poll_interval_ms, broadcast_interval_ms)

    # ---- lifecycle ----------------------------------------------------------------------------
    def start(self) -> None:
        if self._thread is not None:
            return
        if self._sampler is None:
            self._sampler = ResourceSampler()
        self._stop.clear()
        self._thread = threading.Thread(target=self._run, name="timeline", daemon=True)
        self._thread.start()

    def stop(self) -> None:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=5)
            self._thread = None
        self._broadcast()

    def _run(self) -> None:
        last_b = time.monotonic()
        while not self._stop.wait(self.poll_s):
            self.sample_once()
            if time.monotonic() - last_b >= self.broadcast_s:
                self._broadcast()
                last_b = time.monotonic()

    def sample_once(self) -> None:
        if self._sampler is None:
            self._sampler = ResourceSampler()
        r = self._sampler.sample()
        s = TimelineSample(self.elapsed_ms(), r.cpu_percent, r.ram_used_bytes,
                           [dict(index=g.index, util=g.util_percent, vram_used=g.vram_used_bytes, vram_allocated=g.vram_allocated_bytes,
                                 sm_mhz=g.sm_clock_mhz, power_w=g.power_w) for g in r.gpus])
        with self._lock:
            self._samples.append(s)

    # ---- events -------------------------------------------------------------------------------
    def event(self, kind, **fields) -> None:
        if isinstance(kind, EventKind):
            kind, fields = kind.kind, {**kind.fields, **fields}
        ev = TimelineEvent(self.elapsed_ms(), kind, fields)
        with self._lock:
            self._events.append(ev)

    def elapsed_ms(self) -> int:
        return int((time.monotonic() - self._t0) * 1000)

    # ---- subscribers --------------------------------------------------------------------------
    def subscribe(self) -> "queue.Queue":
        q: queue.Queue = queue.Queue()
        with self._lock:
            self._subs.append(q)
        return q

    def _broadcast(self) -> None:
        with self._lock:
            a, b = self._sent
            new_s, new_e = self._samples[a:], self._events[b:]
            self._sent = (len(self._samples), len(self._events))
            subs = list(self._subs)
        if not (new_s or new_e):
            return
        msg = TimelineBroadcast([s.to_dict() for s in new_s], [e.to_dict() for e in new_e])
        for q in subs:
            q.put(msg)

    # ---- analysis -----------------------------------------------------------------------------
    def idle_gaps(self, device: int, threshold_pct: float = 5.0, min_ms: int = 500) -> List[Tuple[int, int]]:
        """Intervals (start_ms, end_ms) during which `device` stayed at or below `threshold_pct`
        utilisation for at least `min_ms`."""
        with self._lock:
            samples = list(self._samples)
        gaps, start, last = [], None, None
        for s in samples:
            g = next((g for g in s.gpus if g["index"] == device), None)
            if g is None or g["util"] is None:
                continue
            if g["util"] <= threshold_pct:
                if start is None:
                    start = s.t_ms
                last = s.t_ms
            else:
                if start is not None and last - start >= min_ms:
                    gaps.append((start, last))
                start = None
        if start is not None and last - start >= min_ms:
            gaps.append((start, last))
        return gaps

    def summary(self) -> TimelineSummary:
        with self._lock:
            samples, events = list(self._samples), list(self._events)
        sync = [e for e in events if e.kind == "SyncEnd"]
        cavg = [e for e in events if e.kind == "CpuAvgEnd"]
        util: Dict[int, List[float]] = {}
        for s in samples:
            for g in s.gpus:
                if g["util"] is not None:
                    util.setdefault(g["index"], []).append(g["util"])
        idle = {i: sum(b - a for a, b in self.idle_gaps(i)) for i in util}
        dur = max([s.t_ms for s in samples] + [e.t_ms for e in events] + [0])
        return TimelineSummary(dur, len(samples), len(events), len(sync), sum(float(e.fields.get("duration_ms", 0.0)) for e in sync),
                               len(cavg), sum(float(e.fields.get("duration_ms", 0.0)) for e in cavg),
                               sum(1 for e in events if e.kind == "Throttle"), sum(1 for e in events if e.kind == "AnchorChanged"),
                               {i: sum(v) / len(v) for i, v in util.items()}, idle)

    def drain(self):
        with self._lock:
            s, e = self._samples, self._events
            self._samples, self._events = [], []
            self._sent = (0, 0)
        return s, e

    def sample_count(self) -> int:
        with self._lock:
            return len(self._samples)

    def events(self) -> List[TimelineEvent]:
        with self._lock:
            return list(self._events)

    # ---- export -------------------------------------------------------------------------------
    def to_dict(self) -> dict:
        with self._lock:
            return {"samples": [s.to_dict() for s in self._samples], "events": [e.to_dict() for e in self._events]}

    def save_json(self, path: str) -> None:
        with open(path, "w") as f:
            json.dump(self.to_dict(), f)

    def save_csv(self, path: str) -> None:
        with self._lock:
            samples, events = list(self._samples), list(self._events)
        with open(path, "w", newline="") as f:
            w = csv.writer(f)
            w.writerow(["t_ms", "type", "cpu_percent", "ram_used_bytes", "gpu", "gpu_util", "vram_used", "event", "detail"])
            for s in samples:
                if not s.gpus:
                    w.writerow([s.t_ms, "sample", s.cpu_percent, s.ram_used_bytes, "", "", "", "", ""])
                for g in s.gpus:
                    w.writerow([s.t_ms, "sample", s.cpu_percent, s.ram_used_bytes, g["index"], g["util"], g["vram_used"], "", ""])
            for e in events:
                w.writerow([e.t_ms, "event", "", "", "", "", "", e.kind, json.dumps(e.fields)])

    def save_html(self, path: str) -> None:
        from .html import timeline_html
        with open(path, "w") as f:
            f.write(timeline_html(self.to_dict()))
