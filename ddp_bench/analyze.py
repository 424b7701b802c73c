"""What a run's timeline says about it (ddp-bench/src/analyze.rs): how often and how long the replicas synchronised,
how the El Che anchor moved, how busy every GPU was, and where the idle stretches came from.

A timeline is the JSON that `Timeline.save_json` writes: `samples` (every 100 ms: CPU %, RAM, per GPU utilisation and
memory) and `events` (`EpochStart/End`, `SyncStart/End{duration_ms}`, `CpuAvgStart/End{duration_ms}`,
`AnchorChanged{from,to}`, `Throttle{rank}`), all on one millisecond clock."""
from __future__ import annotations

import glob
import json
import os
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

IDLE_UTIL_PCT = 5.0          # a sample below this utilisation counts as idle
IDLE_MIN_MS = 500            # shorter idle stretches are not reported
NEAR_MS = 500                # an event this close to a gap explains it


@dataclass
class IdleGap:
    gpu: int
    start_ms: int
    duration_ms: int
    cause: str               # "epoch boundary", "sync", "cpu avg", "unexplained"


@dataclass
class RunAnalysis:
    model: str
    mode: str
    total_ms: int = 0
    sample_count: int = 0
    sync_count: int = 0
    avg_sync_ms: float = 0.0
    sync_interval_p50_ms: float = 0.0
    sync_interval_p95_ms: float = 0.0
    cpu_avg_count: int = 0
    avg_cpu_avg_ms: float = 0.0
    anchor_changes: List[Tuple[int, int]] = field(default_factory=list)
    final_anchor: Optional[int] = None
    throttle_count: int = 0
    gpu_mean_util: Dict[int, float] = field(default_factory=dict)
    gpu_peak_vram_mb: Dict[int, float] = field(default_factory=dict)
    gpu_mean_vram_mb: Dict[int, float] = field(default_factory=dict)
    idle_gaps: List[IdleGap] = field(default_factory=list)
    epoch_losses: List[float] = field(default_factory=list)

    def idle_ms(self, gpu: Optional[int] = None) -> int:
        return sum(g.duration_ms for g in self.idle_gaps if gpu is None or g.gpu == gpu)

    def idle_by_cause(self, gpu: int) -> Dict[str, int]:
        out = {"epoch boundary": 0, "sync": 0, "cpu avg": 0, "unexplained": 0}
        for g in self.idle_gaps:
            if g.gpu == gpu:
                out[g.cause] += g.duration_ms
        return out


def load_timeline(path: str) -> dict:
    try:
        data = json.load(open(path))
    except OSError as e:
        raise ValueError(f"cannot read {path}: {e}")
    except ValueError as e:
        raise ValueError(f"invalid JSON in {path}: {e}")
    if not isinstance(data, dict) or "events" not in data or "samples" not in data:
        raise ValueError(f"{path}: not a timeline (expected `samples` and `events`)")
    return data


def empty_analysis(model: str, mode: str) -> RunAnalysis:
    """For a run that left no timeline: the report shows dashes instead of dropping the row."""
    return RunAnalysis(model, mode)


def _percentile(values: List[float], q: float) -> float:
    if not values:
        return 0.0
    v = sorted(values)
    k = (len(v) - 1) * q
    lo, hi = int(k), min(int(k) + 1, len(v) - 1)
    return v[lo] + (v[hi] - v[lo]) * (k - lo)


_CAUSES = (("epoch boundary", ("EpochStart", "EpochEnd")), ("sync", ("SyncStart", "SyncEnd")), ("cpu avg", ("CpuAvgStart", "CpuAvgEnd")))


def classify_gap(start_ms: int, end_ms: int, events: List[dict]) -> str:
    """The kind of event nearest to an idle stretch (inside it, or within half a second of either end)."""
    best, best_d = "unexplained", None
    for cause, kinds in _CAUSES:
        for e in events:
            if e.get("kind") not in kinds:
                continue
            t = e["t_ms"]
            d = 0 if start_ms <= t <= end_ms else min(abs(t - start_ms), abs(t - end_ms))
            if d <= NEAR_MS and (best_d is None or d < best_d):
                best, best_d = cause, d
    return best


def idle_gaps(samples: List[dict], events: List[dict], gpu: int) -> List[IdleGap]:
    out: List[IdleGap] = []
    start = last = None
    for s in samples:
        g = next((x for x in s.get("gpus", []) if x.get("index") == gpu), None)
        util = None if g is None else g.get("util")
        if util is not None and util < IDLE_UTIL_PCT:
            start = s["t_ms"] if start is None else start
            last = s["t_ms"]
            continue
        if start is not None and last - start >= IDLE_MIN_MS:
            out.append(IdleGap(gpu, start, last - start, classify_gap(start, last, events)))
        start = last = None
    if start is not None and last - start >= IDLE_MIN_MS:
        out.append(IdleGap(gpu, start, last - start, classify_gap(start, last, events)))
    return out


def analyze(model: str, mode: str, tl: dict) -> RunAnalysis:
    samples, events = tl.get("samples", []), tl.get("events", [])
    a = RunAnalysis(model, mode, sample_count=len(samples))
    times = [x["t_ms"] for x in samples] + [x["t_ms"] for x in events]
    a.total_ms = max(times) - min(times) if times else 0
    sync_ends = [e for e in events if e.get("kind") == "SyncEnd"]
    sync_starts = [e["t_ms"] for e in events if e.get("kind") == "SyncStart"]
    a.sync_count = len(sync_starts) or len(sync_ends)
    durs = [float(e["duration_ms"]) for e in sync_ends if e.get("duration_ms") is not None]
    a.avg_sync_ms = sum(durs) / len(durs) if durs else 0.0
    marks = sync_starts or [e["t_ms"] for e in sync_ends]
    gaps = [b - c for b, c in zip(marks[1:], marks[:-1])]
    a.sync_interval_p50_ms, a.sync_interval_p95_ms = _percentile(gaps, 0.5), _percentile(gaps, 0.95)
    cpu = [float(e["duration_ms"]) for e in events if e.get("kind") == "CpuAvgEnd" and e.get("duration_ms") is not None]
    a.cpu_avg_count = sum(1 for e in events if e.get("kind") == "CpuAvgStart") or len(cpu)
    a.avg_cpu_avg_ms = sum(cpu) / len(cpu) if cpu else 0.0
    a.anchor_changes = [(int(e["from"]), int(e["to"])) for e in events if e.get("kind") == "AnchorChanged"]
    a.final_anchor = a.anchor_changes[-1][1] if a.anchor_changes else None
    a.throttle_count = sum(1 for e in events if e.get("kind") == "Throttle")
    a.epoch_losses = [float(e["loss"]) for e in events if e.get("kind") == "EpochEnd" and e.get("loss") is not None]
    gpus = sorted({g["index"] for s in samples for g in s.get("gpus", []) if g.get("index") is not None})
    for i in gpus:
        rows = [g for s in samples for g in s.get("gpus", []) if g.get("index") == i]
        utils = [g["util"] for g in rows if g.get("util") is not None]
        vram = [g["vram_used"] / 2 ** 20 for g in rows if g.get("vram_used") is not None]
        if utils:
            a.gpu_mean_util[i] = sum(utils) / len(utils)
        if vram:
            a.gpu_peak_vram_mb[i], a.gpu_mean_vram_mb[i] = max(vram), sum(vram) / len(vram)
        a.idle_gaps += idle_gaps(samples, events, i)
    return a


def discover_runs(output_dir: str) -> List[Tuple[str, str]]:
    """(model, mode) of every result file in a directory, in name order."""
    out = []
    for path in sorted(glob.glob(os.path.join(output_dir, "*__*.json"))):
        name = os.path.basename(path)
        if name.endswith(".timeline.json"):
            continue
        model, _, mode = name[:-5].partition("__")
        out.append((model, mode))
    return out


def analyze_dir(output_dir: str) -> Dict[Tuple[str, str], RunAnalysis]:
    out = {}
    for model, mode in discover_runs(output_dir):
        path = os.path.join(output_dir, f"{model}__{mode}.timeline.json")
        try:
            out[(model, mode)] = analyze(model, mode, load_timeline(path))
        except ValueError:
            out[(model, mode)] = empty_analysis(model, mode)
    return out
