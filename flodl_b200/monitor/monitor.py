"""`Monitor`: one line per epoch with an adaptive ETA and a resource sample, an optional live
dashboard (HTTP + server-sent events), and HTML / CSV / log exports
(flodl/src/monitor/mod.rs:187-600)."""
from __future__ import annotations

import csv
import json
import time
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple, Union

from .. import log
from .format import format_bytes, format_eta, format_metric
from .html import dashboard_html
from .resources import ResourceSample, ResourceSampler
from .server import DashboardServer


@dataclass
class GpuMetrics:
    """Per-device figures of one epoch in a multi-GPU run (shown as separate dashboard rows)."""
    device: int
    throughput: float = 0.0
    batch_share: float = 0.0
    scalars: Dict[str, float] = field(default_factory=dict)


@dataclass
class EpochRecord:
    epoch: int
    duration_secs: float
    metrics: List[Tuple[str, float]]
    resources: ResourceSample
    gpu_metrics: List[GpuMetrics] = field(default_factory=list)


class Metrics:
    """What `Monitor.log` takes as its `metrics` argument (flodl/src/monitor/mod.rs:68-125): a list of
    `(name, value)` pairs, a dict, a `Graph` (the latest flushed epoch of its observed tags, plus the per-GPU
    shares of a distributed graph), a `(graph, extra_pairs)` tuple, a DDP `EpochMetrics`, or any object
    that implements this interface."""

    def into_metrics(self) -> List[Tuple[str, float]]:
        raise NotImplementedError

    def gpu_metrics(self) -> List["GpuMetrics"]:
        return []


def _graph_gpu_metrics(graph) -> List["GpuMetrics"]:
    if not (hasattr(graph, "is_distributed") and graph.is_distributed()):
        return []
    ratios, tp, shards = graph.chunk_ratios(), graph.throughput(), graph.shard_sizes()
    out = []
    for i, dev in enumerate(graph.devices()):
        idx = getattr(dev, "index", None)
        out.append(GpuMetrics(i if idx is None else int(idx), float(tp[i]) if i < len(tp) else 0.0, float(ratios[i]) if i < len(ratios) else 0.0,
                              {"shard_size": float(shards[i])} if i < len(shards) else {}))
    return out


def _metric_pairs(metrics) -> Tuple[List[Tuple[str, float]], List[GpuMetrics]]:
    """Normalise the accepted forms (see `Metrics`) to (pairs, per-GPU rows)."""
    if isinstance(metrics, tuple) and len(metrics) == 2 and hasattr(metrics[0], "latest_metrics"):
        pairs, gm = _metric_pairs(metrics[0])
        extra, _ = _metric_pairs(metrics[1])
        return pairs + extra, gm
    if hasattr(metrics, "latest_metrics"):
        return [(k, float(v)) for k, v in metrics.latest_metrics()], _graph_gpu_metrics(metrics)
    if hasattr(metrics, "into_metrics"):
        gm = metrics.gpu_metrics() if hasattr(metrics, "gpu_metrics") else []
        return [(k, float(v)) for k, v in metrics.into_metrics()], list(gm)
    if hasattr(metrics, "scalars") and hasattr(metrics, "avg_loss"):
        pairs = [("loss", float(metrics.avg_loss))] + [(k, float(v)) for k, v in sorted(metrics.scalars.items()) if k != "loss"]
        gm = [GpuMetrics(dev, tp, sh, dict(sc)) for dev, tp, sh, sc in
              zip(metrics.device_indices, metrics.per_rank_throughput, metrics.per_rank_batch_share, metrics.per_rank)]
        return pairs, gm
    if isinstance(metrics, dict):
        return [(k, float(v)) for k, v in metrics.items()], []
    return [(k, float(v)) for k, v in metrics], []


class Monitor:
    def __init__(self, total_epochs: int, sampler: Optional[ResourceSampler] = None):
        self.total_epochs = int(total_epochs)
        self.epochs: List[EpochRecord] = []
        self.start_time = time.monotonic()
        self.sampler = sampler or ResourceSampler()
        self.server: Optional[DashboardServer] = None
        self._svg: Optional[str] = None
        self._label: Optional[str] = None
        self._hash: Optional[str] = None
        self._metadata = None
        self._html_path: Optional[str] = None
        self._hardware = self._hardware_summary()

    @classmethod
    def new(cls, total_epochs: int) -> "Monitor":
        return cls(total_epochs)

    @staticmethod
    def _hardware_summary() -> str:
        try:
            from ..tensor import hardware_summary
            return hardware_summary()
        except Exception:
            return ""

    # ---- dashboard ------------------------------------------------------------------------------
    def serve(self, port: int) -> int:
        """Start the live dashboard on `port` (0 = any free port); returns the port in use."""
        self.server = DashboardServer(port, lambda: dashboard_html(self._state(), live=True))
        self.server.set_hardware(self._hardware)
        if self._svg:
            self.server.set_svg(self._svg)
        self.server.set_label_hash(self._label, self._hash)
        if self._metadata is not None:
            self.server.set_metadata(self._metadata)
        log.msg(f"  monitor: http://127.0.0.1:{self.server.port}")
        return self.server.port

    def save_html(self, path: str) -> None:
        """Write the dashboard to `path` at `finish()` (and right now if epochs exist)."""
        self._html_path = path
        if self.epochs:
            self._write_html()

    def set_metadata(self, meta) -> None:
        self._metadata = meta
        if self.server:
            self.server.set_metadata(meta)

    def watch(self, graph) -> None:
        """Show the graph's picture and identity on the dashboard."""
        try:
            svg = graph.svg()
            self.set_svg(svg.decode() if isinstance(svg, (bytes, bytearray)) else svg)
        except Exception:
            pass
        self.set_identity(graph.label(), graph.structural_hash())

    def watch_profiled(self, graph) -> None:
        try:
            svg = graph.svg_with_profile()
            self.set_svg(svg.decode() if isinstance(svg, (bytes, bytearray)) else svg)
        except Exception:
            self.watch(graph)
            return
        self.set_identity(graph.label(), graph.structural_hash())

    def set_svg(self, svg: str) -> None:
        self._svg = svg
        if self.server:
            self.server.set_svg(svg)

    set_architecture_svg = set_svg

    def set_identity(self, label: Optional[str], hash_: Optional[str]) -> None:
        self._label, self._hash = label, hash_
        if self.server:
            self.server.set_label_hash(label, hash_)

    # ---- per epoch ------------------------------------------------------------------------------
    def log(self, epoch: int, duration: Union[float, "object"], metrics) -> str:
        """Record epoch `epoch` (0-based), print its line, push it to the dashboard; returns the line."""
        secs = float(duration.total_seconds()) if hasattr(duration, "total_seconds") else float(duration)
        pairs, gpu_metrics = _metric_pairs(metrics)
        res = self.sampler.sample()
        self.epochs.append(EpochRecord(epoch, secs, pairs, res, gpu_metrics))
        shown = epoch + 1
        width = len(str(self.total_epochs))
        line = f"  epoch {shown:>{width}}/{self.total_epochs}"
        for name, val in pairs:
            line += f"  {name}={format_metric(val)}"
        line += f"  [{format_eta(secs)}"
        if shown < self.total_epochs:
            elapsed = time.monotonic() - self.start_time
            line += f"  ETA {format_eta(elapsed / shown * (self.total_epochs - shown))}"
        line += "]"
        if res.vram_allocated_bytes is not None:
            spill = max(0, res.vram_allocated_bytes - (res.vram_total_bytes or res.vram_allocated_bytes))
            line += f"  VRAM: {format_bytes(res.vram_allocated_bytes)} / {format_bytes(spill)}"
        if res.gpu_util_percent is not None:
            line += f" ({res.gpu_util_percent:.0f}%)"
        log.msg(line)
        if self.server:
            self.server.push_epoch(json.dumps(self._epoch_dict(self.epochs[-1])))
        return line

    def finish(self) -> None:
        total = time.monotonic() - self.start_time
        log.msg(f"  training complete: {len(self.epochs)} epochs in {format_eta(total)}")
        if self._html_path:
            self._write_html()

    def finish_with(self, graph) -> None:
        self.watch_profiled(graph) if getattr(graph, "profiling", lambda: False)() else self.watch(graph)
        self.finish()

    def history(self) -> List[EpochRecord]:
        return self.epochs

    # ---- export ---------------------------------------------------------------------------------
    def _epoch_dict(self, e: EpochRecord) -> dict:
        return {"epoch": e.epoch, "duration_secs": e.duration_secs, "metrics": dict(e.metrics), "resources": e.resources.to_dict(),
                "gpu_metrics": [g.__dict__ for g in e.gpu_metrics]}

    def _state(self) -> dict:
        return {"total_epochs": self.total_epochs, "epochs": [self._epoch_dict(e) for e in self.epochs], "svg": self._svg,
                "label": self._label, "hash": self._hash, "hardware": self._hardware, "metadata": self._metadata}

    def _write_html(self) -> None:
        with open(self._html_path, "w") as f:
            f.write(dashboard_html(self._state(), live=False))

    def write_log(self, path: str) -> None:
        with open(path, "w") as f:
            for e in self.epochs:
                ms = "  ".join(f"{k}={format_metric(v)}" for k, v in e.metrics)
                f.write(f"epoch {e.epoch + 1}/{self.total_epochs}  {ms}  [{format_eta(e.duration_secs)}]  {e.resources.summary()}\n")

    def export_csv(self, path: str) -> None:
        names: List[str] = []
        for e in self.epochs:
            for k, _ in e.metrics:
                if k not in names:
                    names.append(k)
        with open(path, "w", newline="") as f:
            w = csv.writer(f)
            w.writerow(["epoch", "duration_secs"] + names + ["cpu_percent", "ram_used_bytes", "gpu_util_percent", "vram_allocated_bytes"])
            for e in self.epochs:
                d = dict(e.metrics)
                r = e.resources
                w.writerow([e.epoch + 1, f"{e.duration_secs:.6f}"] + [d.get(n, "") for n in names]
                           + [r.cpu_percent, r.ram_used_bytes, r.gpu_util_percent, r.vram_allocated_bytes])
