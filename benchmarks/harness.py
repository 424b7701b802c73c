"""Measurement protocol (benchmarks/src/harness.rs:19-180): `runs` passes of `warmup_epochs` untimed +
`measured_epochs` timed epochs, the first pass discarded as process warm-up, a device synchronize on
both sides of every timed epoch, the median epoch of each pass, and the best (lowest-median) pass
reported. Peak device memory comes from the allocator's peak statistics, reset before the run."""
from __future__ import annotations

import json
import statistics
import time
from dataclasses import asdict, dataclass, field
from typing import Callable, List, Optional

import torch


@dataclass
class BenchConfig:
    name: str = ""
    runs: int = 4
    warmup_epochs: int = 3
    measured_epochs: int = 20
    batches_per_epoch: int = 100
    batch_size: int = 128

    def quick(self) -> "BenchConfig":
        """A seconds-long variant for smoke tests."""
        return BenchConfig(self.name, 2, 1, 2, 2, min(self.batch_size, 8))


@dataclass
class BenchResult:
    name: str
    impl: str
    device: str
    param_count: int
    batch_size: int
    batches_per_epoch: int
    median_epoch_ms: float
    best_epoch_ms: float
    run_medians_ms: List[float] = field(default_factory=list)
    final_loss: float = 0.0
    peak_vram_mb: Optional[float] = None
    samples_per_s: float = 0.0

    def json(self) -> str:
        return json.dumps(asdict(self))


def _sync(device: torch.device) -> None:
    if device.type == "cuda":
        torch.cuda.synchronize(device)


def run_single_pass(cfg: BenchConfig, run_epoch: Callable[[int, bool], float], device: torch.device):
    for i in range(cfg.warmup_epochs):
        run_epoch(i, True)
    _sync(device)
    times, loss = [], 0.0
    for i in range(cfg.measured_epochs):
        t0 = time.perf_counter()
        loss = run_epoch(i, False)
        _sync(device)
        times.append((time.perf_counter() - t0) * 1e3)
    return times, loss


def run_benchmark(cfg: BenchConfig, impl: str, param_count: int, run_epoch: Callable[[int, bool], float], device) -> BenchResult:
    device = torch.device(device)
    if device.type == "cuda":
        torch.cuda.reset_peak_memory_stats(device)
    medians, best_times, loss = [], None, 0.0
    for r in range(max(1, cfg.runs)):
        times, loss = run_single_pass(cfg, run_epoch, device)
        if r == 0 and cfg.runs > 1:
            continue                      # process-level warm-up pass
        med = statistics.median(times)
        medians.append(med)
        if best_times is None or med < statistics.median(best_times):
            best_times = times
    med = statistics.median(best_times)
    peak = torch.cuda.max_memory_allocated(device) / 2 ** 20 if device.type == "cuda" else None
    return BenchResult(cfg.name, impl, str(device), param_count, cfg.batch_size, cfg.batches_per_epoch, med, min(best_times), medians,
                       float(loss), peak, cfg.batch_size * cfg.batches_per_epoch / (med * 1e-3))
