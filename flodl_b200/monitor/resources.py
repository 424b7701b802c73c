"""One-shot resource sampling: CPU utilisation from /proc/stat deltas, RAM from /proc/meminfo,
per-GPU utilisation through NVML (read-only queries) and memory through the CUDA runtime
(flodl/src/monitor/resources.rs). Everything degrades to None where a source is missing."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional

from .format import format_bytes


@dataclass
class GpuSnapshot:
    index: int
    name: str = ""
    util_percent: Optional[float] = None
    vram_used_bytes: Optional[int] = None
    vram_total_bytes: Optional[int] = None
    vram_allocated_bytes: Optional[int] = None
    sm_clock_mhz: Optional[int] = None
    power_w: Optional[float] = None


@dataclass
class ResourceSample:
    cpu_percent: Optional[float] = None
    ram_used_bytes: Optional[int] = None
    ram_total_bytes: Optional[int] = None
    gpu_util_percent: Optional[float] = None
    vram_allocated_bytes: Optional[int] = None
    vram_total_bytes: Optional[int] = None
    gpus: List[GpuSnapshot] = field(default_factory=list)

    def summary(self) -> str:
        parts = []
        if self.cpu_percent is not None:
            parts.append(f"CPU {self.cpu_percent:.0f}%")
        if self.ram_used_bytes is not None and self.ram_total_bytes:
            parts.append(f"RAM {format_bytes(self.ram_used_bytes)}/{format_bytes(self.ram_total_bytes)}")
        for g in self.gpus:
            s = f"GPU{g.index}"
            if g.util_percent is not None:
                s += f" {g.util_percent:.0f}%"
            if g.vram_used_bytes is not None and g.vram_total_bytes:
                s += f" {format_bytes(g.vram_used_bytes)}/{format_bytes(g.vram_total_bytes)}"
            parts.append(s)
        return " | ".join(parts)

    def to_dict(self) -> dict:
        d = {k: getattr(self, k) for k in ("cpu_percent", "ram_used_bytes", "ram_total_bytes", "gpu_util_percent",
                                           "vram_allocated_bytes", "vram_total_bytes")}
        d["gpus"] = [g.__dict__ for g in self.gpus]
        return d


def _read_cpu():
    try:
        with open("/proc/stat") as f:
            vals = [int(x) for x in f.readline().split()[1:]]
        idle = vals[3] + (vals[4] if len(vals) > 4 else 0)
        return sum(vals), idle
    except Exception:
        return None


def _read_mem():
    try:
        info = {}
        with open("/proc/meminfo") as f:
            for line in f:
                k, v = line.split(":", 1)
                info[k] = int(v.split()[0]) * 1024
        total = info["MemTotal"]
        return total - info.get("MemAvailable", info.get("MemFree", 0)), total
    except Exception:
        return None


class ResourceSampler:
    """`nvml` may be injected (an object with the `pynvml` query functions) for tests."""

    def __init__(self, nvml=None, devices: Optional[List[int]] = None):
        self._last_cpu = _read_cpu()
        self._nvml = nvml
        self._handles = {}
        self._devices = devices
        if self._nvml is None:
            try:
                import pynvml
                pynvml.nvmlInit()
                self._nvml = pynvml
            except Exception:
                self._nvml = None

    @classmethod
    def new(cls) -> "ResourceSampler":
        return cls()

    def _gpu_indices(self) -> List[int]:
        if self._devices is not None:
            return self._devices
        try:
            import torch
            return list(range(torch.cuda.device_count())) if torch.cuda.is_available() else []
        except Exception:
            return []

    def _handle(self, i: int):
        h = self._handles.get(i)
        if h is None and self._nvml is not None:
            try:
                h = self._handles[i] = self._nvml.nvmlDeviceGetHandleByIndex(i)
            except Exception:
                h = None
        return h

    def sample(self) -> ResourceSample:
        s = ResourceSample()
        cur = _read_cpu()
        if cur is not None and self._last_cpu is not None:
            dt, di = cur[0] - self._last_cpu[0], cur[1] - self._last_cpu[1]
            if dt > 0:
                s.cpu_percent = 100.0 * (1.0 - di / dt)
        self._last_cpu = cur
        mem = _read_mem()
        if mem is not None:
            s.ram_used_bytes, s.ram_total_bytes = mem
        for i in self._gpu_indices():
            g = GpuSnapshot(i)
            h = self._handle(i)
            if h is not None:
                nv = self._nvml
                try:
                    g.util_percent = float(nv.nvmlDeviceGetUtilizationRates(h).gpu)
                    m = nv.nvmlDeviceGetMemoryInfo(h)
                    g.vram_used_bytes, g.vram_total_bytes = int(m.used), int(m.total)
                    g.sm_clock_mhz = int(nv.nvmlDeviceGetClockInfo(h, getattr(nv, "NVML_CLOCK_SM", 1)))
                    g.power_w = nv.nvmlDeviceGetPowerUsage(h) / 1000.0
                    name = nv.nvmlDeviceGetName(h)
                    g.name = name.decode() if isinstance(name, bytes) else str(name)
                except Exception:
                    pass
            try:
                import torch
                if torch.cuda.is_available() and torch.cuda.is_initialized():
                    g.vram_allocated_bytes = int(torch.cuda.memory_allocated(i))
                    if g.vram_total_bytes is None:
                        free, total = torch.cuda.mem_get_info(i)
                        g.vram_used_bytes, g.vram_total_bytes = int(total - free), int(total)
            except Exception:
                pass
            s.gpus.append(g)
        if s.gpus:
            utils = [g.util_percent for g in s.gpus if g.util_percent is not None]
            s.gpu_util_percent = sum(utils) / len(utils) if utils else None
            allocs = [g.vram_allocated_bytes for g in s.gpus if g.vram_allocated_bytes is not None]
            s.vram_allocated_bytes = sum(allocs) if allocs else None
            tots = [g.vram_total_bytes for g in s.gpus if g.vram_total_bytes is not None]
            s.vram_total_bytes = sum(tots) if tots else None
        return s
