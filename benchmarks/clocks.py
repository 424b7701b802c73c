"""Optional SM clock lock and GPU warm-up for publication runs of the benchmark suite (benchmarks/run.sh:141-215 of the
reference: `nvidia-smi -lgc <MHz>,<MHz>` before the run, `-rgc` after it, a matrix-multiply warm-up in between).

**Off by default, and meant for a machine of your own.** A clock lock is a setting of the GPU, not of the process: it
stays until it is reset and whoever uses the GPU next inherits it. On shared machines leave it alone: `benchmarks.run`
records the clocks it observed (`gpu_clocks()`), which is enough to tell a throttled run from a clean one. Nothing in
this repository's tests or benchmark commands turns the lock on; the logic is exercised against a stand-in for NVML.

The NVML calls go through a small backend object so that they can be replaced: `NvmlBackend` uses `pynvml`
(`nvidia-ml-py`), a test passes its own.
"""
from __future__ import annotations

import time
from typing import List, Optional


class NvmlBackend:
    """The four calls the lock needs, over `pynvml`."""

    def __init__(self):
        import pynvml
        self.nv = pynvml
        self.nv.nvmlInit()

    def device_count(self) -> int:
        return int(self.nv.nvmlDeviceGetCount())

    def default_graphics_clock(self, index: int) -> Optional[int]:
        h = self.nv.nvmlDeviceGetHandleByIndex(index)
        try:
            return int(self.nv.nvmlDeviceGetDefaultApplicationsClock(h, self.nv.NVML_CLOCK_GRAPHICS))
        except self.nv.NVMLError:
            return None

    def lock(self, index: int, mhz: int) -> None:
        self.nv.nvmlDeviceSetGpuLockedClocks(self.nv.nvmlDeviceGetHandleByIndex(index), mhz, mhz)

    def reset(self, index: int) -> None:
        self.nv.nvmlDeviceResetGpuLockedClocks(self.nv.nvmlDeviceGetHandleByIndex(index))


def detect_base_clock(backend, index: int = 0) -> Optional[int]:
    """The default applications clock of the device: the frequency the reference's script locks to when none is given."""
    return backend.default_graphics_clock(index)


class ClockLock:
    """`with ClockLock(backend, mhz=None, devices=None): ...` locks every listed device to `mhz` (the detected base clock
    when None) and always resets the ones it locked on the way out, also after an exception. A device that refuses the lock
    (no permission, unsupported) is reported in `failed` and left as it was; the run goes on with a warning, as the
    reference's script does."""

    def __init__(self, backend, mhz: Optional[int] = None, devices: Optional[List[int]] = None, log=print):
        self.backend, self.mhz, self.log = backend, mhz, log
        self.devices = list(range(backend.device_count())) if devices is None else list(devices)
        self.locked: List[int] = []
        self.failed: List[int] = []

    def __enter__(self) -> "ClockLock":
        for i in self.devices:
            mhz = self.mhz if self.mhz is not None else detect_base_clock(self.backend, i)
            if mhz is None:
                self.log(f"WARNING: GPU {i}: no base clock to lock to; left unlocked")
                self.failed.append(i)
                continue
            try:
                self.backend.lock(i, int(mhz))
                self.locked.append(i)
                self.log(f"=== GPU {i}: clocks locked at {int(mhz)} MHz ===")
            except Exception as e:  # noqa: BLE001  (NVML raises its own error types)
                self.failed.append(i)
                self.log(f"WARNING: GPU {i}: could not lock clocks ({e}); results may show higher variance")
        return self

    def __exit__(self, *exc) -> bool:
        for i in self.locked:
            try:
                self.backend.reset(i)
                self.log(f"=== GPU {i}: clocks unlocked ===")
            except Exception as e:  # noqa: BLE001
                self.log(f"WARNING: GPU {i}: could not reset clocks ({e}); run `nvidia-smi -rgc -i {i}`")
        self.locked = []
        return False


def gpu_warmup(seconds: float, device: str = "cuda", size: int = 4096, now=time.monotonic) -> int:
    """Matrix products for `seconds` so that clocks and temperature settle before the first timed epoch; returns the
    number of products issued (0 without a GPU)."""
    import torch
    if seconds <= 0 or not (device.startswith("cuda") and torch.cuda.is_available()):
        return 0
    a = torch.randn(size, size, device=device)
    n, end = 0, now() + seconds
    while now() < end:
        for _ in range(10):
            a = (a @ a).clamp_(-1.0, 1.0)
            n += 1
        torch.cuda.synchronize()
    return n
