"""Tensor-level facade: `Device`, `DType`, `TensorError`, creation helpers and CUDA queries.

The tensor type itself is `torch.Tensor` (PyTorch stays the tensor/autograd layer underneath,
as libtorch does in the reference). This module supplies the names and helpers of the
reference's tensor layer (flodl/src/tensor/mod.rs:188-223, flodl/src/tensor/cuda.rs:15-401):
device / dtype tags with the C-ABI numbering, `test_device()`, device probing, VRAM and NVML
queries, `hardware_summary`, RSS and live-tensor counters.
"""
from __future__ import annotations

import gc
import os
from dataclasses import dataclass
from enum import Enum
from typing import List, Optional, Sequence

import torch

Tensor = torch.Tensor


class TensorError(RuntimeError):
    """Error type of the framework (flodl/src/tensor/mod.rs `TensorError`)."""

    @classmethod
    def new(cls, msg: str) -> "TensorError":
        return cls(msg)

    def is_cuda_oom(self) -> bool:
        """Whether the message reports that the device ran out of memory."""
        return "out of memory" in str(self)


class DType(Enum):
    """Element types with the C-ABI tags of flodl-sys/shim.h:920-925."""
    Float16 = 5
    BFloat16 = 15
    Float32 = 6
    Float64 = 7
    Int32 = 3
    Int64 = 4

    @property
    def torch(self) -> torch.dtype:
        return _DT2TORCH[self]

    @staticmethod
    def from_torch(dt: torch.dtype) -> "DType":
        for k, v in _DT2TORCH.items():
            if v == dt:
                return k
        raise TensorError(f"unsupported dtype {dt}")

    def element_size(self) -> int:
        return torch.empty((), dtype=self.torch).element_size()


_DT2TORCH = {
    DType.Float16: torch.float16,
    DType.BFloat16: torch.bfloat16,
    DType.Float32: torch.float32,
    DType.Float64: torch.float64,
    DType.Int32: torch.int32,
    DType.Int64: torch.int64,
}


@dataclass(frozen=True)
class Device:
    """`Device::CPU` / `Device::CUDA(i)`; C-ABI tags CPU=0, CUDA=1 (shim.h:928-929)."""
    kind: str = "cpu"
    index: int = 0

    CPU = None  # filled below

    @staticmethod
    def CUDA(index: int = 0) -> "Device":
        return Device("cuda", index)

    @staticmethod
    def of(obj) -> "Device":
        if isinstance(obj, Device):
            return obj
        if isinstance(obj, torch.Tensor):
            obj = obj.device
        d = torch.device(obj)
        return Device(d.type, d.index or 0)

    @property
    def torch(self) -> torch.device:
        return torch.device("cpu") if self.kind == "cpu" else torch.device("cuda", self.index)

    def is_cuda(self) -> bool:
        return self.kind == "cuda"

    def tag(self) -> int:
        return 1 if self.kind == "cuda" else 0

    def __str__(self) -> str:
        return "cpu" if self.kind == "cpu" else f"cuda:{self.index}"


Device.CPU = Device("cpu", 0)


@dataclass
class TensorOptions:
    dtype: DType = DType.Float32
    device: Device = Device.CPU

    def kwargs(self):
        return {"dtype": self.dtype.torch, "device": self.device.torch}


def _dev(device) -> torch.device:
    if device is None:
        return torch.device("cpu")
    return Device.of(device).torch


def cuda_available() -> bool:
    return torch.cuda.is_available()


def cuda_device_count() -> int:
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


def test_device() -> Device:
    """CUDA(0) when a GPU is usable, else CPU, so the same tests run on both
    (flodl/src/tensor/mod.rs:1260-1268)."""
    return Device.CUDA(0) if cuda_available() else Device.CPU


def test_opts() -> TensorOptions:
    return TensorOptions(DType.Float32, test_device())


def probe_device(index: int) -> bool:
    """Allocate and add on the device; False if it cannot run a kernel
    (flodl/src/tensor/cuda.rs:220-254)."""
    try:
        z = torch.zeros(8, device=f"cuda:{index}")
        (z + 1).sum().item()
        return True
    except Exception:
        return False


def usable_cuda_devices() -> List[int]:
    """Indices of the GPUs that pass `probe_device` (flodl/src/tensor/cuda.rs:259-288)."""
    return [i for i in range(cuda_device_count()) if probe_device(i)]


def cuda_synchronize(device=None) -> None:
    if cuda_available():
        torch.cuda.synchronize(None if device is None else _dev(device))


def set_current_cuda_device(index: int) -> None:
    if cuda_available():
        torch.cuda.set_device(index)


def manual_seed(seed: int) -> None:
    torch.manual_seed(seed)


def cuda_memory_info(index: int = 0):
    """(free, total) bytes from the driver (`cudaMemGetInfo`, ops_nn.cpp:499-520)."""
    if not cuda_available():
        return (0, 0)
    return torch.cuda.mem_get_info(index)


def cuda_allocated_bytes(index: int = 0) -> int:
    return torch.cuda.memory_allocated(index) if cuda_available() else 0


def cuda_reserved_bytes(index: int = 0) -> int:
    return torch.cuda.memory_reserved(index) if cuda_available() else 0


def cuda_peak_allocated_bytes(index: int = 0) -> int:
    return torch.cuda.max_memory_allocated(index) if cuda_available() else 0


def cuda_reset_peak_stats(index: int = 0) -> None:
    if cuda_available():
        torch.cuda.reset_peak_memory_stats(index)


def cuda_empty_cache() -> None:
    if cuda_available():
        torch.cuda.empty_cache()


def cuda_device_name(index: int = 0) -> str:
    return torch.cuda.get_device_name(index) if cuda_available() else "cpu"


def cuda_compute_capability(index: int = 0):
    return torch.cuda.get_device_capability(index) if cuda_available() else (0, 0)


_NVML = None


def _nvml():
    """NVML is loaded lazily and only read from (utilisation, clocks); nothing here writes a
    GPU setting. The reference `dlopen`s libnvidia-ml the same way (ops_nn.cpp:636-676)."""
    global _NVML
    if _NVML is None:
        try:
            import pynvml
            pynvml.nvmlInit()
            _NVML = pynvml
        except Exception:
            _NVML = False
    return _NVML or None


def cuda_utilization(index: int = 0) -> Optional[int]:
    nv = _nvml()
    if nv is None:
        return None
    try:
        h = nv.nvmlDeviceGetHandleByIndex(index)
        return int(nv.nvmlDeviceGetUtilizationRates(h).gpu)
    except Exception:
        return None


def cuda_clocks(index: int = 0):
    """(sm MHz, max sm MHz) or None; read-only."""
    nv = _nvml()
    if nv is None:
        return None
    try:
        h = nv.nvmlDeviceGetHandleByIndex(index)
        return (int(nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM)), int(nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM)))
    except Exception:
        return None


def rss_kb() -> int:
    """Resident set size of this process in KiB (flodl/src/tensor/cuda.rs:386-401)."""
    try:
        with open("/proc/self/statm") as f:
            pages = int(f.read().split()[1])
        return pages * os.sysconf("SC_PAGE_SIZE") // 1024
    except Exception:
        return 0


def live_tensor_count() -> int:
    """Number of live tensor objects (leak diagnostics; reference keeps LIVE_TENSOR_COUNT)."""
    return sum(1 for o in gc.get_objects() if isinstance(o, torch.Tensor))


def malloc_trim() -> None:
    try:
        import ctypes
        ctypes.CDLL("libc.so.6").malloc_trim(0)
    except Exception:
        pass


def hardware_summary() -> str:
    lines = [f"CPU threads: {os.cpu_count()}"]
    for i in range(cuda_device_count()):
        free, total = cuda_memory_info(i)
        cc = cuda_compute_capability(i)
        lines.append(f"CUDA({i}): {cuda_device_name(i)} sm_{cc[0]}{cc[1]} {total / 2**30:.1f} GiB ({free / 2**30:.1f} free)")
    if cuda_device_count() == 0:
        lines.append("CUDA: none")
    return "\n".join(lines)


# ---- creation helpers with the reference's names ------------------------------------------------
def zeros(shape: Sequence[int], opts: Optional[TensorOptions] = None) -> Tensor:
    return torch.zeros(tuple(shape), **(opts or TensorOptions()).kwargs())


def ones(shape: Sequence[int], opts: Optional[TensorOptions] = None) -> Tensor:
    return torch.ones(tuple(shape), **(opts or TensorOptions()).kwargs())


def full(shape: Sequence[int], value: float, opts: Optional[TensorOptions] = None) -> Tensor:
    return torch.full(tuple(shape), value, **(opts or TensorOptions()).kwargs())


def rand(shape: Sequence[int], opts: Optional[TensorOptions] = None) -> Tensor:
    return torch.rand(tuple(shape), **(opts or TensorOptions()).kwargs())


def randn(shape: Sequence[int], opts: Optional[TensorOptions] = None) -> Tensor:
    return torch.randn(tuple(shape), **(opts or TensorOptions()).kwargs())


def from_f32(data: Sequence[float], shape: Sequence[int], device=None) -> Tensor:
    return torch.tensor(list(data), dtype=torch.float32, device=_dev(device)).reshape(tuple(shape))


def from_i64(data: Sequence[int], shape: Sequence[int], device=None) -> Tensor:
    return torch.tensor(list(data), dtype=torch.int64, device=_dev(device)).reshape(tuple(shape))


def arange(start: float, end: float, step: float = 1.0, opts: Optional[TensorOptions] = None) -> Tensor:
    return torch.arange(start, end, step, **(opts or TensorOptions()).kwargs())


def to_f32_vec(t: Tensor) -> List[float]:
    return t.detach().float().cpu().reshape(-1).tolist()


def all_finite(t: Tensor) -> bool:
    return bool(torch.isfinite(t).all().item())


# ---- remaining device utilities of the root namespace (flodl/src/tensor/cuda.rs) -------------------
def current_cuda_device() -> int:
    return torch.cuda.current_device() if torch.cuda.is_available() else 0


def cuda_manual_seed_all(seed: int) -> None:
    if torch.cuda.is_available():
        torch.cuda.manual_seed_all(int(seed))


def set_cudnn_benchmark(enabled: bool) -> None:
    torch.backends.cudnn.benchmark = bool(enabled)


class DeviceInfo:
    """Index, name, memory and compute capability of one CUDA device."""

    def __init__(self, index: int):
        p = torch.cuda.get_device_properties(index)
        self.index, self.name, self.total_memory = index, p.name, int(p.total_memory)
        self.sm_major, self.sm_minor, self.multi_processor_count = p.major, p.minor, p.multi_processor_count

    def sm_version(self) -> str:
        return f"sm_{self.sm_major}{self.sm_minor}"

    def __repr__(self) -> str:
        return f"DeviceInfo({self.index}, {self.name!r}, {self.total_memory >> 30} GiB, sm_{self.sm_major}{self.sm_minor}, {self.multi_processor_count} SMs)"


def cuda_devices() -> List["DeviceInfo"]:
    return [DeviceInfo(i) for i in range(cuda_device_count())]


def cuda_peak_reserved_bytes(index: int = 0) -> int:
    return int(torch.cuda.max_memory_reserved(index)) if cuda_available() else 0


def _alloc_stat(index: int, key: str) -> int:
    return int(torch.cuda.memory_stats(index).get(key, 0)) if cuda_available() else 0


def cuda_active_bytes(index: Optional[int] = None) -> int:
    """Bytes in blocks the caching allocator has handed out and not yet taken back (what
    `CUDACachingAllocator::getDeviceStats` calls active; ops_nn.cpp:560-600), current device."""
    return _alloc_stat(current_cuda_device() if index is None else index, "active_bytes.all.current")


def cuda_peak_active_bytes(index: Optional[int] = None) -> int:
    return _alloc_stat(current_cuda_device() if index is None else index, "active_bytes.all.peak")


# `*_idx(i)`: the same queries for an explicit device index (flodl/src/tensor/cuda.rs:30-110)
def cuda_memory_info_idx(index: int): return cuda_memory_info(index)
def cuda_allocated_bytes_idx(index: int) -> int: return cuda_allocated_bytes(index)
def cuda_active_bytes_idx(index: int) -> int: return cuda_active_bytes(index)
def cuda_peak_active_bytes_idx(index: int) -> int: return cuda_peak_active_bytes(index)
def cuda_peak_reserved_bytes_idx(index: int) -> int: return cuda_peak_reserved_bytes(index)
def cuda_reset_peak_stats_idx(index: int) -> None: cuda_reset_peak_stats(index)
def cuda_utilization_idx(index: int): return cuda_utilization(index)
def cuda_device_name_idx(index: int) -> str: return cuda_device_name(index)


Result = object     # Rust's `Result<T>`: calls here return the value or raise `TensorError`
