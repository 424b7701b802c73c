"""Types shared by the asynchronous-DDP coordinator and its workers: policies, configuration,
the message protocol, per-epoch metrics and the partition generator
(flodl/src/distributed/ddp_run/mod.rs:60-783)."""
from __future__ import annotations

import threading
from dataclasses import dataclass, field
from enum import Enum
from typing import Callable, Dict, List, Optional, Tuple

import torch

from ... import _ext


class ApplyPolicy(Enum):
    """When averaged parameters are applied (ddp_run/mod.rs:60-110).
    Sync: average after every batch. Cadence: every `anchor` batches of the slowest rank
    (wall-time trigger). Async: batch-count trigger proportional to throughput, ranks may
    overshoot."""
    Sync = "sync"
    Cadence = "cadence"
    Async = "async"


class AverageBackend(Enum):
    """How parameters are averaged. `Nccl`: in-place collective over NVLink (here the fused
    peer-memory kernel, or `torch.distributed` where that is not available). `Cpu`: snapshots
    travel to the coordinator, which averages on the host and sends the result back."""
    Nccl = "nccl"
    Cpu = "cpu"


@dataclass
class DdpRunConfig:
    """Tuning knobs with the reference's defaults (ddp_run/mod.rs:300-436)."""
    overhead_target: Optional[float] = None
    max_anchor: Optional[int] = None
    anchor: Optional[int] = None
    divergence_threshold: Optional[float] = None
    no_divergence_guard: bool = False
    max_batch_diff: Optional[int] = None
    checkpoint_every: Optional[int] = None
    snapshot_timeout_secs: float = 5.0
    partition_ratios: Optional[List[float]] = None
    progressive_dispatch: Optional[bool] = None
    max_grad_norm: Optional[float] = None
    timeline: object = None
    max_overshoot: Optional[int] = None
    lr_scale_ratio: float = 1.0

    @classmethod
    def new(cls) -> "DdpRunConfig":
        return cls()

    def with_overhead_target(self, t): self.overhead_target = float(t); return self
    def with_max_anchor(self, m): self.max_anchor = int(m); return self
    def with_anchor(self, a): self.anchor = int(a); return self
    def with_divergence_threshold(self, t): self.divergence_threshold = float(t); return self
    def with_no_divergence_guard(self): self.no_divergence_guard = True; return self
    def with_max_batch_diff(self, d): self.max_batch_diff = int(d); return self
    def with_checkpoint_every(self, n): self.checkpoint_every = int(n); return self
    def with_snapshot_timeout(self, secs): self.snapshot_timeout_secs = float(secs); return self
    def with_partition_ratios(self, r): self.partition_ratios = list(r); return self
    def with_progressive_dispatch(self, on): self.progressive_dispatch = bool(on); return self
    def with_max_grad_norm(self, n): self.max_grad_norm = float(n); return self
    def with_timeline(self, tl): self.timeline = tl; return self
    def with_max_overshoot(self, n): self.max_overshoot = int(n); return self
    def with_lr_scale_ratio(self, r): self.lr_scale_ratio = float(r); return self


# ---- worker -> coordinator -------------------------------------------------------------------------
@dataclass
class TimingBatch:
    rank: int
    batch_ms: float
    step_count: int
    param_norm: Optional[float] = None
    batch_loss: float = 0.0
    sync_divergence: Optional[float] = None


@dataclass
class TimingSyncAck:
    rank: int
    step_count: int
    divergence: Optional[float] = None


@dataclass
class TimingExiting:
    rank: int
    error: Optional[str] = None      # set when the worker leaves because of an exception


class TimingMsg:
    """Namespace mirroring the reference's enum variants."""
    Batch = TimingBatch
    SyncAck = TimingSyncAck
    Exiting = TimingExiting


@dataclass
class MetricsMsg:
    rank: int
    epoch: int
    avg_loss: float
    batches_processed: int
    epoch_ms: float
    samples_processed: int
    scalars: Dict[str, Tuple[float, int]] = field(default_factory=dict)


@dataclass
class ParamSnapshot:
    rank: int
    params: List[torch.Tensor]
    buffers: List[torch.Tensor]
    batch_count: int


# ---- coordinator -> worker -------------------------------------------------------------------------
@dataclass
class EpochPlan:
    epoch: int
    partition_offset: int
    partition_size: int


@dataclass
class AveragedParams:
    params: List[torch.Tensor]
    buffers: List[torch.Tensor]
    version: int


@dataclass
class ControlMsg:
    """`kind` is one of RequestParams, Update, SyncNow, StartEpoch, Throttle, SetGlobalStep,
    Checkpoint, Shutdown; `payload` carries AveragedParams / EpochPlan / int as the kind needs."""
    kind: str
    payload: object = None

    @staticmethod
    def RequestParams(): return ControlMsg("RequestParams")
    @staticmethod
    def Update(avg: AveragedParams): return ControlMsg("Update", avg)
    @staticmethod
    def SyncNow(): return ControlMsg("SyncNow")
    @staticmethod
    def StartEpoch(plan: EpochPlan): return ControlMsg("StartEpoch", plan)
    @staticmethod
    def Throttle(): return ControlMsg("Throttle")
    @staticmethod
    def SetGlobalStep(step: int): return ControlMsg("SetGlobalStep", int(step))
    @staticmethod
    def Checkpoint(version: int): return ControlMsg("Checkpoint", int(version))
    @staticmethod
    def Shutdown(): return ControlMsg("Shutdown")


@dataclass
class WorkerConfig:
    rank: int
    world_size: int
    device: torch.device
    initial_params: Optional[List[torch.Tensor]]
    initial_buffers: Optional[List[torch.Tensor]]
    total_samples: int
    batch_size: int
    seed: int = 42
    max_grad_norm: Optional[float] = None
    timeline: object = None
    policy: ApplyPolicy = ApplyPolicy.Cadence
    fixed_cadence: Optional[int] = None     # workers average on their own every K local steps
    cuda_graph: bool = False


@dataclass
class TrainedState:
    """Averaged final parameters and buffers, on the CPU, in `model.parameters()` /
    `model.buffers()` order (ddp_run/mod.rs:470-500)."""
    params: List[torch.Tensor]
    buffers: List[torch.Tensor]


@dataclass
class EpochMetrics:
    epoch: int
    scalars: Dict[str, float]
    per_rank: List[Dict[str, float]]
    avg_loss: float
    epoch_ms: float
    per_rank_throughput: List[float]
    per_rank_batch_share: List[float]
    device_indices: List[int]


MetricsFn = Callable[[EpochMetrics], None]

# ---- per-thread scalar accumulator (ddp_run/mod.rs:112-160) ----------------------------------------
_tls = threading.local()


def record_scalar(name: str, value: float) -> None:
    """Call from `train_fn`: accumulates `value` under `name` for the running epoch; the worker
    drains the sums into its `MetricsMsg` and the coordinator averages them (batch-weighted)."""
    acc = getattr(_tls, "scalars", None)
    if acc is None:
        acc = _tls.scalars = {}
    s, c = acc.get(name, (0.0, 0))
    acc[name] = (s + float(value), c + 1)


def drain_scalars() -> Dict[str, Tuple[float, int]]:
    acc = getattr(_tls, "scalars", None) or {}
    _tls.scalars = {}
    return acc


def make_partition(offset: int, size: int, total: int, epoch: int, seed: int) -> List[int]:
    """Every rank shuffles 0..total with the same generator (seed + epoch) and takes its slice, so
    partitions of one epoch never overlap (ddp_run/mod.rs:751-783)."""
    perm = _ext.require().Rng(int(seed) + int(epoch)).permutation(int(total))
    end = min(int(offset) + int(size), int(total))
    part = perm[int(offset):end]
    return part.tolist() if hasattr(part, "tolist") else [int(i) for i in part]
