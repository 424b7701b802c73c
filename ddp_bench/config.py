"""Execution modes (ddp-bench/src/config.rs:20-75).

    solo-N        one device (rank N's GPU, or the CPU), no distribution: the convergence reference
    sync          `Trainer.setup` on a graph model: gradients all-reduced inside `model.step()`
    nccl-sync     builder path, collective averaging, every batch         (ApplyPolicy.Sync)
    nccl-cadence  builder path, collective averaging, El Che cadence      (ApplyPolicy.Cadence)
    nccl-async    builder path, collective averaging, independent workers (ApplyPolicy.Async)
    cpu-*         the same three policies with host-side averaging        (AverageBackend.Cpu)
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional

from flodl_b200.parallel.ddp_run import ApplyPolicy, AverageBackend

ALL_MODES = ["solo-0", "solo-1", "sync", "nccl-sync", "nccl-cadence", "nccl-async", "cpu-sync", "cpu-cadence", "cpu-async"]


@dataclass(frozen=True)
class DdpMode:
    kind: str                               # "solo" | "sync" | "builder"
    solo_index: int = 0
    policy: Optional[ApplyPolicy] = None
    backend: Optional[AverageBackend] = None

    @staticmethod
    def parse(s: str) -> Optional["DdpMode"]:
        if s.startswith("solo-"):
            try:
                return DdpMode("solo", int(s[5:]))
            except ValueError:
                return None
        if s == "sync":
            return DdpMode("sync")
        head, _, tail = s.partition("-")
        backend = {"nccl": AverageBackend.Nccl, "cpu": AverageBackend.Cpu}.get(head)
        policy = {"sync": ApplyPolicy.Sync, "cadence": ApplyPolicy.Cadence, "async": ApplyPolicy.Async}.get(tail)
        if backend is None or policy is None:
            return None
        return DdpMode("builder", 0, policy, backend)

    def name(self) -> str:
        if self.kind == "solo":
            return f"solo-{self.solo_index}"
        if self.kind == "sync":
            return "sync"
        return f"{'nccl' if self.backend == AverageBackend.Nccl else 'cpu'}-{self.policy.name.lower()}"

    def requires_multi_gpu(self) -> bool:
        return self.kind != "solo"


@dataclass
class RunOptions:
    epochs: Optional[int] = None            # None: the model's default
    batches_per_epoch: Optional[int] = None
    batch_size: Optional[int] = None
    lr: Optional[float] = None
    seed: int = 42
    device: str = "auto"                    # auto: cuda when available
    output_dir: str = ""
    monitor_port: int = 0                   # > 0: serve the live dashboard while training
    tiny: bool = False                      # shrink data and model for smoke tests
    lr_scale: Optional[float] = None        # multiplies the learning rate (given or default)


def all_modes() -> List[DdpMode]:
    return [DdpMode.parse(m) for m in ALL_MODES]
