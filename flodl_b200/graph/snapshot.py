"""CPU snapshots of a model for background saving (flodl/src/graph/snapshot.rs:43-72): named
tensors copied to host memory now, written later (by a `CpuWorker`) as an `.fdl` with a zero hash."""
from __future__ import annotations

from typing import List, Tuple

import torch

from .. import _ext


class ModelSnapshot:
    def __init__(self, params: List[Tuple[str, torch.Tensor]], buffers: List[Tuple[str, torch.Tensor]]):
        self.params, self.buffers = params, buffers

    def save(self) -> bytes:
        return _ext.require().fdl_save_bytes(self.params + self.buffers, b"\0" * 32, 2)

    def save_file(self, path: str) -> None:
        _ext.require().fdl_save(path, self.params + self.buffers, b"\0" * 32, 2)


def snapshot_cpu(graph) -> ModelSnapshot:
    ps = [(n, p.variable.data().to("cpu", copy=True)) for n, p in graph.named_parameters()]
    bs = [(n, b.get().to("cpu", copy=True)) for n, b in graph.named_buffers()]
    return ModelSnapshot(ps, bs)
