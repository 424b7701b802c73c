"""CUDA graph capture / replay (flodl/src/nn/cuda_graph.rs, flodl-sys/ops_cuda.cpp:21-139).

Launch-bound inner loops (small models, many tiny kernels) are captured once and replayed; the
native kernels of this library read their per-step scalars (learning rate, dropout seed offset,
collective epochs) from device memory precisely so that a replay does the right thing."""
from __future__ import annotations

from enum import Enum
from typing import Callable, Optional

import torch

from ..tensor import TensorError


class CaptureMode(Enum):
    Global = "global"
    ThreadLocal = "thread_local"
    Relaxed = "relaxed"


MemPoolId = tuple


def cuda_graph_pool_handle() -> MemPoolId:
    return torch.cuda.graph_pool_handle()


class CudaGraph:
    def __init__(self):
        if not torch.cuda.is_available():
            raise TensorError("CudaGraph requires a CUDA device")
        self._g = torch.cuda.CUDAGraph()
        self._stream: Optional[torch.cuda.Stream] = None
        self._ctx = None
        self._captured = False

    @classmethod
    def new(cls): return cls()

    def capture_begin(self, pool: Optional[MemPoolId] = None, mode: CaptureMode = CaptureMode.ThreadLocal) -> None:
        self._stream = torch.cuda.Stream()
        self._stream.wait_stream(torch.cuda.current_stream())
        self._ctx = torch.cuda.stream(self._stream)
        self._ctx.__enter__()
        self._g.capture_begin(pool=pool, capture_error_mode=mode.value)

    def capture_end(self) -> None:
        self._g.capture_end()
        self._ctx.__exit__(None, None, None)
        torch.cuda.current_stream().wait_stream(self._stream)
        self._captured = True

    def replay(self) -> None:
        if not self._captured:
            raise TensorError("CudaGraph.replay before capture")
        self._g.replay()

    def reset(self) -> None:
        self._g.reset()
        self._captured = False

    def pool(self) -> MemPoolId:
        return self._g.pool()


def cuda_graph_capture(warmup_runs: int, pool: Optional[MemPoolId], f: Callable[[], None]) -> CudaGraph:
    """Run `f` `warmup_runs` times, synchronise, then capture one more run (cuda_graph.rs:166-190)."""
    for _ in range(warmup_runs):
        f()
    torch.cuda.synchronize()
    g = CudaGraph()
    g.capture_begin(pool)
    try:
        f()
    finally:
        g.capture_end()
    return g
