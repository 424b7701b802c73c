"""Device-side timing helpers shared by the benchmark scripts.

Rules they implement: warm up first, time with CUDA events on the launching stream, synchronise on
both sides, and either flush the L2 cache between timed calls (a write larger than the cache) or
leave it warm on purpose. Very short kernels are timed as a batch of `inner` back-to-back launches
so the result is not quantised by the event resolution."""
from __future__ import annotations

import statistics
from typing import Callable, List, Optional

import torch

_FLUSH: Optional[torch.Tensor] = None


def flush_l2(nbytes: int = 256 << 20) -> None:
    """Overwrite a buffer larger than the L2 cache (126 MB on B200) so the next kernel starts cold."""
    global _FLUSH
    if _FLUSH is None or _FLUSH.numel() < nbytes:
        _FLUSH = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    _FLUSH.zero_()


def cuda_time_ms(fn: Callable[[], object], iters: int = 20, warmup: int = 3, cold_l2: bool = True, inner: int = 1) -> List[float]:
    """Per-call device times in milliseconds (one entry per timed iteration; each iteration runs
    `fn` `inner` times between the two events and reports the mean)."""
    for _ in range(max(0, warmup)):
        fn()
    torch.cuda.synchronize()
    out = []
    for _ in range(iters):
        if cold_l2:
            flush_l2()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(inner):
            fn()
        b.record()
        torch.cuda.synchronize()
        out.append(a.elapsed_time(b) / inner)
    return out


def median_ms(fn: Callable[[], object], iters: int = 20, warmup: int = 3, cold_l2: bool = True, inner: int = 1) -> float:
    return statistics.median(cuda_time_ms(fn, iters, warmup, cold_l2, inner))


def graph_chain_us(fn: Callable[[], object], reps: int = 40, rounds: int = 5) -> float:
    """Steady-state time of one call of `fn` in microseconds: `reps` calls captured back to back in
    one CUDA graph, best of `rounds` replays, divided by `reps`. Launch latency and clock ramp-up
    are outside the figure, the way they are inside a captured training step; the cache is warm."""
    fn()
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        fn()
    torch.cuda.current_stream().wait_stream(side)
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for _ in range(reps):
            fn()
    g.replay()
    torch.cuda.synchronize()
    best = float("inf")
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for _ in range(rounds):
        a.record()
        g.replay()
        b.record()
        torch.cuda.synchronize()
        best = min(best, a.elapsed_time(b) * 1e3 / reps)
    return best
