"""Per-epoch pool of samples handed out in chunks to whichever rank asks next
(flodl/src/distributed/ddp_run/coordinator/chunk_pool.rs). Offsets index the epoch's global
permutation, so chunks never overlap."""
from __future__ import annotations

import time
from typing import List, Optional, Tuple


class ChunkPool:
    @classmethod
    def new(cls, *args, **kw):
        return cls(*args, **kw)

    def __init__(self, epoch: int, total_samples: int, world_size: int):
        self.epoch = epoch
        self.total_samples = int(total_samples)
        self.cursor = 0
        self.dispatched: List[int] = [0] * world_size
        self.completed: List[int] = [0] * world_size
        self.chunks_sent: List[int] = [0] * world_size
        self.epoch_start = time.perf_counter()

    def take_chunk(self, size: int, rank: int) -> Optional[Tuple[int, int]]:
        """(offset, actual size) of the next `size` samples for `rank`, or None when exhausted."""
        if self.cursor >= self.total_samples:
            return None
        actual = min(int(size), self.total_samples - self.cursor)
        offset = self.cursor
        self.cursor += actual
        self.dispatched[rank] += actual
        self.chunks_sent[rank] += 1
        return offset, actual

    def remaining(self) -> int:
        return max(0, self.total_samples - self.cursor)

    def mark_completed(self, rank: int, samples: int) -> None:
        self.completed[rank] += int(samples)

    def in_flight(self, rank: int) -> int:
        return max(0, self.dispatched[rank] - self.completed[rank])

    def is_epoch_done(self) -> bool:
        return self.cursor >= self.total_samples and all(c >= d for d, c in zip(self.dispatched, self.completed))

    def epoch_elapsed_ms(self) -> float:
        return (time.perf_counter() - self.epoch_start) * 1e3
