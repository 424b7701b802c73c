"""Background batch producer (flodl/src/data/prefetch.rs:163-285).

For a `TensorDataSet` whose tensors live in host memory the native worker is used: a C++ thread
gathers the rows of each batch into pinned staging buffers and copies them to the device on its
own CUDA stream; `next()` makes the consumer's stream wait on the copy's event, never the host.
Any other `BatchDataSet` is served by a Python thread that calls `get_batch`, pins and copies.
Both keep at most `depth` batches in flight.
"""
from __future__ import annotations

import queue
import threading
from typing import List, Optional, Sequence

import torch

from .. import _ext
from .dataset import BatchDataSet, TensorDataSet


class PrefetchWorker:
    def __init__(self, dataset: BatchDataSet, device, depth: int = 4):
        self.dataset = dataset
        self.device = torch.device(device)
        self.depth = max(1, int(depth))
        self._native = None
        self._thread: Optional[threading.Thread] = None
        self._q: Optional["queue.Queue"] = None
        self._stop = threading.Event()
        self._cmd: Optional["queue.Queue"] = None          # distributed mode: index lists, one per requested batch
        if isinstance(dataset, TensorDataSet) and all(t.device.type == "cpu" for t in dataset.tensors()) and _ext.available():
            srcs = [t.contiguous() for t in dataset.tensors()]
            self._native = _ext.require().PrefetchWorker(srcs, self.device.index if self.device.type == "cuda" else -1, self.depth)

    @classmethod
    def new(cls, dataset: BatchDataSet, device, prefetch_depth: int = 4) -> "PrefetchWorker":
        return cls(dataset, device, prefetch_depth)

    def prefetch_depth(self) -> int:
        return self.depth

    def set_prefetch_depth(self, depth: int) -> None:
        """Takes effect at the next `start_epoch`."""
        self.depth = max(1, int(depth))

    def is_native(self) -> bool:
        return self._native is not None

    def start_epoch(self, order: Sequence[int], batch_size: int, drop_last: bool = True) -> None:
        self.stop()
        if self._native is not None:
            self._native.start_epoch(torch.as_tensor(list(order), dtype=torch.long), int(batch_size), bool(drop_last))
            return
        order = list(order)
        nb = len(order) // batch_size if drop_last else -(-len(order) // batch_size)
        self._q = queue.Queue(maxsize=self.depth)
        self._stop = threading.Event()
        q, stop = self._q, self._stop
        stream = torch.cuda.Stream(self.device) if self.device.type == "cuda" else None

        def work():
            try:
                for b in range(nb):
                    if stop.is_set():
                        return
                    batch = self.dataset.get_batch(order[b * batch_size:(b + 1) * batch_size])
                    ev = None
                    if stream is not None:
                        with torch.cuda.stream(stream):
                            batch = [t.pin_memory().to(self.device, non_blocking=True) if t.device.type == "cpu" else t for t in batch]
                            ev = torch.cuda.Event()
                            ev.record(stream)
                    while not stop.is_set():
                        try:
                            q.put((batch, ev), timeout=0.05)
                            break
                        except queue.Full:
                            continue
                q.put(None)
            except BaseException as e:
                q.put(e)

        self._thread = threading.Thread(target=work, name="prefetch", daemon=True)
        self._thread.start()

    def _load(self, indices, stream):
        batch = self.dataset.get_batch(indices)
        ev = None
        if stream is not None:
            with torch.cuda.stream(stream):
                batch = [t.pin_memory().to(self.device, non_blocking=True) if t.device.type == "cpu" else t for t in batch]
                ev = torch.cuda.Event()
                ev.record(stream)
        return batch, ev

    def start_distributed_epoch(self) -> "queue.Queue":
        """Open an epoch whose batches are asked for one at a time with `load_batch(indices)` (the
        shard sizes of a heterogeneous run change from batch to batch, so the order cannot be
        handed over up front). Results come back in request order from `next()`, or from the
        returned queue as `(tensors, ready_event)` items (prefetch.rs:108-123)."""
        self.stop()
        self._q = queue.Queue(maxsize=self.depth)
        self._cmd = queue.Queue()
        self._stop = threading.Event()
        q, cmd, stop = self._q, self._cmd, self._stop
        stream = torch.cuda.Stream(self.device) if self.device.type == "cuda" else None

        def work():
            try:
                while not stop.is_set():
                    try:
                        indices = cmd.get(timeout=0.05)
                    except queue.Empty:
                        continue
                    if indices is None:
                        break
                    item = self._load(indices, stream)
                    while not stop.is_set():
                        try:
                            q.put(item, timeout=0.05)
                            break
                        except queue.Full:
                            continue
                q.put(None)
            except BaseException as e:
                q.put(e)

        self._thread = threading.Thread(target=work, name="prefetch-dist", daemon=True)
        self._thread.start()
        return q

    def load_batch(self, indices: Sequence[int]) -> None:
        """Request one batch (distributed mode); `end_distributed_epoch()` after the last one."""
        if self._cmd is None:
            raise RuntimeError("PrefetchWorker.load_batch: call start_distributed_epoch() first")
        self._cmd.put(list(indices))

    def end_distributed_epoch(self) -> None:
        if self._cmd is not None:
            self._cmd.put(None)

    def next(self) -> Optional[List[torch.Tensor]]:
        """Next batch on the device, or None at the end of the epoch."""
        if self._native is not None and self._cmd is None:
            return self._native.next()
        if self._q is None:
            return None
        item = self._q.get()
        if item is None:
            self._q = None
            return None
        if isinstance(item, BaseException):
            self._q = None
            raise item
        batch, ev = item
        if ev is not None:
            torch.cuda.current_stream(self.device).wait_event(ev)
        return batch

    def stop(self) -> None:
        if self._native is not None and self._cmd is None:
            self._native.stop()
            return
        self._cmd = None
        self._stop.set()
        if self._thread is not None:
            if self._q is not None:
                try:
                    while True:
                        self._q.get_nowait()
                except queue.Empty:
                    pass
            self._thread.join(timeout=5)
            self._thread = None
        self._q = None
