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
        if isinstance(dataset, TensorDataSet) and all(t.device.type == "cpu" for t in dataset.tensors()) and _ext.available():
            srcs = [t.contiguous() for t in dataset.tensors()]
            self._native = _ext.require().PrefetchWorker(srcs, self.device.index if self.device.type == "cuda" else -1, self.depth)

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

    def next(self) -> Optional[List[torch.Tensor]]:
        """Next batch on the device, or None at the end of the epoch."""
        if self._native is not None:
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
        if self._native is not None:
            self._native.stop()
            return
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
