"""Control-plane transports between the coordinator and its workers.

The reference wires them with `std::sync::mpsc` channels inside one process
(flodl/src/distributed/ddp_run/orchestrator.rs:170-190). Two transports implement the same
mailbox interface here:

* `LocalTransport`  - `queue.Queue`s, for workers that are threads of the coordinator's process;
* `StoreTransport`  - a `torch.distributed.TCPStore` hosted by rank 0, for one-process-per-GPU
  jobs. Every mailbox is a sequence of keys `<box>/<n>`; the sender numbers messages, the
  receiver polls for the next number (`check` is non-blocking) and deletes what it has read.
  Payloads are pickled; tensors travel as CPU tensors.

A mailbox has one reader. Boxes: `ctl<rank>` (coordinator -> worker), `tim<rank>`, `met<rank>`,
`par<rank>`, `fin<rank>` (worker -> coordinator).
"""
from __future__ import annotations

import pickle
import queue
import time
from typing import Dict, Optional


class Mailbox:
    def send(self, msg) -> None: raise NotImplementedError
    def try_recv(self): raise NotImplementedError

    def recv(self, timeout: Optional[float] = None, poll_s: float = 0.0002):
        """Blocking receive; None on timeout."""
        deadline = None if timeout is None else time.monotonic() + timeout
        while True:
            m = self.try_recv()
            if m is not None:
                return m
            if deadline is not None and time.monotonic() >= deadline:
                return None
            time.sleep(poll_s)


class _QueueBox(Mailbox):
    def __init__(self):
        self.q: "queue.Queue" = queue.Queue()

    def send(self, msg) -> None:
        self.q.put(msg)

    def try_recv(self):
        try:
            return self.q.get_nowait()
        except queue.Empty:
            return None

    def recv(self, timeout: Optional[float] = None, poll_s: float = 0.0002):
        try:
            return self.q.get(timeout=timeout)
        except queue.Empty:
            return None


class LocalTransport:
    def __init__(self):
        self._boxes: Dict[str, _QueueBox] = {}

    def box(self, name: str) -> Mailbox:
        b = self._boxes.get(name)
        if b is None:
            b = self._boxes[name] = _QueueBox()
        return b


class _StoreBox(Mailbox):
    """Message n of a box lives under `<box>/<n>`: a small header (the number of chunks) written LAST, and the
    pickled payload in chunks `<box>/<n>/c<k>` of at most `CHUNK` bytes (the store's server refuses requests above
    8 MB; parameter snapshots are hundreds of megabytes)."""
    CHUNK = 4 << 20

    def __init__(self, store, name: str):
        self.store, self.name = store, name
        self.tx = 0
        self.rx = 0

    def send(self, msg) -> None:
        data = pickle.dumps(msg, protocol=pickle.HIGHEST_PROTOCOL)
        key = f"{self.name}/{self.tx}"
        n = max(1, (len(data) + self.CHUNK - 1) // self.CHUNK)
        for k in range(n):
            self.store.set(f"{key}/c{k}", data[k * self.CHUNK:(k + 1) * self.CHUNK])
        self.store.set(key, str(n).encode())          # the receiver looks for this key: every chunk is there by now
        self.tx += 1

    def try_recv(self):
        key = f"{self.name}/{self.rx}"
        if not self.store.check([key]):
            return None
        n = int(bytes(self.store.get(key)).decode())
        raw = b"".join(bytes(self.store.get(f"{key}/c{k}")) for k in range(n))
        for k in [key] + [f"{key}/c{k}" for k in range(n)]:
            try:
                self.store.delete_key(k)
            except Exception:
                pass
        self.rx += 1
        return pickle.loads(raw)


class StoreTransport:
    """`store`: a `torch.distributed.TCPStore` (or any object with set/get/check/delete_key).
    `namespace` separates successive runs that share one store."""

    def __init__(self, store, namespace: str = "ddp0"):
        self.store, self.ns = store, namespace
        self._boxes: Dict[str, _StoreBox] = {}

    def box(self, name: str) -> Mailbox:
        b = self._boxes.get(name)
        if b is None:
            b = self._boxes[name] = _StoreBox(self.store, f"{self.ns}/{name}")
        return b


def make_store_transport(namespace: str = "ddp0", timeout_s: float = 600.0) -> StoreTransport:
    """A TCPStore of its own for the control plane: rank 0 listens on a free port and tells the
    others through the existing process group."""
    import datetime
    import os
    import socket

    import torch.distributed as dist

    rank, world = dist.get_rank(), dist.get_world_size()
    host = os.environ.get("MASTER_ADDR", "127.0.0.1")
    port = [0]
    if rank == 0:
        with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
            s.bind(("", 0))
            port[0] = s.getsockname()[1]
    dist.broadcast_object_list(port, src=0)
    store = dist.TCPStore(host, int(port[0]), world, is_master=(rank == 0), timeout=datetime.timedelta(seconds=timeout_s),
                          wait_for_workers=False)
    return StoreTransport(store, namespace)
