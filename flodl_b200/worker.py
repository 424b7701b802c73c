"""`CpuWorker`: one background thread running submitted closures in order, for work that must not
stall the training loop (writing checkpoints from CPU snapshots, exporting metrics)
(flodl/src/worker.rs:22-75). `finish()` drains the queue and joins."""
from __future__ import annotations

import queue
import threading
from typing import Callable, List, Optional

from . import log


class CpuWorker:
    def __init__(self, name: str = "cpu-worker"):
        self._q: "queue.Queue[Optional[Callable[[], None]]]" = queue.Queue()
        self._errors: List[BaseException] = []
        self._done = threading.Event()
        self._thread = threading.Thread(target=self._run, name=name, daemon=True)
        self._thread.start()

    @classmethod
    def new(cls) -> "CpuWorker":
        return cls()

    def _run(self) -> None:
        while True:
            job = self._q.get()
            if job is None:
                break
            try:
                job()
            except BaseException as e:   # a failing job must not kill the queue
                self._errors.append(e)
                log.msg(f"  cpu-worker: job failed: {e!r}")
            finally:
                self._q.task_done()
        self._done.set()

    def submit(self, job: Callable[[], None]) -> None:
        if self._done.is_set() or not self._thread.is_alive():
            raise RuntimeError("CpuWorker: already finished")
        self._q.put(job)

    def pending(self) -> int:
        return self._q.unfinished_tasks

    def is_idle(self) -> bool:
        """Nothing queued or running: submit the next checkpoint only then (worker.rs:57-63)."""
        return self._q.unfinished_tasks == 0

    def errors(self) -> List[BaseException]:
        return list(self._errors)

    def wait_idle(self) -> None:
        self._q.join()

    def finish(self) -> None:
        """Run everything still queued, then stop the thread. Idempotent."""
        if self._thread.is_alive():
            self._q.put(None)
            self._thread.join()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.finish()
        return False
