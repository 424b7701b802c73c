"""Bucketed gradient all-reduce overlapped with backward.

The reference all-reduces one gradient tensor per NCCL call after backward has finished, on the
default stream (flodl/src/distributed/ddp.rs:133-147; 65 calls per step for ResNet-20, ~200 for
BERT-base). Here gradients live in one flat fp32 buffer in peer-mapped memory, cut into ~25 MB
buckets; the moment the last gradient of a bucket has been produced during backward, the bucket's
all-reduce kernel (csrc/comm: P2P loads/stores over NVLink, averaging fused) is launched on a
high-priority side stream, and the optimizer waits for all of them through one event.

Bucket readiness: every gradient producer reports the parameter it touched - the native ops
through `ops.core.GRAD_HOOK` (they write into the flat buffer themselves), everything else through
`register_post_accumulate_grad_hook`. The number of reports a parameter gets per step (tied
weights get several) is learned on the first step, which runs without overlap.
"""
from __future__ import annotations

import os
from typing import Dict, List, Optional, Sequence

import torch

from ..ops import core as _core
from . import comm as _comm
from .flat import FlatParams


class GradSync:
    def __init__(self, flat: FlatParams, symm: Optional[_comm.SymmetricBuffer], bucket_bytes: int = 25 * 1024 * 1024,
                 overlap: bool = True, blocks: int = 24, backend: str = "symm", world: Optional[int] = None, tail_blocks: int = 96):
        self.flat, self.symm, self.blocks = flat, symm, blocks
        # The last bucket of a step (and anything launched after backward has ended) has no compute
        # left to overlap with, so it may use most of the GPU instead of the few blocks that keep the
        # overlapped buckets out of the GEMMs' way.
        self.tail_blocks = max(int(tail_blocks), int(blocks))
        # How many of the last buckets (the first parameters of the buffer: embeddings and the first layers, whose
        # gradients are complete only as backward ends) the optimizer leaves for a second pass, see finish().
        self.tail_buckets = max(1, int(os.environ.get("FLODL_B200_TAIL_BUCKETS", "1")))
        self._done_recorded = False
        self.world = _comm.world_size() if world is None else int(world)   # world=1: no gradient exchange (Local SGD)
        self.backend = backend if self.world > 1 else "none"
        self.overlap = overlap and self.world > 1
        self.buckets = flat.buckets(bucket_bytes)
        self.index: Dict[int, int] = {id(t): i for i, t in enumerate(flat.tensors)}
        self.bucket_of: List[int] = [0] * len(flat.tensors)
        for bi, b in enumerate(self.buckets):
            for i in b["members"]:
                self.bucket_of[i] = bi
        self.expected: Optional[List[int]] = None
        self.touch = [0] * len(flat.tensors)
        self.pending = [0] * len(self.buckets)
        self.launched = [False] * len(self.buckets)
        self.weights: Optional[List[float]] = None
        self.stream = (torch.cuda.Stream(priority=int(os.environ.get("FLODL_B200_COMM_PRIORITY", "-1")))
                       if flat.device.type == "cuda" and self.world > 1 else None)
        self.done = torch.cuda.Event() if self.stream is not None else None
        self.done_tail = torch.cuda.Event() if self.stream is not None else None
        self.active = False
        self.launch_count = 0
        self.next_bucket = 0
        self.mismatch = False
        self._hooks = []
        # per-bucket exchange timing (eager steps only: timing events cannot be recorded into a CUDA graph)
        self._timing = False
        self._timing_events: List[tuple] = []
        if self.world > 1:
            for t in flat.tensors:
                if t.requires_grad:
                    self._hooks.append(t.register_post_accumulate_grad_hook(self._on_touch))

    # ---- per step -------------------------------------------------------------------------------
    def begin_step(self) -> None:
        """Call before forward: arms the readiness tracking for this step. Raises if a collective
        of an earlier step has reported a give-up since (the status word is host-mapped, so this
        costs one host read, no device sync)."""
        if self.world <= 1:
            return
        if self.symm is not None:
            self.symm.check_async()
        self.active = True
        _core.GRAD_HOOK["fn"] = self._on_touch
        for i in range(len(self.touch)):
            self.touch[i] = 0
        self.next_bucket = 0
        self.mismatch = False
        self._done_recorded = False
        for bi, b in enumerate(self.buckets):
            self.launched[bi] = False
            self.pending[bi] = sum(1 for i in b["members"] if self.expected is not None and self.expected[i] > 0)

    def _on_touch(self, p: torch.Tensor) -> None:
        if not self.active:
            return
        members = getattr(p, "_fb_members", None)
        if members is not None:
            for m in members:
                self._on_touch(m)
            return
        i = self.index.get(id(p))
        if i is None:
            return
        self.touch[i] += 1
        if self.expected is None or not self.overlap:
            return
        bi = self.bucket_of[i]
        if self.launched[bi] or self.touch[i] > self.expected[i]:
            # a gradient arrived for a bucket that has already been reduced (or a parameter got more
            # contributions than on the step the counts were learned from): this step's result for
            # the bucket would miss it. finish() reports it and turns the overlap off.
            self.mismatch = True
            return
        if self.touch[i] == self.expected[i]:
            self.pending[bi] -= 1
            self._launch_ready()

    def _launch_ready(self) -> None:
        """Buckets go out strictly in index order, each index always with the same block count, so
        the per-block flags of a launch can only ever meet the same launch on the other ranks,
        whatever the order in which gradients became ready there."""
        while self.next_bucket < len(self.buckets) - 1 and self.pending[self.next_bucket] == 0 and not self.launched[self.next_bucket]:
            self._launch(self.next_bucket)
            self.next_bucket += 1

    def _launch(self, bi: int, tail: bool = False) -> None:
        b = self.buckets[bi]
        self.launched[bi] = True
        tail = bi == len(self.buckets) - 1    # the last index has no compute left to overlap with: always the wide launch
        if self.stream is None:               # CPU replicas (gloo): reduce in line
            self._reduce_range(b["start"], b["end"])
            self.launch_count += 1
            return
        cur = torch.cuda.current_stream()
        ev = torch.cuda.Event()
        ev.record(cur)
        self._mark_rest_done(bi)
        self.stream.wait_event(ev)
        timed = self._timing and not torch.cuda.is_current_stream_capturing()
        with torch.cuda.stream(self.stream):
            if timed:
                t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                t0.record(self.stream)
            self._reduce_range(b["start"], b["end"], self.tail_blocks if tail else self.blocks)
            if timed:
                t1.record(self.stream)
                self._timing_events.append((bi, t0, t1))
        self.launch_count += 1

    def _first_tail(self) -> int:
        return max(0, len(self.buckets) - self.tail_buckets)

    def _mark_rest_done(self, bi: int) -> None:
        """Called before bucket `bi` is put on the exchange stream: `done` is recorded in front of the first tail
        bucket, so waiting for it means "every bucket before the tail has been exchanged" and nothing more."""
        if self.stream is not None and not self._done_recorded and bi >= self._first_tail():
            self.done.record(self.stream)
            self._done_recorded = True

    def _reduce_range(self, start: int, end: int, blocks: Optional[int] = None) -> None:
        n = end - start
        if self.backend == "symm":
            self.symm.all_reduce(start * 4, n, torch.float32, self.weights, self.blocks if blocks is None else blocks)
        elif self.backend == "nccl":
            g = self.flat.grads[start:end]
            if self.weights is not None:
                g.mul_(self.weights[_comm.rank()])
                torch.distributed.all_reduce(g, torch.distributed.ReduceOp.SUM)
            else:
                _comm.all_reduce_nccl([g], _comm.ReduceOp.Avg)

    def finish(self, defer_tail: bool = False):
        """Call after backward: launches whatever has not been launched, then makes the current
        stream wait for every bucket.

        `defer_tail=True`: the current stream waits for every bucket but the last `tail_buckets` ones (the first
        parameters of the buffer: their gradients are complete only as backward ends, so their exchange can
        overlap little or nothing of it) and `(lo, hi)`, the element range of those buckets, is returned. The
        caller applies the optimizer to the rest, calls `wait_tail()`, then applies it to `[lo, hi)`: the last
        exchanges run behind the optimizer instead of in front of it."""
        if self.world <= 1:
            return None
        self.active = False
        _core.GRAD_HOOK["fn"] = None
        if self.expected is None:
            self.expected = list(self.touch)
        tail = None
        split = defer_tail and self.stream is not None and len(self.buckets) > 1 and not self.mismatch
        for bi in range(len(self.buckets)):
            if not self.launched[bi]:
                self._launch(bi)
        if self.stream is not None:
            if split:
                # `done` sits in front of the first tail bucket (see _mark_rest_done): the optimizer may start on
                # everything behind the tail while the tail buckets are still being exchanged
                self._mark_rest_done(len(self.buckets))
                torch.cuda.current_stream().wait_event(self.done)
                self.done_tail.record(self.stream)
                tail = (self.buckets[-1]["start"], self.buckets[self._first_tail()]["end"])
            else:
                self.done_tail.record(self.stream)
                torch.cuda.current_stream().wait_event(self.done_tail)
        if self.mismatch:
            self.overlap = False
            raise RuntimeError(
                "gradient exchange: a gradient was produced after its bucket had been reduced (the set of parameters that "
                "receive gradients changed between steps). This step's gradients are incomplete on this rank; overlap is now "
                "off. Build the trainer with overlap=False for models whose backward differs from step to step.")
        return tail

    # ---- diagnostics ------------------------------------------------------------------------------
    def enable_timing(self, on: bool = True) -> None:
        """Bracket every bucket exchange of the following eager steps with CUDA events (`bucket_report`)."""
        self._timing = bool(on)
        self._timing_events.clear()

    def bucket_report(self, link_gbs: float = 900.0) -> List[dict]:
        """Per bucket, over the steps timed so far: payload, mean device time of the exchange kernel (which includes
        waiting for the peers at its barriers), bus bandwidth 2 (W - 1) / W x bytes / time and that as a fraction
        of `link_gbs` (NVLink per direction per GPU). Synchronises the device."""
        if self.stream is not None:
            torch.cuda.synchronize()
        acc: Dict[int, List[float]] = {}
        for bi, t0, t1 in self._timing_events:
            acc.setdefault(bi, []).append(t0.elapsed_time(t1))
        out = []
        w = max(1, self.world)
        for bi in sorted(acc):
            b = self.buckets[bi]
            nbytes = (b["end"] - b["start"]) * 4
            ms = sum(acc[bi]) / len(acc[bi])
            bus = 2.0 * (w - 1) / w * nbytes / (ms * 1e-3) / 1e9 if ms > 0 else 0.0
            out.append({"bucket": bi, "bytes": nbytes, "launches": len(acc[bi]), "ms": round(ms, 4), "bus_GBs": round(bus, 1),
                        "frac_of_link": round(bus / link_gbs, 3), "tail": bi >= self._first_tail()})
        return out

    def wait_tail(self) -> None:
        """Make the current stream wait for the bucket `finish(defer_tail=True)` left in flight."""
        if self.stream is not None:
            torch.cuda.current_stream().wait_event(self.done_tail)

    # ---- one-off collectives --------------------------------------------------------------------
    def set_weights(self, weights: Optional[Sequence[float]]) -> None:
        """Per-rank contribution weights (sum to 1) for unbalanced shards
        (`weighted_all_reduce_gradients`, ddp.rs:206-225); None = plain average."""
        self.weights = None if weights is None else [float(w) for w in weights]

    def all_reduce_now(self) -> None:
        """Non-overlapped all-reduce of the whole gradient buffer on the current stream."""
        if self.world <= 1:
            return
        for b in self.buckets:
            self._reduce_range(b["start"], b["end"])

    def check(self) -> None:
        if self.symm is not None:
            self.symm.check()

    def guard(self, optimizer) -> None:
        """Tie `optimizer` to the status word of the gradient exchange: fused kernels get the word's
        device address as their `skip` argument, anything else waits for the exchange and checks."""
        if self.symm is None or self.world <= 1:
            return
        if hasattr(optimizer, "set_skip_flag") and getattr(optimizer, "fused", False):
            optimizer.set_skip_flag(self.symm.status_address())
            self.symm.check_async()
        else:
            self.symm.check()

    def reset(self) -> None:
        """Forget the step in flight (after `SymmetricBuffer.recover`)."""
        self.active = False
        _core.GRAD_HOOK["fn"] = None
        for bi in range(len(self.buckets)):
            self.launched[bi] = False
