"""`GpuWorker`: one replica's training loop under asynchronous DDP
(flodl/src/distributed/ddp_run/worker.rs).

A worker owns a model replica, its optimizer and a `TrainEngine` that runs without gradient
exchange. It takes `EpochPlan`s (a slice of the epoch's global permutation) from the coordinator,
trains batch by batch, reports the time and loss of every batch, and between batches obeys
control messages: average now (`SyncNow`: the fused peer-memory averaging kernel, or a
`torch.distributed` all-reduce where that does not apply), send a snapshot / load an average
(`RequestParams` / `Update`, CPU backend), wait (`Throttle`), checkpoint, stop.

Nothing here forces a host-device sync per batch: the loss and the two divergence sums are
copied into pinned host slots, batch times come from CUDA events, and both are read once the
event that follows them has completed. The reference reads `loss.item()` every batch
(worker.rs:430-470).
"""
from __future__ import annotations

import time
from collections import deque, namedtuple
from typing import Callable, List, Optional, Sequence

import torch

from ... import log
from .. import comm as _comm
from ..engine import TrainEngine
from .messages import (ApplyPolicy, AveragedParams, ControlMsg, EpochPlan, MetricsMsg, ParamSnapshot, TimingBatch,
                       TimingExiting, TimingSyncAck, WorkerConfig, drain_scalars, make_partition)

_RING = 64


class _SchedAdapter:
    """Learning rate for the engine: scheduler evaluated at global_step + steps since the last
    averaging (worker.rs:648-651)."""

    def __init__(self, worker: "GpuWorker", sched):
        self.w, self.sched = worker, sched

    def lr(self, _step: int) -> float:
        return self.sched.lr(self.w.global_step + self.w.steps_since_avg)


WorkerEndpoints = namedtuple("WorkerEndpoints", "timing_tx metrics_tx param_tx final_param_tx control_rx")
WorkerChannels = namedtuple("WorkerChannels", "timing_rx metrics_rx param_rx final_param_rx control_tx")


class GpuWorker:
    def __init__(self, config: WorkerConfig, model_factory: Callable, optim_factory: Callable, dataset, transport,
                 checkpoint_fn: Optional[Callable] = None, collective: bool = False, comm_timeout_s: float = 30.0):
        self.cfg = config
        self.rank_, self.world = config.rank, config.world_size
        self.device_ = torch.device(config.device)
        self.batch_size = config.batch_size
        self.dataset = dataset
        self.base_seed = config.seed
        self.policy = config.policy
        self.checkpoint_fn = checkpoint_fn
        self.collective = bool(collective) and _comm.world_size() > 1
        self.model_ = model_factory(self.device_)
        if config.initial_params is not None:
            with torch.no_grad():
                for p, src in zip(self.model_.parameters(), config.initial_params):
                    p.t.copy_(src.to(p.t.device))
                for b, src in zip(self.model_.buffers(), config.initial_buffers or []):
                    b.get().copy_(src.to(b.get().device))
        self.model_.set_training(True)
        self.engine = TrainEngine(self.model_, optim_factory, max_grad_norm=config.max_grad_norm, grad_sync=False,
                                  param_staging=self.collective, sync_params=self.collective, comm_timeout_s=comm_timeout_s)
        self.optimizer = self.engine.optimizer
        self.cuda = self.device_.type == "cuda"
        self.use_graph = bool(config.cuda_graph) and self.cuda
        # mailboxes
        r = self.rank_
        self.ctl, self.tim, self.met = transport.box(f"ctl{r}"), transport.box(f"tim{r}"), transport.box(f"met{r}")
        self.par, self.fin = transport.box(f"par{r}"), transport.box(f"fin{r}")
        # counters
        self.local_step_ = 0
        self.steps_since_avg = 0
        self.global_step = 0
        self.current_version_ = 0
        self.current_epoch_ = -1
        self.lr_scale = 1.0
        self.scheduler = None
        self.pending_plan: Optional[EpochPlan] = None
        self.partition: List[int] = []
        self.fixed_cadence = config.fixed_cadence if self.collective else None
        # deferred readback
        self._host = torch.zeros(_RING, 3, dtype=torch.float32, pin_memory=self.cuda) if self.cuda else None
        self._inflight: deque = deque()      # (slot, start_event, end_event, step_count, has_div)
        self._last_event = None
        self._pending_div = False
        self._loss_sum = 0.0
        self._loss_n = 0
        self._shutdown_seen = False
        self._averaging_broken = False       # set when an averaging collective failed because a peer was gone

    @classmethod
    def new(cls, config: WorkerConfig, model_factory: Callable, optim_factory: Callable, dataset, transport, **kw) -> "GpuWorker":
        return cls(config, model_factory, optim_factory, dataset, transport, **kw)

    @staticmethod
    def channels(transport, rank: int):
        """The five mailboxes of worker `rank`, as (worker side, coordinator side): the worker sends on
        `timing, metrics, params, final_params` and receives on `control`; the coordinator holds the
        other ends. Both sides are views of the same named boxes of `transport`, which is how a worker
        built later in its own thread (or process) finds them (worker.rs:157-173)."""
        boxes = {k: transport.box(f"{k}{rank}") for k in ("tim", "met", "par", "fin", "ctl")}
        worker_side = WorkerEndpoints(boxes["tim"], boxes["met"], boxes["par"], boxes["fin"], boxes["ctl"])
        coord_side = WorkerChannels(boxes["tim"], boxes["met"], boxes["par"], boxes["fin"], boxes["ctl"])
        return worker_side, coord_side

    # ---- accessors (worker.rs:371-436) ----------------------------------------------------------
    def rank(self) -> int: return self.rank_
    def device(self): return self.device_
    def local_step(self) -> int: return self.local_step_
    def current_version(self) -> int: return self.current_version_
    def current_epoch(self) -> int: return self.current_epoch_
    def model(self): return self.model_
    def current_lr(self) -> float: return self.optimizer.lr()
    def set_lr(self, lr: float) -> None: self.optimizer.set_lr(lr)
    def scale_lr(self, factor: float) -> None: self.optimizer.scale_lr(factor)
    def set_lr_scale(self, scale: float) -> None:
        self.lr_scale = float(scale)
        self.engine.lr_scale = self.lr_scale

    def set_scheduler(self, sched) -> None:
        self.scheduler = sched
        self.engine.set_scheduler(_SchedAdapter(self, sched), self.lr_scale)

    # ---- one batch ------------------------------------------------------------------------------
    def train_step(self, batch: Sequence[torch.Tensor], train_fn: Callable) -> None:
        """Forward, backward, clip, optimizer on one batch. Timing and loss are reported to the
        coordinator as soon as the device has finished the batch (see `_flush`)."""
        if self.cuda:
            if self._last_event is None:
                self._last_event = torch.cuda.Event(enable_timing=True)
                self._last_event.record()
            if self.use_graph:
                if self.engine._graph is None:
                    self.engine.capture(lambda *xs: train_fn(self.model_, list(xs)), list(batch))
                    self._last_event = torch.cuda.Event(enable_timing=True)
                    self._last_event.record()
                loss = self.engine.replay(list(batch))
            else:
                loss = self.engine.step(lambda: train_fn(self.model_, list(batch)))
            if len(self._inflight) >= _RING - 1:
                self._flush(block=True)
            slot = self.local_step_ % _RING
            self._host[slot, 0:1].copy_(loss.detach().reshape(1).float(), non_blocking=True)
            has_div = self._pending_div
            if has_div:
                self._host[slot, 1:3].copy_(self._div_out, non_blocking=True)
                self._pending_div = False
            end = torch.cuda.Event(enable_timing=True)
            end.record()
            self.local_step_ += 1
            self.steps_since_avg += 1
            self._inflight.append((slot, self._last_event, end, self.local_step_, has_div))
            self._last_event = end
            self._flush(block=False)
        else:
            t0 = time.perf_counter()
            loss = self.engine.step(lambda: train_fn(self.model_, list(batch)))
            lv = float(loss)
            ms = (time.perf_counter() - t0) * 1e3
            self.local_step_ += 1
            self.steps_since_avg += 1
            div = None
            if self._pending_div:
                d2, n2 = (float(x) for x in self._div_out)
                div = (d2 ** 0.5) / (n2 ** 0.5) if n2 > 0 else 0.0
                self._pending_div = False
            self._report(ms, lv, self.local_step_, div)

    def _report(self, ms: float, loss: float, step_count: int, div: Optional[float]) -> None:
        self._loss_sum += loss
        self._loss_n += 1
        self.tim.send(TimingBatch(self.rank_, ms, step_count, None, loss, div))

    def _flush(self, block: bool) -> None:
        """Report every batch whose trailing event has completed (all of them when `block`)."""
        while self._inflight:
            slot, a, b, step_count, has_div = self._inflight[0]
            if not b.query():
                if not block:
                    return
                b.synchronize()
            self._inflight.popleft()
            row = self._host[slot]
            div = None
            if has_div:
                d2, n2 = float(row[1]), float(row[2])
                div = (d2 ** 0.5) / (n2 ** 0.5) if n2 > 0 else 0.0
            self._report(a.elapsed_time(b), float(row[0]), step_count, div)

    # ---- averaging ------------------------------------------------------------------------------
    def sync_now(self) -> None:
        """Average parameters (and floating-point buffers) with the other replicas, in place."""
        self._div_out = self.engine.average_params()
        self._pending_div = True
        bufs = [b.get() for b in self.model_.buffers() if b.get().is_floating_point() and b.get().numel() > 0]
        if bufs and self.collective:
            pack = torch.cat([b.reshape(-1).float() for b in bufs])
            torch.distributed.all_reduce(pack, torch.distributed.ReduceOp.SUM)
            pack.div_(_comm.world_size())
            off = 0
            with torch.no_grad():
                for b in bufs:
                    b.copy_(pack[off:off + b.numel()].view(b.shape))
                    off += b.numel()
        self.steps_since_avg = 0
        self.local_step_ += 1
        self.current_version_ += 1
        self.tim.send(TimingSyncAck(self.rank_, self.local_step_, None))

    def snapshot_params(self) -> ParamSnapshot:
        with torch.no_grad():
            params = [p.t.detach().to("cpu", copy=True) for p in self.model_.parameters()]
            buffers = [b.get().detach().to("cpu", copy=True) for b in self.model_.buffers()]
        return ParamSnapshot(self.rank_, params, buffers, self.steps_since_avg)

    def load_averaged(self, avg: AveragedParams) -> None:
        with torch.no_grad():
            for p, src in zip(self.model_.parameters(), avg.params):
                p.t.copy_(src.to(p.t.device, non_blocking=True))
            for b, src in zip(self.model_.buffers(), avg.buffers):
                b.get().copy_(src.to(b.get().device, non_blocking=True))
        self.engine.flat.refresh_shadow()
        self.current_version_ = avg.version

    # ---- control plane --------------------------------------------------------------------------
    def handle_control(self) -> bool:
        """Process everything that is waiting; True = shut down."""
        while True:
            msg = self.ctl.try_recv()
            if msg is None:
                return False
            if self.dispatch_control(msg):
                return True

    def dispatch_control(self, msg: ControlMsg) -> bool:
        k = msg.kind
        if k == "RequestParams":
            if self.cuda:
                self._flush(block=True)
            self.par.send(self.snapshot_params())
        elif k == "Update":
            self.load_averaged(msg.payload)
            self.steps_since_avg = 0
        elif k == "SyncNow":
            if self.fixed_cadence is None and not self._averaging_broken:
                log.debug(f"  ddp-worker: rank {self.rank_} SyncNow (step={self.local_step_}, epoch={self.current_epoch_})")
                try:
                    self.sync_now()
                except RuntimeError as e:
                    # A peer left between the coordinator's decision and this collective (its `Exiting` and our `SyncNow` crossed).
                    # The weights are this rank's own again; it trains on alone, answers the coordinator so that nobody waits for
                    # an acknowledgement, and takes part in no further averaging (the group is no longer whole).
                    log.msg(f"  ddp: rank {self.rank_}: averaging failed ({type(e).__name__}: {str(e)[:120]}); continuing without it")
                    self._averaging_broken = True
                    self.steps_since_avg = 0
                    self.tim.send(TimingSyncAck(self.rank_, self.local_step_, None))
        elif k == "StartEpoch":
            self.pending_plan = msg.payload
        elif k == "Throttle":
            while True:
                m = self.ctl.recv(timeout=None)
                if m.kind == "Throttle":
                    continue
                releases = m.kind in ("SyncNow", "Update", "Shutdown")
                shutdown = self.dispatch_control(m)
                if shutdown or releases:
                    return shutdown
        elif k == "SetGlobalStep":
            self.global_step = int(msg.payload)
        elif k == "Checkpoint":
            if self.checkpoint_fn is not None:
                try:
                    self.checkpoint_fn(int(msg.payload), self.model_)
                except Exception as e:
                    log.msg(f"  ddp: checkpoint failed (v{msg.payload}): {e}")
        elif k == "Shutdown":
            self._shutdown_seen = True
            return True
        return False

    def wait_for_epoch_plan(self) -> Optional[EpochPlan]:
        while True:
            if self.pending_plan is not None:
                plan, self.pending_plan = self.pending_plan, None
                return plan
            if self.cuda and self._inflight:
                self._flush(block=True)       # the coordinator needs these before it can decide anything
            msg = self.ctl.recv(timeout=0.05)
            if msg is None:
                continue
            if msg.kind == "StartEpoch":
                return msg.payload
            if msg.kind == "Shutdown":
                self._shutdown_seen = True
                return None
            if self.dispatch_control(msg):
                return None

    def report_epoch(self, avg_loss: float, batches: int, epoch_ms: float) -> None:
        self.met.send(MetricsMsg(self.rank_, self.current_epoch_, avg_loss, batches, epoch_ms, batches * self.batch_size, drain_scalars()))

    def run_epoch_plan(self, plan: EpochPlan, train_fn: Callable) -> bool:
        """Train the plan's slice; True = shutdown received on the way."""
        self.current_epoch_ = plan.epoch
        self.partition = make_partition(plan.partition_offset, plan.partition_size, len(self.dataset), plan.epoch, self.base_seed)
        num_batches = len(self.partition) // self.batch_size
        if num_batches == 0:
            self.report_epoch(0.0, 0, 0.0)
            return False
        if self.cfg.timeline is not None:
            self.cfg.timeline.event("EpochStart", epoch=plan.epoch)
        t0 = time.perf_counter()
        self._loss_sum, self._loss_n = 0.0, 0
        for bi in range(num_batches):
            idx = self.partition[bi * self.batch_size:(bi + 1) * self.batch_size]
            batch = self.dataset.get_batch(idx)
            if self.cuda:
                batch = [t.to(self.device_, non_blocking=True) for t in batch]
            self.train_step(batch, train_fn)
            if self.fixed_cadence is not None and self.steps_since_avg >= self.fixed_cadence and not self._averaging_broken:
                try:
                    self.sync_now()
                except RuntimeError as e:       # a peer is gone (see `dispatch_control`): train on alone
                    log.msg(f"  ddp: rank {self.rank_}: averaging failed ({type(e).__name__}: {str(e)[:120]}); continuing without it")
                    self._averaging_broken = True
                    self.steps_since_avg = 0
            if self.handle_control():
                return True
        if self.cuda:
            self._flush(block=True)
        epoch_ms = (time.perf_counter() - t0) * 1e3
        avg_loss = self._loss_sum / max(1, self._loss_n)
        if self.cfg.timeline is not None:
            self.cfg.timeline.event("EpochEnd", epoch=plan.epoch, loss=avg_loss)
        self.report_epoch(avg_loss, num_batches, epoch_ms)
        return False

    # ---- exit -----------------------------------------------------------------------------------
    def send_final_snapshot(self) -> None:
        if self.cuda:
            self._flush(block=True)
        self.fin.send(self.snapshot_params())

    def report_exiting(self) -> None:
        self.tim.send(TimingExiting(self.rank_))

    def report_timing(self, batch_ms: float, param_norm: Optional[float], batch_loss: float, sync_divergence: Optional[float] = None) -> None:
        """Send one batch's timing report to the coordinator now (worker.rs:776-791)."""
        self.tim.send(TimingBatch(self.rank_, float(batch_ms), self.local_step_, param_norm, float(batch_loss), sync_divergence))

    def abort_nccl(self) -> None:
        """Reference name of `abort_collectives` (worker.rs:820-830)."""
        self.abort_collectives()

    def abort_collectives(self) -> None:
        """Make any device-side wait of this rank's averaging kernels return at once."""
        for s in (self.engine.symm_params, self.engine.symm_stage):
            if s is not None:
                s.abort()

    def drain_until_shutdown(self, timeout_s: float = 30.0) -> None:
        if self._shutdown_seen:
            return
        deadline = time.monotonic() + timeout_s
        while time.monotonic() < deadline:
            msg = self.ctl.recv(timeout=0.1)
            if msg is None:
                continue
            if msg.kind == "Shutdown":
                return
            if msg.kind == "SyncNow":
                continue                     # a collective with departed peers would never finish
            if msg.kind in ("RequestParams", "StartEpoch", "Throttle"):
                continue
            if self.dispatch_control(msg):
                return

    def run(self, train_fn: Callable, epoch_fn: Optional[Callable] = None, stop=None) -> None:
        """The worker thread's body (ddp_run/orchestrator.rs:368-440)."""
        self.current_epoch_ = -1
        while stop is None or not stop.is_set():
            plan = self.wait_for_epoch_plan()
            if plan is None:
                break
            if plan.epoch != self.current_epoch_:
                self.current_epoch_ = plan.epoch
                if epoch_fn is not None:
                    epoch_fn(plan.epoch, self)
            if self.run_epoch_plan(plan, train_fn):
                break
        self.send_final_snapshot()
        self.report_exiting()
        self.drain_until_shutdown()
