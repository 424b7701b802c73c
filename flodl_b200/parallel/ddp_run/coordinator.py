"""The coordinator of asynchronous DDP: decides when replicas average their parameters, hands
out data, throttles ranks that run ahead, aggregates per-epoch metrics
(flodl/src/distributed/ddp_run/coordinator/{mod,cpu_avg}.rs).

It never touches a GPU. With the collective backend it only says *when* (`SyncNow`); the
workers then run the averaging kernel among themselves. With the CPU backend it collects
parameter snapshots, averages them on a helper thread (weighted by the batches each rank
contributed; buffers equally) and sends the result back.
"""
from __future__ import annotations

import threading
import time
from typing import Callable, Dict, List, Optional, Sequence, Tuple

import torch

from ... import log
from ..el_che import ElChe
from .chunk_pool import ChunkPool
from .convergence import ConvergenceAction, ConvergenceGuard, DivergenceReport
from .messages import (ApplyPolicy, AverageBackend, AveragedParams, ControlMsg, EpochMetrics, EpochPlan, MetricsMsg,
                       ParamSnapshot, TimingBatch, TimingExiting, TimingSyncAck, TrainedState)


# ---- partition sizing (coordinator/mod.rs:1210-1284) ------------------------------------------------
def equal_sizes(world_size: int, total: int) -> List[int]:
    base, rem = divmod(total, world_size)
    return [base + (1 if r < rem else 0) for r in range(world_size)]


def _largest_first_fill(shares: Sequence[float], total: int) -> List[int]:
    sizes = [int(s * total) for s in shares]
    remaining = max(0, total - sum(sizes))
    for r in sorted(range(len(shares)), key=lambda i: -shares[i]):
        if remaining == 0:
            break
        sizes[r] += 1
        remaining -= 1
    return sizes


def throughput_sizes(el_che: ElChe, total: int) -> List[int]:
    tp = [1.0 / max(m, 0.001) for m in el_che.ms_per_batch()]
    s = sum(tp)
    if s <= 0:
        return equal_sizes(len(tp), total)
    return _largest_first_fill([t / s for t in tp], total)


def ratio_to_sizes(ratios: Sequence[float], total: int) -> List[int]:
    s = float(sum(ratios))
    norm = [r / s for r in ratios] if s > 0 else [1.0 / len(ratios)] * len(ratios)
    return _largest_first_fill(norm, total)


def aggregate_epoch_metrics(epoch: int, msgs: Sequence[MetricsMsg], device_indices: Sequence[int]) -> EpochMetrics:
    """Fold the per-rank (possibly per-chunk) messages of one epoch: batch-weighted loss and
    scalars, slowest rank's time, per-rank throughput and data share (coordinator/mod.rs:1286-1376)."""
    w = len(device_indices)
    batches, samples, loss_sum, time_ms = [0] * w, [0] * w, [0.0] * w, [0.0] * w
    rank_sc: List[Dict[str, List[float]]] = [dict() for _ in range(w)]
    for m in msgs:
        r = min(m.rank, w - 1)
        batches[r] += m.batches_processed
        samples[r] += m.samples_processed
        loss_sum[r] += m.avg_loss * m.batches_processed
        time_ms[r] = max(time_ms[r], m.epoch_ms)
        for k, (s, c) in m.scalars.items():
            e = rank_sc[r].setdefault(k, [0.0, 0])
            e[0] += s
            e[1] += c
    total_b = sum(batches)
    per_rank = [{k: (s / c if c > 0 else 0.0) for k, (s, c) in sc.items()} for sc in rank_sc]
    scalars: Dict[str, float] = {}
    weights: Dict[str, float] = {}
    for r, sc in enumerate(rank_sc):
        for k, (s, c) in sc.items():
            if c > 0:
                scalars[k] = scalars.get(k, 0.0) + (s / c) * batches[r]
                weights[k] = weights.get(k, 0.0) + batches[r]
    for k in scalars:
        if weights.get(k, 0.0) > 0:
            scalars[k] /= weights[k]
    total_s = sum(samples)
    return EpochMetrics(
        epoch=epoch, scalars=scalars, per_rank=per_rank, avg_loss=(sum(loss_sum) / total_b if total_b else 0.0),
        epoch_ms=max(time_ms, default=0.0),
        per_rank_throughput=[samples[r] / time_ms[r] if time_ms[r] > 0 else 0.0 for r in range(w)],
        per_rank_batch_share=[samples[r] / total_s if total_s else 0.0 for r in range(w)], device_indices=list(device_indices))


def _weights(snapshots: Sequence[ParamSnapshot]) -> List[float]:
    total = float(sum(s.batch_count for s in snapshots))
    n = len(snapshots)
    return [s.batch_count / total for s in snapshots] if total > 0 else [1.0 / n] * n


def _average_buffers(snapshots: Sequence[ParamSnapshot]) -> List[torch.Tensor]:
    n = len(snapshots)
    buffers = []
    for i in range(len(snapshots[0].buffers)):
        b0 = snapshots[0].buffers[i].detach().cpu()
        if b0.is_floating_point():
            acc = b0.to(torch.float32) / n
            for s in snapshots[1:]:
                acc.add_(s.buffers[i].detach().to("cpu", torch.float32), alpha=1.0 / n)
            buffers.append(acc.to(b0.dtype))
        else:
            buffers.append(b0.clone())
    return buffers


def average_params(snapshots: Sequence[ParamSnapshot], version: int) -> AveragedParams:
    """Batch-count-weighted mean of parameters, equal-weight mean of buffers, on the host
    (coordinator/cpu_avg.rs:540-599). Tensor operations only; `average_and_divergence` is what the coordinator runs."""
    if not snapshots:
        raise ValueError("average_params: no snapshots")
    weights = _weights(snapshots)
    params = []
    for i in range(len(snapshots[0].params)):
        acc = snapshots[0].params[i].detach().to("cpu", torch.float32) * weights[0]
        for s, w in zip(snapshots[1:], weights[1:]):
            acc.add_(s.params[i].detach().to("cpu", torch.float32), alpha=w)
        params.append(acc.to(snapshots[0].params[i].dtype))
    return AveragedParams(params, _average_buffers(snapshots), version)


def divergence_of(snapshots: Sequence[ParamSnapshot], averaged: AveragedParams) -> DivergenceReport:
    """||pre - post|| / ||post|| per rank, plus the norms for the cosine decomposition."""
    post_sq = sum(float(p.double().pow(2).sum()) for p in averaged.params)
    deltas_sq, pre_sq = [], []
    for s in snapshots:
        d2 = p2 = 0.0
        for a, b in zip(s.params, averaged.params):
            a64 = a.detach().to("cpu", torch.float64)
            d2 += float((a64 - b.double()).pow(2).sum())
            p2 += float(a64.pow(2).sum())
        deltas_sq.append(d2)
        pre_sq.append(p2)
    return _report(snapshots, deltas_sq, pre_sq, post_sq)


def _report(snapshots: Sequence[ParamSnapshot], deltas_sq: Sequence[float], pre_sq: Sequence[float], post_sq: float) -> DivergenceReport:
    post = post_sq ** 0.5
    deltas, pre = [0.0] * len(snapshots), [0.0] * len(snapshots)
    for s, d2, p2 in zip(snapshots, deltas_sq, pre_sq):
        r = min(s.rank, len(snapshots) - 1)
        deltas[r] = (d2 ** 0.5) / post if post > 1e-10 else 0.0
        pre[r] = p2 ** 0.5
    return DivergenceReport(deltas, pre, post)


def average_and_divergence(snapshots: Sequence[ParamSnapshot], version: int) -> Tuple[AveragedParams, DivergenceReport]:
    """The mean and the divergence report of one averaging round. With the native library this is a single threaded pass
    over the snapshots (`cpu_weighted_average`, csrc/runtime/cpu_avg.cpp): every element is read once, the mean written
    once, the norms accumulated on the way, with the interpreter lock released. Without it, the two functions above."""
    if not snapshots:
        raise ValueError("average_and_divergence: no snapshots")
    from ... import _ext
    if _ext.available() and hasattr(_ext.require(), "cpu_weighted_average"):
        per_rank = [[p.detach() if p.device.type == "cpu" else p.detach().cpu() for p in s.params] for s in snapshots]
        params, d2, p2, post2 = _ext.require().cpu_weighted_average(per_rank, _weights(snapshots), True)
        return AveragedParams(list(params), _average_buffers(snapshots), version), _report(snapshots, d2, p2, post2)
    avg = average_params(snapshots, version)
    return avg, divergence_of(snapshots, avg)


class CoordinatorBuilder:
    """Collects the optional settings of a `Coordinator` by name; `build()` makes it."""

    def __init__(self, transport, policy, backend, world_size, total_samples, el_che):
        self._args = (transport, policy, backend, world_size, total_samples, el_che)
        self._kw: Dict[str, object] = {}

    def _set(self, **kw):
        self._kw.update(kw)
        return self

    def progressive(self, enabled: bool): return self._set(progressive=bool(enabled))
    def batch_size(self, bs: int): return self._set(batch_size=int(bs))
    def timeline(self, tl): return self._set(timeline=tl)
    def divergence_threshold(self, t: float): return self._set(divergence_threshold=float(t))
    def no_divergence_guard(self): return self._set(divergence_guard=False)
    def checkpoint_every(self, n: int): return self._set(checkpoint_every=int(n))
    def snapshot_timeout_secs(self, secs: float): return self._set(snapshot_timeout_secs=float(secs))
    def epoch_metrics_tx(self, sink): return self._set(epoch_metrics_sink=sink)
    def metrics_fn(self, f): return self._set(metrics_fn=f)
    def device_indices(self, idx): return self._set(device_indices=list(idx))
    def num_epochs(self, n: int): return self._set(num_epochs=int(n))
    def partition_ratios(self, ratios): return self._set(partition_ratios=None if ratios is None else list(ratios))
    def max_overshoot(self, n: int): return self._set(max_overshoot=int(n))
    def fixed_cadence(self, k: Optional[int]): return self._set(fixed_cadence=k)
    def overshoot_ceiling(self, n: int): return self._set(overshoot_ceiling=int(n))

    def overhead_target(self, target: float):
        self._args[5].with_overhead_target(float(target))          # the cadence controller owns these two
        return self

    def max_anchor(self, m: int):
        self._args[5].with_max_anchor(int(m))
        return self

    def build(self) -> "Coordinator":
        return Coordinator(*self._args, **self._kw)


class Coordinator:
    """State machine driven by `tick()` (or `run()`), fed by the workers' mailboxes."""

    def __init__(self, transport, policy: ApplyPolicy, backend: AverageBackend, world_size: int, total_samples: int,
                 el_che: ElChe, *, batch_size: int = 1, num_epochs: int = 1, progressive: Optional[bool] = None,
                 divergence_threshold: float = 0.05, divergence_guard: bool = True, checkpoint_every: Optional[int] = None,
                 snapshot_timeout_secs: float = 5.0, partition_ratios: Optional[Sequence[float]] = None,
                 max_overshoot: Optional[int] = None, overshoot_ceiling: int = 15, device_indices: Optional[Sequence[int]] = None,
                 metrics_fn: Optional[Callable[[EpochMetrics], None]] = None, epoch_metrics_sink=None, timeline=None,
                 min_chunk_batches: int = 4, fixed_cadence: Optional[int] = None):
        self.t = transport
        self.policy, self.backend = policy, backend
        self.world_size, self.total_samples = int(world_size), int(total_samples)
        self.el_che = el_che
        self.batch_size = max(1, int(batch_size))
        self.num_epochs = int(num_epochs)
        self.progressive = (policy != ApplyPolicy.Sync) if progressive is None else bool(progressive)
        self.convergence_guard = ConvergenceGuard(policy, divergence_guard, divergence_threshold)
        self.checkpoint_every = checkpoint_every
        self.snapshot_timeout_secs = float(snapshot_timeout_secs)
        self.partition_ratios = None if partition_ratios is None else list(partition_ratios)
        self.device_indices = list(device_indices) if device_indices is not None else list(range(world_size))
        self.metrics_fn, self.epoch_metrics_sink, self.timeline = metrics_fn, epoch_metrics_sink, timeline
        self.min_chunk_batches = int(min_chunk_batches)
        self.fixed_cadence = fixed_cadence
        total_batches = self.total_samples // self.batch_size
        self.overshoot_auto = max_overshoot is None
        self.overshoot_initial = max(2, min(5, total_batches // 100)) if max_overshoot is None else int(max_overshoot)
        self.max_overshoot = self.overshoot_initial
        self.overshoot_ceiling = int(overshoot_ceiling)
        w = self.world_size
        self.ctl = [transport.box(f"ctl{r}") for r in range(w)]
        self.tim = [transport.box(f"tim{r}") for r in range(w)]
        self.met = [transport.box(f"met{r}") for r in range(w)]
        self.par = [transport.box(f"par{r}") for r in range(w)]
        self.fin = [transport.box(f"fin{r}") for r in range(w)]
        self.version = 0
        self.avg_count = 0
        self.abort_count = 0
        self.global_step = 0
        self.calibrated = False
        self.active_count = w
        self.steps_since_avg = [0] * w
        self.wall_ms_accum = [0.0] * w
        self.last_step_count = [0] * w
        self.last_batch_ms = [0.0] * w
        self.loss_accum = [0.0] * w
        self.loss_count = [0] * w
        self.throttled = [False] * w
        self.nccl_ack = [True] * w
        self.nccl_sync_step = [0] * w
        self.nccl_sync_divergence: List[Optional[float]] = [None] * w
        self.acks_pending: List[int] = [0] * w      # fixed-cadence mode: SyncAcks seen per rank
        self.last_avg_ms = 0.0
        self.nccl_sync_start: Optional[float] = None
        self.rank_epoch = [0] * w
        self.rank_waiting = [False] * w
        self.last_aggregated_epoch: Optional[int] = None
        self.epoch_plan_cache: Dict[int, List[EpochPlan]] = {}
        self.chunk_pools: Dict[int, ChunkPool] = {}
        self.epoch_buffer: Dict[int, List[MetricsMsg]] = {}
        self.epochs_finished = 0
        # CPU averaging: ("idle",) | ("collecting", {...}) | ("computing", {...})
        self.avg_state: tuple = ("idle",)
        self.stop = threading.Event()
        self.error: Optional[BaseException] = None
        self.failed_ranks: List[int] = []

    @staticmethod
    def builder(transport, policy: ApplyPolicy, backend: AverageBackend, world_size: int, total_samples: int, el_che: ElChe) -> "CoordinatorBuilder":
        """Fluent construction: `Coordinator.builder(...).batch_size(32).num_epochs(3).progressive(True).build()`
        (coordinator/mod.rs:178-300, 389-425)."""
        return CoordinatorBuilder(transport, policy, backend, world_size, total_samples, el_che)

    def drain_timing_blocking(self, timeout_s: float) -> bool:
        """Wait up to `timeout_s` for a timing message, then take everything else that is queued.
        False once the run is being wound down (a rank failed or `stop` is set), true otherwise
        (coordinator/mod.rs:904-915)."""
        deadline = time.monotonic() + max(0.0, float(timeout_s))
        while self.drain_timing() == 0 and time.monotonic() < deadline and not self.stop.is_set():
            time.sleep(0.0005)
        return not self.stop.is_set()

    def debug_state_dump(self, tick: int) -> None:
        """One line of coordinator state at debug verbosity (`-vv`)."""
        if not log.enabled(log.Verbosity.Debug):
            return
        pools = ", ".join(f"e{e}(cur={p.cursor}/{p.total_samples} [" + " ".join(f"{r}:{p.completed[r]}/{p.dispatched[r]}" for r in range(self.world_size)) + "])"
                          for e, p in self.chunk_pools.items())
        log.debug(f"  ddp-state: tick={tick} steps={self.steps_since_avg} wall={[round(w, 1) for w in self.wall_ms_accum]} "
                  f"throttled={self.throttled} nccl_ack={self.nccl_ack} rank_epoch={self.rank_epoch} active={self.active_count} "
                  f"last_agg={self.last_aggregated_epoch} avg#={self.avg_count} pools=[{pools}]")

    # ---- small accessors ------------------------------------------------------------------------
    def is_calibrated(self) -> bool: return self.calibrated
    def is_cpu_averaging(self) -> bool: return self.avg_state[0] != "idle"
    def all_epochs_done(self) -> bool:
        return self.last_aggregated_epoch is not None and self.last_aggregated_epoch + 1 >= self.num_epochs

    def _send(self, rank: int, msg: ControlMsg) -> None:
        try:
            self.ctl[rank].send(msg)
        except Exception as e:  # a dead worker must not take the coordinator down
            log.verbose(f"  ddp: could not deliver {msg.kind} to rank {rank}: {e}")

    def _event(self, kind: str, **kw) -> None:
        if self.timeline is not None:
            self.timeline.event(kind, **kw)

    # ---- data dispatch --------------------------------------------------------------------------
    def compute_partition_sizes(self) -> List[int]:
        if self.fixed_cadence is not None:
            # every rank must reach its k-th, 2k-th, ... step: same number of whole batches each
            per = (self.total_samples // self.batch_size // self.world_size) * self.batch_size
            return [per] * self.world_size
        if self.partition_ratios is not None:
            return ratio_to_sizes(self.partition_ratios, self.total_samples)
        if self.policy == ApplyPolicy.Sync:
            return equal_sizes(self.world_size, self.total_samples)
        if self.el_che.is_calibrated() or self.el_che.has_speed_hint():
            return throughput_sizes(self.el_che, self.total_samples)
        return equal_sizes(self.world_size, self.total_samples)

    def plans_for_epoch(self, epoch: int) -> List[EpochPlan]:
        plans = self.epoch_plan_cache.get(epoch)
        if plans is None:
            sizes = self.compute_partition_sizes()
            plans, off = [], 0
            for s in sizes:
                plans.append(EpochPlan(epoch, off, s))
                off += s
            log.verbose(f"  ddp: epoch {epoch} | partitions {sizes}")
            self.epoch_plan_cache[epoch] = plans
        return plans

    def send_all_plans(self, epoch: int) -> None:
        if self.progressive:
            self._start_epoch_progressive(epoch)
            return
        for rank, plan in enumerate(self.plans_for_epoch(epoch)):
            self.rank_epoch[rank] = epoch
            self.rank_waiting[rank] = False
            self._send(rank, ControlMsg.StartEpoch(plan))

    def _batch_total(self) -> int:
        return (self.total_samples // self.batch_size) * self.batch_size

    def _start_epoch_progressive(self, epoch: int) -> None:
        self.chunk_pools[epoch] = ChunkPool(epoch, self._batch_total(), self.world_size)
        sizes = [self.compute_chunk_batches(r, epoch) for r in range(self.world_size)]
        log.verbose(f"  ddp: epoch {epoch} progressive | initial chunks (batches) {sizes}")
        for rank, b in enumerate(sizes):
            self._dispatch_with_batches(rank, epoch, b)

    def _dispatch_with_batches(self, rank: int, epoch: int, batches: int) -> None:
        samples = batches * self.batch_size
        pool = self.chunk_pools.get(epoch)
        if samples == 0 or pool is None:
            return
        got = pool.take_chunk(samples, rank)
        if got is None:
            return
        self.rank_epoch[rank] = epoch
        self.rank_waiting[rank] = False
        self._send(rank, ControlMsg.StartEpoch(EpochPlan(epoch, got[0], got[1])))

    def compute_chunk_batches(self, rank: int, epoch: int) -> int:
        """Size of the next chunk for `rank`: a probe (a tenth of an equal share, at least 4
        batches) until speeds are known, afterwards the rank's throughput share of what is left,
        shrunk near the end of the epoch so no rank finishes long after the others."""
        pool = self.chunk_pools.get(epoch)
        if pool is None:
            return 0
        remaining = pool.remaining() // self.batch_size
        if remaining == 0:
            return 0
        if not self.el_che.is_calibrated() and not self.el_che.has_speed_hint():
            probe = max(4, self.total_samples // (self.world_size * 10 * self.batch_size))
            return min(probe, remaining)
        counts = self.el_che.batch_counts()
        tot = sum(counts)
        if tot == 0:
            return min(remaining, self.min_chunk_batches)
        import math
        target = math.ceil(remaining * counts[rank] / tot)
        if remaining < target * self.world_size:
            my_ms = self.last_batch_ms[rank]
            if my_ms > 0:
                per_sample = my_ms / self.batch_size
                other = 0.0
                for r in range(self.world_size):
                    if r == rank:
                        continue
                    r_ms = self.last_batch_ms[r] / self.batch_size if self.last_batch_ms[r] > 0 else per_sample
                    other = max(other, pool.in_flight(r) * r_ms)
                if other > my_ms:
                    fill = math.ceil(other / per_sample)
                    target = min(target, -(-fill // self.batch_size))
        return min(max(target, self.min_chunk_batches), remaining)

    def dispatch_next_chunk(self, rank: int) -> None:
        epoch = self.rank_epoch[rank]
        pool = self.chunk_pools.get(epoch)
        if pool is not None and pool.remaining() > 0:
            self._dispatch_with_batches(rank, epoch, self.compute_chunk_batches(rank, epoch))
            return
        first_live = 0 if self.last_aggregated_epoch is None else self.last_aggregated_epoch + 1
        nxt = max(epoch + 1, first_live)
        if nxt >= self.num_epochs:
            return
        if self.backend != AverageBackend.Nccl:
            aggregated = self.last_aggregated_epoch is not None and epoch <= self.last_aggregated_epoch
            if not aggregated:
                planned = self.el_che.batch_counts()[rank]
                if planned > 0 and self.steps_since_avg[rank] >= planned + self.max_overshoot:
                    log.debug(f"  ddp: overshoot gate blocked rank {rank} | steps={self.steps_since_avg[rank]} planned={planned} overshoot={self.max_overshoot}")
                    return
        if nxt not in self.chunk_pools:
            self.chunk_pools[nxt] = ChunkPool(nxt, self._batch_total(), self.world_size)
            log.verbose(f"  ddp: streaming -> epoch {nxt} pool created")
        self._dispatch_with_batches(rank, nxt, self.compute_chunk_batches(rank, nxt))

    def _send_rank_plan(self, rank: int, epoch: int) -> None:
        plans = self.plans_for_epoch(epoch)
        if rank < len(plans):
            self.rank_epoch[rank] = epoch
            self.rank_waiting[rank] = False
            self._send(rank, ControlMsg.StartEpoch(plans[rank]))

    def on_rank_done(self, rank: int, finished_epoch: int) -> None:
        """Async policy, whole-partition dispatch: a rank that finished may start the next epoch
        at most one epoch ahead of the last aggregated one."""
        if self.policy != ApplyPolicy.Async:
            return
        nxt = finished_epoch + 1
        if nxt >= self.num_epochs:
            return
        ok = nxt <= 1 if self.last_aggregated_epoch is None else max(0, nxt - self.last_aggregated_epoch) <= 1
        if ok:
            self._send_rank_plan(rank, nxt)
        else:
            self.rank_waiting[rank] = True

    def on_epoch_aggregated(self, epoch: int) -> None:
        self.last_aggregated_epoch = epoch
        self.epoch_plan_cache.pop(epoch, None)
        if self.checkpoint_every and (epoch + 1) % self.checkpoint_every == 0:
            self._send(0, ControlMsg.Checkpoint(epoch + 1))
        if epoch + 1 >= self.num_epochs:
            self.shutdown_workers()
            return
        if self.progressive:
            self._redispatch_idle()
            return
        if self.policy in (ApplyPolicy.Sync, ApplyPolicy.Cadence):
            self.send_all_plans(epoch + 1)
        else:
            for rank in range(self.world_size):
                if self.rank_waiting[rank] and self.rank_epoch[rank] + 1 < self.num_epochs:
                    self._send_rank_plan(rank, self.rank_epoch[rank] + 1)

    def _redispatch_idle(self) -> None:
        for rank in range(self.world_size):
            if not any(p.in_flight(rank) > 0 for p in self.chunk_pools.values()):
                self.dispatch_next_chunk(rank)

    # ---- timing ---------------------------------------------------------------------------------
    def process_timing_msg(self, msg) -> None:
        if isinstance(msg, TimingBatch):
            r = msg.rank
            self.steps_since_avg[r] += 1
            self.wall_ms_accum[r] += msg.batch_ms
            self.last_step_count[r] = max(self.last_step_count[r], msg.step_count)
            self.last_batch_ms[r] = msg.batch_ms
            if msg.batch_loss > 0.0:
                self.loss_accum[r] += msg.batch_loss
                self.loss_count[r] += 1
            if msg.sync_divergence is not None:
                self.nccl_sync_divergence[r] = msg.sync_divergence
            if not self.nccl_ack[r] and msg.step_count > self.nccl_sync_step[r]:
                self.nccl_ack[r] = True
        elif isinstance(msg, TimingSyncAck):
            r = msg.rank
            self.last_step_count[r] = max(self.last_step_count[r], msg.step_count)
            if msg.divergence is not None:
                self.nccl_sync_divergence[r] = msg.divergence
            if not self.nccl_ack[r] and msg.step_count > self.nccl_sync_step[r]:
                self.nccl_ack[r] = True
            self.acks_pending[r] += 1
        elif isinstance(msg, TimingExiting):
            self.active_count = max(0, self.active_count - 1)
            if msg.error is not None:
                # a replica died: no collective may be started with it, and in a multi-process job
                # nobody else will tell the survivors, so wind the whole run down
                log.msg(f"  ddp: rank {msg.rank} failed ({msg.error}); stopping the run")
                self.failed_ranks.append(msg.rank)
                self.stop.set()

    def drain_timing(self) -> int:
        n = 0
        for box in self.tim:
            while True:
                m = box.try_recv()
                if m is None:
                    break
                self.process_timing_msg(m)
                n += 1
        return n

    def drain_metrics(self) -> List[MetricsMsg]:
        msgs = []
        for box in self.met:
            while True:
                m = box.try_recv()
                if m is None:
                    break
                if self.progressive:
                    pool = self.chunk_pools.get(m.epoch)
                    if pool is not None:
                        pool.mark_completed(m.rank, m.samples_processed)
                    self.epoch_buffer.setdefault(m.epoch, []).append(m)
                    self.dispatch_next_chunk(m.rank)
                else:
                    self.on_rank_done(m.rank, m.epoch)
                    self.epoch_buffer.setdefault(m.epoch, []).append(m)
                msgs.append(m)
        self._try_aggregate_epochs()
        return msgs

    def _emit_epoch(self, epoch: int, msgs: Sequence[MetricsMsg], epoch_ms: Optional[float]) -> None:
        metrics = aggregate_epoch_metrics(epoch, msgs, self.device_indices)
        if epoch_ms is not None:
            metrics.epoch_ms = epoch_ms
        if self.metrics_fn is not None:
            try:
                self.metrics_fn(metrics)
            except Exception as e:
                log.msg(f"  ddp: metrics_fn raised (epoch {epoch}): {e}")
        if self.epoch_metrics_sink is not None:
            self.epoch_metrics_sink.put(metrics)
        self.on_epoch_aggregated(epoch)

    def _try_aggregate_epochs(self) -> None:
        if self.progressive:
            done = []
            for epoch in sorted(self.chunk_pools):
                pool = self.chunk_pools[epoch]
                if not pool.is_epoch_done():
                    break
                done.append((epoch, pool.epoch_elapsed_ms()))
            for epoch, ms in done:
                del self.chunk_pools[epoch]
                msgs = self.epoch_buffer.pop(epoch, None)
                if msgs is not None:
                    log.verbose(f"  ddp: epoch {epoch} progressive complete | {ms:.0f}ms")
                    self._emit_epoch(epoch, msgs, ms)
            return
        expected = self.active_count
        for epoch in sorted(e for e, m in self.epoch_buffer.items() if len(m) >= expected):
            self._emit_epoch(epoch, self.epoch_buffer.pop(epoch), None)

    # ---- when to average ------------------------------------------------------------------------
    def should_average(self) -> bool:
        if self.fixed_cadence is not None or self.world_size < 2:
            return False                       # workers keep their own cadence (poll_fixed_cadence) / nothing to average
        if self.avg_state[0] != "idle":
            return False
        if self.backend == AverageBackend.Nccl and not all(self.nccl_ack):
            return False
        if self.all_epochs_done():
            return False
        if self.active_count < self.world_size:
            return False
        if 0 in self.steps_since_avg:
            return False
        if self.policy == ApplyPolicy.Sync:
            return all(s >= 1 for s in self.steps_since_avg)
        if self.policy == ApplyPolicy.Cadence:
            target = self.el_che.anchor_wall_ms()
            if target > 0.0:
                return min(self.wall_ms_accum) >= target
        counts = self.el_che.batch_counts()
        return all(s >= counts[r] for r, s in enumerate(self.steps_since_avg))

    def check_throttle(self) -> None:
        """CPU backend only: a rank more than `max_batch_diff` batches ahead of the slowest one
        is told to wait for the next averaging."""
        if self.backend == AverageBackend.Nccl:
            return
        max_diff = self.el_che.max_batch_diff()
        if max_diff is None or self.active_count < self.world_size:
            return
        lo = min(self.steps_since_avg)
        for rank, steps in enumerate(self.steps_since_avg):
            if steps > lo + max_diff and not self.throttled[rank]:
                self._send(rank, ControlMsg.Throttle())
                self.throttled[rank] = True
                self._event("Throttle", rank=rank)

    def trigger_averaging(self) -> None:
        self._event("SyncStart")
        if self.backend == AverageBackend.Nccl:
            self.nccl_sync_start = time.perf_counter()
            for r in range(self.world_size):
                self._send(r, ControlMsg.SyncNow())
                self.nccl_sync_step[r] = self.last_step_count[r]
                self.nccl_ack[r] = False
            self.finish_averaging_nccl()
            return
        sync_throttle = self.policy == ApplyPolicy.Sync
        for r in range(self.world_size):
            self._send(r, ControlMsg.RequestParams())
            if sync_throttle:
                self._send(r, ControlMsg.Throttle())
                self.throttled[r] = True
        now = time.perf_counter()
        self.avg_state = ("collecting", dict(snapshots=[], received=[False] * self.world_size, deadline=now + self.snapshot_timeout_secs,
                                             start=now, steps=list(self.steps_since_avg), wall=list(self.wall_ms_accum)))

    def _apply_action(self, action: ConvergenceAction) -> None:
        if action.kind == "Stable":
            if self.overshoot_auto and self.policy == ApplyPolicy.Async:
                cap = max(3, min(10, self.total_samples // self.batch_size // 50))
                self.max_overshoot = min(self.max_overshoot + 1, cap)
        elif action.kind == "NudgeDown":
            old = self.el_che.anchor()
            self.el_che.nudge_anchor_down(action.factor)
            log.verbose(f"  ddp: weight-space divergence nudge, anchor {old} -> {self.el_che.anchor()}")
            if self.overshoot_auto and self.policy == ApplyPolicy.Async:
                self.max_overshoot = self.overshoot_initial
        if self.policy == ApplyPolicy.Async:
            self.max_overshoot = min(self.max_overshoot, self.overshoot_ceiling)

    def _after_average(self, old_anchor: int, cycle_batches: int, dur_ms: float) -> None:
        self.version += 1
        self.avg_count += 1
        self._event("SyncEnd", duration_ms=dur_ms)
        if self.el_che.anchor() != old_anchor:
            self._event("AnchorChanged", **{"from": old_anchor, "to": self.el_che.anchor()})
        self.global_step += cycle_batches
        for r in range(self.world_size):
            self._send(r, ControlMsg.SetGlobalStep(self.global_step))

    def finish_averaging_nccl(self, steps: Optional[List[int]] = None, wall: Optional[List[float]] = None) -> None:
        steps = self.steps_since_avg if steps is None else steps
        wall = self.wall_ms_accum if wall is None else wall
        old_anchor = self.el_che.anchor()
        if any(ms > 0.0 for ms in wall):
            self.el_che.report_timing(wall, steps, self.last_avg_ms)
            self.last_avg_ms = 0.0
            if self.el_che.is_calibrated():
                self.calibrated = True
        report = DivergenceReport([d or 0.0 for d in self.nccl_sync_divergence])
        self._apply_action(self.convergence_guard.report(report))
        dur = (time.perf_counter() - self.nccl_sync_start) * 1e3 if self.nccl_sync_start is not None else 0.0
        self.nccl_sync_start = None
        self._after_average(old_anchor, sum(steps), dur)
        log.verbose(f"  ddp: collective averaging #{self.avg_count} complete (v{self.version}, global_step={self.global_step})")
        w = self.world_size
        if steps is self.steps_since_avg:
            self.steps_since_avg = [0] * w
            self.wall_ms_accum = [0.0] * w
        else:
            self.steps_since_avg = [max(0, s - t) for s, t in zip(self.steps_since_avg, steps)]
            self.wall_ms_accum = [max(0.0, a - b) for a, b in zip(self.wall_ms_accum, wall)]
        self.throttled = [False] * w
        self.loss_accum = [0.0] * w
        self.loss_count = [0] * w
        self.nccl_sync_divergence = [None] * w
        if self.progressive:
            self._redispatch_idle()

    def poll_fixed_cadence(self) -> None:
        """Fixed-cadence mode: workers average every K local steps without being told; once every
        rank has acknowledged a round the coordinator does the bookkeeping for it."""
        if self.fixed_cadence is None:
            return
        while all(a > 0 for a in self.acks_pending):
            for r in range(self.world_size):
                self.acks_pending[r] -= 1
            k = self.fixed_cadence
            steps = [min(k, s) for s in self.steps_since_avg]
            wall = [a * (t / s) if s > 0 else 0.0 for a, s, t in zip(self.wall_ms_accum, self.steps_since_avg, steps)]
            self.finish_averaging_nccl(steps, wall)

    def finish_averaging_cpu(self, avg_ms: float, steps: List[int], wall: List[float], report: Optional[DivergenceReport]) -> None:
        self.last_avg_ms = avg_ms
        old_anchor = self.el_che.anchor()
        if any(ms > 0.0 for ms in wall):
            self.el_che.report_timing(wall, steps, self.last_avg_ms)
            self.last_avg_ms = 0.0
            if self.el_che.is_calibrated():
                self.calibrated = True
        self._apply_action(self.convergence_guard.report(report) if report is not None else ConvergenceAction.Stable())
        self._event("CpuAvgEnd", duration_ms=avg_ms)
        self._after_average(old_anchor, sum(steps), avg_ms)
        log.verbose(f"  ddp: CPU averaging #{self.avg_count} complete (v{self.version}, {avg_ms:.1f}ms, global_step={self.global_step})")
        self.steps_since_avg = [max(0, s - t) for s, t in zip(self.steps_since_avg, steps)]
        self.wall_ms_accum = [max(0.0, a - b) for a, b in zip(self.wall_ms_accum, wall)]
        self.throttled = [False] * self.world_size
        if self.progressive:
            self._redispatch_idle()

    def _drain_param_boxes(self) -> List[ParamSnapshot]:
        out = []
        for box in self.par:
            while True:
                s = box.try_recv()
                if s is None:
                    break
                out.append(s)
        return out

    def poll_cpu_averaging(self) -> None:
        kind = self.avg_state[0]
        if kind == "idle":
            return
        st = self.avg_state[1]
        if kind == "collecting":
            for snap in self._drain_param_boxes():
                if snap.rank < self.world_size and not st["received"][snap.rank]:
                    st["received"][snap.rank] = True
                    st["snapshots"].append(snap)
            if len(st["snapshots"]) >= self.world_size:
                self._event("CpuAvgStart")
                version = self.version + 1
                result: dict = {}
                snaps = st["snapshots"]

                def work():
                    try:
                        result["avg"], result["div"] = average_and_divergence(snaps, version)
                    except BaseException as e:  # surfaced by the poll below
                        result["err"] = e

                th = threading.Thread(target=work, name="cpu-avg-compute", daemon=True)
                th.start()
                self.avg_state = ("computing", dict(thread=th, result=result, start=st["start"], steps=st["steps"], wall=st["wall"]))
            elif time.perf_counter() >= st["deadline"]:
                missing = [r for r, got in enumerate(st["received"]) if not got]
                self.abort_count += 1
                log.verbose(f"  ddp: CPU averaging timeout, missing ranks: {missing} (abort #{self.abort_count}, will retry)")
                self.avg_state = ("idle",)
                self._drain_param_boxes()
            return
        th = st["thread"]
        if th.is_alive():
            return
        self.avg_state = ("idle",)
        res = st["result"]
        if "err" in res:
            raise RuntimeError(f"CPU averaging failed: {res['err']!r}")
        avg_ms = (time.perf_counter() - st["start"]) * 1e3
        for r in range(self.world_size):
            self._send(r, ControlMsg.Update(res["avg"]))
        self.finish_averaging_cpu(avg_ms, st["steps"], st["wall"], res.get("div"))

    def drain_avg_state(self) -> None:
        """Discard an averaging round that is still in flight (used on the way out)."""
        kind = self.avg_state[0]
        if kind == "computing":
            self.avg_state[1]["thread"].join(timeout=30)
        self.avg_state = ("idle",)
        self._drain_param_boxes()

    # ---- main loop ------------------------------------------------------------------------------
    def tick(self) -> List[MetricsMsg]:
        self.drain_timing()
        self.poll_fixed_cadence()
        self.check_throttle()
        self.poll_cpu_averaging()
        metrics = self.drain_metrics()
        if self.should_average():
            self.drain_timing()        # catch a last-second Exiting before sending SyncNow
            if self.should_average():
                self.trigger_averaging()
        return metrics

    def run(self, poll_s: float = 0.001) -> Optional[TrainedState]:
        """Until every epoch is aggregated, every worker has left, or `stop` is set; then shut the
        workers down and return the average of their final snapshots. An idle coordinator sleeps
        `poll_s` between looks at its queues: it shares the interpreter lock with the worker thread of
        its process, and a tighter loop (measured at 0.1 ms) slowed that worker's launches several-fold."""
        self.send_all_plans(0)
        try:
            while not self.stop.is_set():
                got = self.drain_timing()
                if self.active_count == 0 or self.all_epochs_done():
                    break
                for m in self.tick():
                    log.verbose(f"  ddp: rank {m.rank} epoch {m.epoch} | loss={m.avg_loss:.4f} batches={m.batches_processed} time={m.epoch_ms:.0f}ms")
                if not got:
                    time.sleep(poll_s)
        except BaseException as e:
            self.error = e
            self.stop.set()
        self.drain_avg_state()
        self.shutdown_workers()
        state = self.collect_final_state()
        if state is None and self.error is not None:
            raise self.error
        return state

    def collect_final_state(self, timeout_s: float = 10.0) -> Optional[TrainedState]:
        snaps = []
        for rank, box in enumerate(self.fin):
            s = box.recv(timeout=0.05 if rank in self.failed_ranks else timeout_s)
            if s is None:
                log.verbose(f"  ddp: timeout waiting for final snapshot from rank {rank}")
            else:
                snaps.append(s)
        if not snaps:
            return None
        try:
            avg = average_params(snaps, self.version)
            return TrainedState(avg.params, avg.buffers)
        except Exception:
            return TrainedState([p.detach().cpu() for p in snaps[0].params], [b.detach().cpu() for b in snaps[0].buffers])

    def shutdown_workers(self) -> None:
        for r in range(self.world_size):
            self._send(r, ControlMsg.Shutdown())
