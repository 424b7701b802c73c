"""Asynchronous DDP on CPU: pure pieces, the coordinator driven by hand-made messages (no
workers), workers as threads with host averaging, and process-per-rank runs over gloo, including
a worker that fails on the host."""
import threading
import time

import pytest
import torch

from flodl_b200 import nn
from flodl_b200.data import TensorDataSet
from flodl_b200.graph import FlowBuilder
from flodl_b200.parallel.ddp import Trainer
from flodl_b200.parallel.ddp_run import (ApplyPolicy, AverageBackend, AveragedParams, ChunkPool, ControlMsg, ConvergenceGuard,
                                         Coordinator, DdpRunConfig, DivergenceReport, EpochPlan, GpuWorker, LocalTransport,
                                         MetricsMsg, ParamSnapshot, StoreTransport, TimingBatch, TimingExiting, TimingSyncAck,
                                         WorkerConfig, aggregate_epoch_metrics, average_params, divergence_of, drain_scalars,
                                         equal_sizes, make_partition, ratio_to_sizes, record_scalar)
from flodl_b200.parallel.el_che import ElChe
from test_ddp_cpu import run_ranks


# ---- pure pieces ------------------------------------------------------------------------------------
def test_chunk_pool():
    pool = ChunkPool(0, 100, 2)
    assert pool.take_chunk(80, 0) == (0, 80)
    assert pool.take_chunk(50, 1) == (80, 20)
    assert pool.take_chunk(10, 0) is None and pool.remaining() == 0
    assert not pool.is_epoch_done()
    pool.mark_completed(0, 80)
    assert pool.in_flight(0) == 0 and pool.in_flight(1) == 20
    pool.mark_completed(1, 20)
    assert pool.is_epoch_done()


def test_partition_sizing():
    assert equal_sizes(3, 10) == [4, 3, 3]
    assert ratio_to_sizes([3.0, 1.0], 10) == [8, 2] or ratio_to_sizes([3.0, 1.0], 10) == [7, 3]
    assert sum(ratio_to_sizes([0.3, 0.3, 0.4], 101)) == 101
    assert ratio_to_sizes([0.0, 0.0], 10) == [5, 5]


def test_make_partition_is_a_slice_of_one_permutation():
    a = make_partition(0, 40, 100, 3, 42)
    b = make_partition(40, 60, 100, 3, 42)
    assert sorted(a + b) == list(range(100))
    assert make_partition(0, 40, 100, 4, 42) != a            # another epoch, another order
    assert make_partition(0, 40, 100, 3, 42) == a


def test_convergence_guard():
    g = ConvergenceGuard(ApplyPolicy.Cadence, True, 0.05)
    acts = [g.report(DivergenceReport([d])).kind for d in (0.01, 0.02, 0.04, 0.06, 0.08)]
    assert acts == ["Stable", "Stable", "Stable", "SuppressGrowth", "SuppressGrowth"]
    assert len(g.history()) == 5
    g.report(DivergenceReport([0.01]))
    assert len(g.history()) == 5 and g.history()[-1] == 0.01
    assert ConvergenceGuard(ApplyPolicy.Sync, True, 0.0).report(DivergenceReport([9.0])).kind == "Stable"
    off = ConvergenceGuard(ApplyPolicy.Async, False, 0.0)
    for d in (1.0, 2.0, 3.0):
        assert off.report(DivergenceReport([d])).kind == "Stable"


def test_divergence_report_decomposition():
    r = DivergenceReport([0.001], [10.0], 10.0)
    assert r.cosine_similarities()[0] > 0.999
    assert DivergenceReport([0.01, 0.02], [10.5, 9.8], 10.0).magnitude_shifts() == pytest.approx([0.5, -0.2])
    assert DivergenceReport([0.1]).cosine_similarities() is None
    assert DivergenceReport([]).max_relative_delta() == 0.0


def test_record_scalar_accumulates_per_thread():
    drain_scalars()
    record_scalar("acc", 1.0)
    record_scalar("acc", 3.0)
    seen = {}
    th = threading.Thread(target=lambda: seen.update(drain_scalars()))
    th.start()
    th.join()
    assert seen == {}
    assert drain_scalars() == {"acc": (4.0, 2)} and drain_scalars() == {}


def test_average_params_weights_by_batch_count():
    s0 = ParamSnapshot(0, [torch.zeros(3)], [torch.zeros(2), torch.tensor(5)], 1)
    s1 = ParamSnapshot(1, [torch.full((3,), 4.0)], [torch.full((2,), 2.0), torch.tensor(7)], 3)
    avg = average_params([s0, s1], 9)
    assert avg.version == 9 and avg.params[0].tolist() == [3.0, 3.0, 3.0]
    assert avg.buffers[0].tolist() == [1.0, 1.0] and int(avg.buffers[1]) == 5
    div = divergence_of([s0, s1], avg)
    assert div.deltas[0] == pytest.approx(1.0) and div.deltas[1] == pytest.approx(1.0 / 3.0)


def test_aggregate_epoch_metrics():
    msgs = [MetricsMsg(0, 2, 1.0, 10, 100.0, 80, {"acc": (5.0, 10)}), MetricsMsg(1, 2, 2.0, 30, 200.0, 240, {"acc": (27.0, 30)})]
    m = aggregate_epoch_metrics(2, msgs, [0, 1])
    assert m.avg_loss == pytest.approx(1.75) and m.epoch_ms == 200.0
    assert m.scalars["acc"] == pytest.approx((0.5 * 10 + 0.9 * 30) / 40)
    assert m.per_rank_batch_share == pytest.approx([0.25, 0.75]) and m.per_rank_throughput == pytest.approx([0.8, 1.2])


def test_run_config_defaults():
    c = DdpRunConfig()
    assert c.snapshot_timeout_secs == 5 and c.lr_scale_ratio == 1.0 and c.max_anchor is None and not c.no_divergence_guard
    assert DdpRunConfig.new().with_anchor(8).with_max_anchor(8).anchor == 8


# ---- coordinator with hand-made messages ----------------------------------------------------------
def coord(policy, backend=AverageBackend.Nccl, world=2, total=1000, **kw):
    t = LocalTransport()
    kw.setdefault("progressive", False)
    c = Coordinator(t, policy, backend, world, total, ElChe(world, kw.pop("anchor", 10)), batch_size=kw.pop("batch_size", 10),
                    num_epochs=kw.pop("num_epochs", 5), **kw)
    return c, t


def feed(c, t, rank, n, ms=10.0, start=1):
    for i in range(n):
        t.box(f"tim{rank}").send(TimingBatch(rank, ms, start + i, None, 1.0))
    c.drain_timing()


def controls(t, rank):
    out = []
    while True:
        m = t.box(f"ctl{rank}").try_recv()
        if m is None:
            return out
        out.append(m)


def test_should_average_sync_needs_every_rank():
    c, t = coord(ApplyPolicy.Sync)
    assert not c.should_average()
    feed(c, t, 0, 1)
    assert not c.should_average()
    feed(c, t, 1, 1)
    assert c.should_average()


def test_should_average_cadence_uses_wall_time_once_calibrated():
    c, t = coord(ApplyPolicy.Cadence)
    feed(c, t, 0, 9)
    feed(c, t, 1, 12)
    assert not c.should_average()                 # uncalibrated: batch-count fallback, rank 0 at 9 < 10
    feed(c, t, 0, 1, start=10)
    assert c.should_average()
    c.el_che.report_timing([200.0, 100.0], [10, 10], 1.0)      # 20 ms and 10 ms per batch
    c.steps_since_avg, c.wall_ms_accum = [5, 9], [100.0, 90.0]
    target = c.el_che.anchor_wall_ms()
    assert target > 0 and not c.should_average()
    c.wall_ms_accum = [target + 1, target + 1]
    assert c.should_average()
    c.wall_ms_accum = [target + 50, target - 1]              # the slower accumulation governs
    assert not c.should_average()


def test_should_average_async_batch_counts():
    c, t = coord(ApplyPolicy.Async)
    c.el_che.report_timing([200.0, 100.0], [10, 10], 1.0)
    counts = c.el_che.batch_counts()
    c.steps_since_avg = [counts[0], counts[1] - 1]
    assert not c.should_average()
    c.steps_since_avg = list(counts)
    assert c.should_average()


def test_should_average_blocked_by_exit_end_and_pending_ack():
    c, t = coord(ApplyPolicy.Sync)
    feed(c, t, 0, 1)
    feed(c, t, 1, 1)
    t.box("tim1").send(TimingExiting(1))
    c.drain_timing()
    assert c.active_count == 1 and not c.should_average()
    c, t = coord(ApplyPolicy.Sync, num_epochs=1)
    feed(c, t, 0, 1)
    feed(c, t, 1, 1)
    c.last_aggregated_epoch = 0
    assert c.all_epochs_done() and not c.should_average()
    c, t = coord(ApplyPolicy.Sync)
    feed(c, t, 0, 1)
    feed(c, t, 1, 1)
    c.trigger_averaging()
    assert [m.kind for m in controls(t, 0)] == ["SyncNow", "SetGlobalStep"]
    assert c.version == 1 and c.global_step == 2 and c.steps_since_avg == [0, 0]
    feed(c, t, 0, 1, start=1)                     # step_count not beyond the sync step: no acknowledgement yet
    feed(c, t, 1, 1, start=1)
    assert not c.should_average()
    t.box("tim0").send(TimingSyncAck(0, 5))
    t.box("tim1").send(TimingSyncAck(1, 5))
    c.drain_timing()
    assert c.should_average()


def test_cpu_averaging_state_machine():
    c, t = coord(ApplyPolicy.Cadence, AverageBackend.Cpu, snapshot_timeout_secs=0.2)
    feed(c, t, 0, 10)
    feed(c, t, 1, 10)
    c.tick()
    assert c.is_cpu_averaging() and [m.kind for m in controls(t, 0)] == ["RequestParams"]
    assert not c.should_average()                 # no re-trigger while a round is in flight
    t.box("par0").send(ParamSnapshot(0, [torch.zeros(2)], [], 10))
    c.tick()
    assert c.is_cpu_averaging()
    time.sleep(0.25)                              # rank 1 never answers: the round is abandoned
    c.tick()
    assert c.abort_count == 1 and c.version == 0
    controls(t, 0), controls(t, 1)
    c.tick()                                      # retried at once: counters still say "due"
    assert c.is_cpu_averaging()
    t.box("par0").send(ParamSnapshot(0, [torch.zeros(2)], [], 10))
    t.box("par1").send(ParamSnapshot(1, [torch.full((2,), 2.0)], [], 10))
    deadline = time.time() + 5
    while c.version == 0 and time.time() < deadline:
        c.tick()
        time.sleep(0.01)
    assert c.version == 1 and not c.is_cpu_averaging()
    kinds = [m.kind for m in controls(t, 1)]
    assert "Update" in kinds and "SetGlobalStep" in kinds
    assert c.global_step == 20 and c.steps_since_avg == [0, 0]


def test_throttle_only_with_cpu_backend():
    c, t = coord(ApplyPolicy.Async, AverageBackend.Cpu)
    c.el_che.with_max_batch_diff(3)
    feed(c, t, 0, 1)
    feed(c, t, 1, 6)
    c.check_throttle()
    assert [m.kind for m in controls(t, 1)] == ["Throttle"] and controls(t, 0) == []
    c.check_throttle()
    assert controls(t, 1) == []                   # told once
    c2, t2 = coord(ApplyPolicy.Async, AverageBackend.Nccl)
    c2.el_che.with_max_batch_diff(3)
    feed(c2, t2, 0, 1)
    feed(c2, t2, 1, 6)
    c2.check_throttle()
    assert controls(t2, 1) == []


def test_plans_and_epoch_aggregation_without_progressive_dispatch():
    c, t = coord(ApplyPolicy.Cadence, num_epochs=2, total=100)
    c.send_all_plans(0)
    p0, p1 = controls(t, 0)[0].payload, controls(t, 1)[0].payload
    assert (p0.partition_offset, p0.partition_size, p1.partition_offset, p1.partition_size) == (0, 50, 50, 50)
    t.box("met0").send(MetricsMsg(0, 0, 1.0, 5, 10.0, 50))
    assert c.drain_metrics() and c.last_aggregated_epoch is None
    t.box("met1").send(MetricsMsg(1, 0, 3.0, 5, 12.0, 50))
    c.drain_metrics()
    assert c.last_aggregated_epoch == 0
    assert controls(t, 0)[0].payload.epoch == 1   # next epoch's plan went out
    t.box("met0").send(MetricsMsg(0, 1, 1.0, 5, 10.0, 50))
    t.box("met1").send(MetricsMsg(1, 1, 1.0, 5, 10.0, 50))
    c.drain_metrics()
    assert c.all_epochs_done() and controls(t, 0)[-1].kind == "Shutdown"


def test_progressive_dispatch_hands_out_the_whole_epoch_once():
    c, t = coord(ApplyPolicy.Async, AverageBackend.Cpu, total=400, num_epochs=1, progressive=True)
    c.send_all_plans(0)
    seen = []
    for _ in range(200):
        progressed = False
        for r in range(2):
            for m in controls(t, r):
                if m.kind == "StartEpoch":
                    p = m.payload
                    seen.append((p.partition_offset, p.partition_size))
                    t.box(f"met{r}").send(MetricsMsg(r, p.epoch, 1.0, p.partition_size // 10, 1.0, p.partition_size))
                    progressed = True
        c.drain_metrics()
        if c.all_epochs_done():
            break
        if not progressed:
            break
    seen.sort()
    assert seen[0][0] == 0 and sum(s for _, s in seen) == 400
    assert all(a[0] + a[1] == b[0] for a, b in zip(seen, seen[1:]))
    assert c.all_epochs_done()


def test_async_lookahead_of_one_epoch():
    c, t = coord(ApplyPolicy.Async, num_epochs=5)
    c.on_rank_done(0, 0)
    assert controls(t, 0)[0].payload.epoch == 1
    c.on_rank_done(0, 1)                          # epoch 0 not aggregated yet: wait
    assert controls(t, 0) == [] and c.rank_waiting[0]
    c2, t2 = coord(ApplyPolicy.Sync)
    c2.on_rank_done(0, 0)
    assert controls(t2, 0) == []


def test_checkpoint_message_goes_to_rank_zero():
    c, t = coord(ApplyPolicy.Cadence, checkpoint_every=2, num_epochs=4)
    c.on_epoch_aggregated(0)
    assert "Checkpoint" not in [m.kind for m in controls(t, 0)]
    c.on_epoch_aggregated(1)
    ck = [m for m in controls(t, 0) if m.kind == "Checkpoint"]
    assert ck and ck[0].payload == 2 and "Checkpoint" not in [m.kind for m in controls(t, 1)]


def test_collect_final_state_survives_a_missing_rank():
    c, t = coord(ApplyPolicy.Cadence)
    t.box("fin0").send(ParamSnapshot(0, [torch.ones(2)], [], 1))
    st = c.collect_final_state(timeout_s=0.1)
    assert st is not None and st.params[0].tolist() == [1.0, 1.0]
    c2, _ = coord(ApplyPolicy.Cadence)
    assert c2.collect_final_state(timeout_s=0.05) is None


def test_overshoot_auto_tuning():
    c, t = coord(ApplyPolicy.Async, total=100000, batch_size=10)
    assert c.max_overshoot == 5                    # clamp(10000 / 100, 2, 5)
    c2, _ = coord(ApplyPolicy.Async, total=1000, batch_size=10)
    assert c2.max_overshoot == 2
    c3, _ = coord(ApplyPolicy.Async, max_overshoot=7)
    assert c3.max_overshoot == 7 and not c3.overshoot_auto


# ---- transports -------------------------------------------------------------------------------------
class FakeStore:
    def __init__(self): self.d = {}
    def set(self, k, v): self.d[k] = v
    def get(self, k): return self.d[k]
    def check(self, ks): return all(k in self.d for k in ks)
    def delete_key(self, k): self.d.pop(k, None)


def test_store_transport_is_fifo_and_cleans_up():
    store = FakeStore()
    a, b = StoreTransport(store, "x"), StoreTransport(store, "x")
    for i in range(3):
        a.box("ctl0").send(ControlMsg.SetGlobalStep(i))
    assert [b.box("ctl0").try_recv().payload for _ in range(3)] == [0, 1, 2]
    assert b.box("ctl0").try_recv() is None and store.d == {}
    assert b.box("ctl0").recv(timeout=0.01) is None


def test_store_transport_splits_large_messages():
    """Parameter snapshots are far above the store's 8 MB request limit: they travel in chunks."""
    class LimitedStore(FakeStore):
        def set(self, k, v):
            assert len(v) <= 8 << 20, "request above the store's limit"
            super().set(k, v)
    store = LimitedStore()
    a, b = StoreTransport(store, "y"), StoreTransport(store, "y")
    big = torch.arange(5_000_000, dtype=torch.float32)            # 20 MB
    a.box("fin0").send(ParamSnapshot(0, [big], [], 7))
    a.box("fin0").send(ParamSnapshot(0, [torch.ones(3)], [], 8))
    got = b.box("fin0").try_recv()
    assert got.batch_count == 7 and torch.equal(got.params[0], big)
    assert b.box("fin0").try_recv().batch_count == 8
    assert store.d == {}


# ---- workers ----------------------------------------------------------------------------------------
def _model(dev=None):
    torch.manual_seed(3)
    return FlowBuilder.from_(nn.Linear(4, 16)).through(nn.Tanh()).through(nn.Linear(16, 2)).build()


def _data(n=256):
    g = torch.Generator().manual_seed(5)
    x = torch.randn(n, 4, generator=g)
    return x, x @ torch.randn(4, 2, generator=g)


def _train_fn(m, batch):
    loss = nn.mse_loss(m.forward(batch[0]), batch[1])
    record_scalar("mse", float(loss.t.detach()))
    return loss


def _worker(t, rank=0, world=2, **kw):
    x, y = _data(64)
    cfg = WorkerConfig(rank, world, torch.device("cpu"), None, None, 64, 8, **kw)
    return GpuWorker(cfg, _model, lambda ps: nn.SGD(ps, 0.05), TensorDataSet(x, y), t)


def test_worker_runs_a_plan_and_reports():
    t = LocalTransport()
    w = _worker(t)
    assert not w.run_epoch_plan(EpochPlan(0, 0, 32), _train_fn)
    tim = []
    while True:
        m = t.box("tim0").try_recv()
        if m is None:
            break
        tim.append(m)
    assert len(tim) == 4 and [m.step_count for m in tim] == [1, 2, 3, 4] and all(m.batch_ms > 0 for m in tim)
    met = t.box("met0").try_recv()
    assert met.batches_processed == 4 and met.samples_processed == 32 and met.scalars["mse"][1] == 4
    assert w.local_step() == 4 and w.current_epoch() == 0


def test_worker_snapshot_update_and_global_step():
    t = LocalTransport()
    w = _worker(t)
    t.box("ctl0").send(ControlMsg.RequestParams())
    t.box("ctl0").send(ControlMsg.SetGlobalStep(77))
    assert not w.handle_control()
    snap = t.box("par0").try_recv()
    assert snap.rank == 0 and len(snap.params) == 4
    new = AveragedParams([torch.full_like(p, 0.5) for p in snap.params], [], 3)
    t.box("ctl0").send(ControlMsg.Update(new))
    w.steps_since_avg = 5
    w.handle_control()
    assert w.current_version() == 3 and w.steps_since_avg == 0 and w.global_step == 77
    assert all(float(p.t.detach().mean()) == 0.5 for p in w.model().parameters())
    t.box("ctl0").send(ControlMsg.Shutdown())
    assert w.handle_control()


def test_worker_throttle_blocks_until_released():
    t = LocalTransport()
    w = _worker(t)
    t.box("ctl0").send(ControlMsg.Throttle())
    done = []
    th = threading.Thread(target=lambda: done.append(w.handle_control()))
    th.start()
    time.sleep(0.1)
    assert th.is_alive()
    t.box("ctl0").send(ControlMsg.SetGlobalStep(3))     # does not release
    time.sleep(0.1)
    assert th.is_alive() and w.global_step == 3
    t.box("ctl0").send(ControlMsg.Update(AveragedParams([p.t.detach().clone() for p in w.model().parameters()], [], 1)))
    th.join(timeout=5)
    assert done == [False]


def test_drain_until_shutdown_ignores_sync_requests():
    t = LocalTransport()
    w = _worker(t)
    for m in (ControlMsg.SyncNow(), ControlMsg.RequestParams(), ControlMsg.Shutdown()):
        t.box("ctl0").send(m)
    w.drain_until_shutdown(timeout_s=2)
    assert t.box("par0").try_recv() is None and w.local_step() == 0


def test_scheduler_uses_global_step_plus_local_steps():
    t = LocalTransport()
    w = _worker(t)
    w.set_lr_scale(2.0)
    w.set_scheduler(nn.StepDecay(1.0, 10, 0.1))
    w.global_step = 9
    x, y = _data(8)
    w.train_step([x, y], _train_fn)                # lr(9 + 0) * 2
    assert w.current_lr() == pytest.approx(2.0)
    w.train_step([x, y], _train_fn)                # lr(9 + 1) * 2
    assert w.current_lr() == pytest.approx(0.2)


# ---- end to end ---------------------------------------------------------------------------------------
@pytest.mark.parametrize("policy", [ApplyPolicy.Sync, ApplyPolicy.Cadence, ApplyPolicy.Async])
def test_threads_end_to_end(policy):
    x, y = _data(256)
    seen = []
    h = (Trainer.builder(_model, lambda ps: nn.SGD(ps, 0.05), _train_fn).dataset(TensorDataSet(x, y)).batch_size(8)
         .num_epochs(3).policy(policy).backend(AverageBackend.Cpu).devices(["cpu", "cpu"]).metrics_fn(seen.append).run())
    assert h.world_size() == 2
    state = h.join()
    assert [m.epoch for m in seen] == [0, 1, 2] and seen[-1].avg_loss < seen[0].avg_loss
    assert "mse" in seen[-1].scalars and len(state.params) == 4
    assert h.join() is state                       # idempotent


def test_single_device_run():
    x, y = _data(64)
    h = (Trainer.builder(_model, lambda ps: nn.SGD(ps, 0.05), _train_fn).dataset(TensorDataSet(x, y)).batch_size(8)
         .num_epochs(2).devices(["cpu"]).run())
    st = h.join()
    assert len(h.poll_metrics()) == 2 and len(st.params) == 4


def test_workers_inherit_the_launching_threads_autocast_state():
    """Autocast state is per thread; `with AutocastGuard(...): builder.run()` must reach the worker threads."""
    from flodl_b200 import ops
    x, y = _data(32)
    seen = []

    def fn(m, batch):
        seen.append((ops.FLAGS.autocast, torch.is_autocast_enabled("cpu")))
        return _train_fn(m, batch)
    with nn.AutocastGuard(torch.bfloat16, "cpu"):
        h = (Trainer.builder(_model, lambda ps: nn.SGD(ps, 0.05), fn).dataset(TensorDataSet(x, y)).batch_size(8)
             .num_epochs(1).devices(["cpu"]).run())
        h.join()
    assert seen and all(a == torch.bfloat16 and b for a, b in seen)
    seen.clear()
    h = (Trainer.builder(_model, lambda ps: nn.SGD(ps, 0.05), fn).dataset(TensorDataSet(x, y)).batch_size(8)
         .num_epochs(1).devices(["cpu"]).run())
    h.join()
    assert seen and all(a is None and not b for a, b in seen)


def test_thread_worker_error_is_reported():
    x, y = _data(64)

    def bad(m, batch):
        raise RuntimeError("injected")
    h = (Trainer.builder(_model, lambda ps: nn.SGD(ps, 0.05), bad).dataset(TensorDataSet(x, y)).batch_size(8)
         .num_epochs(2).backend(AverageBackend.Cpu).devices(["cpu", "cpu"]).run())
    # the surviving worker's parameters are still returned; the failure is kept for the caller
    try:
        state = h.join()
        assert state is not None
    except RuntimeError as e:
        assert "injected" in repr(e)
    assert any("injected" in repr(e) for e in h.errors())


def test_builder_requires_dataset_batch_size_epochs():
    b = Trainer.builder(_model, lambda ps: nn.SGD(ps, 0.05), _train_fn)
    with pytest.raises(Exception):
        b.run()
    with pytest.raises(Exception):
        b.dataset(TensorDataSet(*_data(8))).run()


@pytest.mark.parametrize("scenario", ["run_fixed", "run_cadence", "run_sync", "run_cpu_backend", "run_worker_failure"])
def test_processes_over_gloo(scenario):
    run_ranks(scenario)


def test_native_average_and_divergence_matches_the_tensor_op_path():
    """One pass in C++ against the reference arithmetic with tensor operations: fp32 fast path across block and thread
    boundaries, a non-contiguous and a bf16 tensor through the generic path, rank order, weights, buffers."""
    from flodl_b200 import _ext
    from flodl_b200.parallel.ddp_run import average_and_divergence
    if not _ext.available():
        pytest.skip("native extension not built")
    g = torch.Generator().manual_seed(3)
    shapes = [(16384 * 3 + 17,), (129, 65), (1,), (7, 5, 3), (40000,)]

    def snap(rank, count):
        ps = [torch.randn(s, generator=g) * (1 + rank) for s in shapes]
        ps[1] = ps[1].t().contiguous().t()                          # same shape, not contiguous
        ps[3] = ps[3].to(torch.bfloat16)
        bufs = [torch.randn(9, generator=g), torch.tensor(rank + 4)]
        return ParamSnapshot(rank, ps, bufs, count)
    snaps = [snap(2, 5), snap(0, 1), snap(1, 10)]                   # arrival order differs from rank order
    ref = average_params(snaps, 4)
    ref_div = divergence_of(snaps, ref)
    avg, div = average_and_divergence(snaps, 4)
    assert avg.version == 4 and len(avg.params) == len(shapes)
    for a, b in zip(avg.params, ref.params):
        assert a.dtype == b.dtype and a.shape == b.shape
        torch.testing.assert_close(a.float(), b.float(), rtol=1e-6, atol=1e-6)
    for a, b in zip(avg.buffers, ref.buffers):
        assert torch.equal(a, b)
    assert div.deltas == pytest.approx(ref_div.deltas, rel=1e-5) and div.pre_norms == pytest.approx(ref_div.pre_norms, rel=1e-6)
    assert div.post_norm == pytest.approx(ref_div.post_norm, rel=1e-6)
    threads = torch.get_num_threads()
    torch.set_num_threads(1)                                        # the sums do not depend on the number of threads
    try:
        _, div1 = average_and_divergence(snaps, 4)
    finally:
        torch.set_num_threads(threads)
    assert div1.deltas == div.deltas and div1.post_norm == div.post_norm
    with pytest.raises(RuntimeError, match="shape"):
        _ext.require().cpu_weighted_average([[torch.zeros(3)], [torch.zeros(4)]], [0.5, 0.5], True)
    with pytest.raises(RuntimeError, match="weights"):
        _ext.require().cpu_weighted_average([[torch.zeros(3)]], [0.5, 0.5], True)
