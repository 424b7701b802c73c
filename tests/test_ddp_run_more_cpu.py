"""More scheduling cases of the asynchronous DDP coordinator and worker (the behaviours pinned by
flodl/src/distributed/ddp_run/tests.rs), driven with hand-made messages on CPU."""
import time

import pytest
import torch

from flodl_b200 import nn
from flodl_b200.data import TensorDataSet
from flodl_b200.parallel.ddp import Trainer
from flodl_b200.parallel.ddp_run import ApplyPolicy, AverageBackend, ControlMsg, Coordinator, LocalTransport
from flodl_b200.parallel.ddp_run.convergence import ConvergenceAction
from flodl_b200.parallel.ddp_run.messages import MetricsMsg, ParamSnapshot, TimingBatch, TimingExiting, WorkerConfig
from flodl_b200.parallel.ddp_run.worker import GpuWorker, make_partition
from flodl_b200.parallel.el_che import ElChe


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


# ---- initial state, counters -----------------------------------------------------------------------
def test_initial_state_and_timing_accumulation():
    c, t = coord(ApplyPolicy.Cadence, world=3)
    assert c.version == 0 and c.global_step == 0 and c.active_count == 3 and c.steps_since_avg == [0, 0, 0]
    assert not c.is_cpu_averaging() and not c.all_epochs_done() and c.last_aggregated_epoch is None
    feed(c, t, 0, 3, ms=7.0)
    feed(c, t, 2, 1, ms=11.0)
    assert c.steps_since_avg == [3, 0, 1]
    assert c.wall_ms_accum[0] == pytest.approx(21.0) and c.wall_ms_accum[2] == pytest.approx(11.0)
    assert c.last_batch_ms[0] == pytest.approx(7.0) and c.last_step_count[0] == 3


def test_async_policy_ignores_wall_time():
    c, t = coord(ApplyPolicy.Async)
    c.el_che.report_timing([100.0, 100.0], [10, 10], 1.0)
    counts = c.el_che.batch_counts()
    c.steps_since_avg = [counts[0] - 1, counts[1] - 1]
    c.wall_ms_accum = [1e9, 1e9]                      # any amount of wall time does not trigger averaging
    assert not c.should_average()


def test_cadence_with_unequal_ranks_waits_for_the_slow_one():
    c, t = coord(ApplyPolicy.Cadence)
    c.el_che.report_timing([300.0, 100.0], [10, 10], 1.0)      # rank 0 is three times slower
    target = c.el_che.anchor_wall_ms()
    feed(c, t, 1, 30, ms=target / 10)                 # the fast rank passes the target three times over
    feed(c, t, 0, 1, ms=target / 2)
    assert not c.should_average()
    feed(c, t, 0, 1, ms=target / 2 + 1, start=2)
    assert c.should_average()


# ---- partitions ----------------------------------------------------------------------------------------
def test_partition_sizes_follow_measured_throughput():
    c, t = coord(ApplyPolicy.Cadence, total=1200)
    assert c.compute_partition_sizes() == [600, 600]
    c.el_che.report_timing([200.0, 100.0], [10, 10], 1.0)      # rank 1 twice as fast
    a, b = c.compute_partition_sizes()
    assert a + b == 1200 and b > a and abs(b - 2 * a) <= 20
    c2, _ = coord(ApplyPolicy.Sync, total=1200)
    c2.el_che.report_timing([200.0, 100.0], [10, 10], 1.0)
    assert c2.compute_partition_sizes() == [600, 600]          # Sync keeps equal shares whatever the speeds
    c3, _ = coord(ApplyPolicy.Cadence, total=1000, partition_ratios=[0.7, 0.3])
    assert c3.compute_partition_sizes() == [700, 300]


def test_partitions_of_one_epoch_do_not_overlap_and_change_per_epoch():
    total = 103
    a = make_partition(0, 50, total, 3, 42)
    b = make_partition(50, 53, total, 3, 42)
    assert len(a) == 50 and len(b) == 53 and not set(a) & set(b) and set(a) | set(b) == set(range(total))
    assert make_partition(0, 50, total, 3, 42) == a                      # deterministic
    assert make_partition(0, 50, total, 4, 42) != a                      # reshuffled per epoch
    assert make_partition(0, 50, total, 3, 43) != a                      # and per seed
    smaller = make_partition(0, 20, total, 3, 42) + make_partition(20, 20, total, 3, 42)
    assert len(set(smaller)) == 40


def test_fixed_cadence_gives_every_rank_the_same_number_of_whole_batches():
    c, t = coord(ApplyPolicy.Cadence, total=1035, batch_size=10, fixed_cadence=8)
    assert c.compute_partition_sizes() == [510, 510]
    assert not c.should_average()                     # the workers keep the cadence themselves


# ---- throttle ------------------------------------------------------------------------------------------
def test_throttle_zero_is_lockstep_and_none_disables():
    c, t = coord(ApplyPolicy.Async, AverageBackend.Cpu)
    c.el_che.with_max_batch_diff(0)
    feed(c, t, 0, 1)
    feed(c, t, 1, 2)
    c.check_throttle()
    assert [m.kind for m in controls(t, 1)] == ["Throttle"]
    c2, t2 = coord(ApplyPolicy.Async, AverageBackend.Cpu)
    feed(c2, t2, 0, 1)
    feed(c2, t2, 1, 50)
    c2.check_throttle()
    assert controls(t2, 1) == []                      # no max_batch_diff configured


def test_throttle_within_limit_sends_nothing_and_release_rearms():
    c, t = coord(ApplyPolicy.Async, AverageBackend.Cpu)
    c.el_che.with_max_batch_diff(5)
    feed(c, t, 0, 1)
    feed(c, t, 1, 6)
    c.check_throttle()
    assert controls(t, 1) == []
    feed(c, t, 1, 1, start=7)
    c.check_throttle()
    assert [m.kind for m in controls(t, 1)] == ["Throttle"] and c.throttled[1]
    # an averaging round releases the rank and clears the mark
    c.finish_averaging_cpu(1.0, list(c.steps_since_avg), list(c.wall_ms_accum), None)
    assert not any(c.throttled)


# ---- metrics, checkpoints --------------------------------------------------------------------------------
def test_metrics_fn_fires_once_per_epoch_and_its_errors_do_not_stop_training():
    calls = []

    def fn(m):
        calls.append(m.epoch)
        raise RuntimeError("user callback failed")
    c, t = coord(ApplyPolicy.Cadence, num_epochs=2, total=100, metrics_fn=fn)
    c.send_all_plans(0)
    for epoch in (0, 1):
        for r in (0, 1):
            t.box(f"met{r}").send(MetricsMsg(r, epoch, 1.0, 5, 10.0, 50))
        c.drain_metrics()
    assert calls == [0, 1] and c.all_epochs_done()


def test_checkpoint_goes_to_rank_zero_every_n_epochs():
    c, t = coord(ApplyPolicy.Cadence, num_epochs=4, total=100, checkpoint_every=2)
    c.send_all_plans(0)
    for epoch in range(4):
        for r in (0, 1):
            t.box(f"met{r}").send(MetricsMsg(r, epoch, 1.0, 5, 10.0, 50))
        c.drain_metrics()
    k0 = [(m.kind, m.payload) for m in controls(t, 0) if m.kind == "Checkpoint"]
    assert k0 == [("Checkpoint", 2), ("Checkpoint", 4)]
    assert not [m for m in controls(t, 1) if m.kind == "Checkpoint"]


def test_epoch_aggregates_only_when_every_active_rank_reported():
    c, t = coord(ApplyPolicy.Async, world=3, num_epochs=3, total=300)
    c.send_all_plans(0)
    t.box("met0").send(MetricsMsg(0, 0, 1.0, 5, 10.0, 100))
    t.box("met1").send(MetricsMsg(1, 1, 1.0, 5, 10.0, 100))   # a rank that is already an epoch ahead
    c.drain_metrics()
    assert c.last_aggregated_epoch is None
    t.box("met1").send(MetricsMsg(1, 0, 1.0, 5, 10.0, 100))
    t.box("met2").send(MetricsMsg(2, 0, 3.0, 5, 10.0, 100))
    c.drain_metrics()
    assert c.last_aggregated_epoch == 0
    # a rank that left no longer counts towards "everyone"
    t.box("tim2").send(TimingExiting(2))
    c.drain_timing()
    t.box("met0").send(MetricsMsg(0, 1, 1.0, 5, 10.0, 100))
    c.drain_metrics()
    assert c.last_aggregated_epoch == 1


# ---- divergence guard and overshoot ----------------------------------------------------------------------
def test_divergence_nudges_the_anchor_down_and_stable_leaves_it():
    c, t = coord(ApplyPolicy.Async, anchor=20)
    before = c.el_che.anchor()
    c._apply_action(ConvergenceAction("Stable"))
    assert c.el_che.anchor() == before
    c._apply_action(ConvergenceAction("NudgeDown", 0.5))
    assert c.el_che.anchor() < before


def test_overshoot_auto_tuning_grows_when_stable_and_resets_on_divergence():
    c, t = coord(ApplyPolicy.Async, total=100000, batch_size=10)
    if not c.overshoot_auto:
        pytest.skip("overshoot fixed by configuration")
    start = c.max_overshoot
    for _ in range(20):
        c._apply_action(ConvergenceAction("Stable"))
    assert start < c.max_overshoot <= 10
    c._apply_action(ConvergenceAction("NudgeDown", 0.5))
    assert c.max_overshoot == c.overshoot_initial
    fixed, _ = coord(ApplyPolicy.Async, total=100000, batch_size=10, max_overshoot=2)
    for _ in range(5):
        fixed._apply_action(ConvergenceAction("Stable"))
    assert fixed.max_overshoot == 2 and not fixed.overshoot_auto


# ---- CPU averaging -------------------------------------------------------------------------------------------
def test_stale_snapshot_from_an_abandoned_round_is_not_mixed_into_the_next():
    c, t = coord(ApplyPolicy.Cadence, AverageBackend.Cpu, snapshot_timeout_secs=0.1)
    feed(c, t, 0, 10)
    feed(c, t, 1, 10)
    c.tick()
    t.box("par0").send(ParamSnapshot(0, [torch.full((2,), 100.0)], [], 10))
    c.tick()
    time.sleep(0.15)
    c.tick()                                          # rank 1 never answered: abandoned
    assert c.abort_count == 1
    controls(t, 0), controls(t, 1)
    c.tick()                                          # new round
    t.box("par0").send(ParamSnapshot(0, [torch.zeros(2)], [], 10))
    t.box("par1").send(ParamSnapshot(1, [torch.full((2,), 2.0)], [], 10))
    deadline = time.time() + 5
    while c.version == 0 and time.time() < deadline:
        c.tick()
        time.sleep(0.01)
    upd = [m for m in controls(t, 0) if m.kind == "Update"]
    assert upd and torch.allclose(upd[-1].payload.params[0], torch.ones(2))   # (0 + 2) / 2; the 100s are gone


def test_exiting_rank_blocks_further_averaging_and_final_state_uses_survivors():
    c, t = coord(ApplyPolicy.Cadence, AverageBackend.Cpu)
    feed(c, t, 0, 10)
    feed(c, t, 1, 10)
    t.box("tim1").send(TimingExiting(1, "boom"))
    c.drain_timing()
    assert not c.should_average() and c.active_count == 1
    t.box("fin0").send(ParamSnapshot(0, [torch.full((2,), 4.0)], [], 3))
    st = c.collect_final_state(timeout_s=0.3)
    assert st is not None and torch.allclose(st.params[0], torch.full((2,), 4.0))


# ---- worker ------------------------------------------------------------------------------------------------
def _model(dev):
    torch.manual_seed(0)
    return nn.Linear(4, 1)


def _train_fn(m, batch):
    from flodl_b200.autograd import Variable
    return nn.mse_loss(m.forward(Variable.wrap(batch[0])), Variable.wrap(batch[1]))


def _worker(total=64, batch=8, **kw):
    t = LocalTransport()
    x = torch.randn(total, 4)
    y = x.sum(1, keepdim=True)
    cfg = WorkerConfig(0, 1, torch.device("cpu"), None, None, total, batch, 42, None, None, ApplyPolicy.Cadence, None, False)
    w = GpuWorker(cfg, _model, lambda ps: nn.SGD(ps, 0.05), TensorDataSet(x, y), t, kw.get("checkpoint_fn"), False)
    return w, t


def test_worker_load_averaged_rejects_a_wrong_parameter_count():
    from flodl_b200.parallel.ddp_run.messages import AveragedParams
    w, t = _worker()
    good = [p.t.detach().clone() for p in w.model().parameters()]
    w.load_averaged(AveragedParams(good, [], 3))
    assert w.current_version() == 3
    with pytest.raises(Exception):
        w.load_averaged(AveragedParams(good[:1] + [torch.zeros(7, 7)], [], 4))


def test_worker_stops_mid_epoch_on_shutdown_and_reports_what_it_did():
    from flodl_b200.parallel.ddp_run.messages import EpochPlan
    w, t = _worker(total=80, batch=8)
    seen = {"n": 0}

    def fn(m, batch):
        seen["n"] += 1
        if seen["n"] == 3:
            t.box("ctl0").send(ControlMsg.Shutdown())
        return _train_fn(m, batch)
    assert w.run_epoch_plan(EpochPlan(0, 0, 80), fn) is True
    assert seen["n"] == 3 and w.local_step() == 3


def test_worker_epoch_plan_sets_epoch_partition_and_metrics():
    from flodl_b200.parallel.ddp_run.messages import EpochPlan
    w, t = _worker(total=64, batch=8)
    assert w.run_epoch_plan(EpochPlan(2, 16, 32), _train_fn) is False
    assert w.current_epoch() == 2 and len(w.partition) == 32
    m = t.box("met0").try_recv()
    assert m.epoch == 2 and m.batches_processed == 4 and m.samples_processed == 32 and m.avg_loss > 0
    tim = []
    while True:
        x = t.box("tim0").try_recv()
        if x is None:
            break
        tim.append(x)
    assert [b.step_count for b in tim] == [1, 2, 3, 4]


def test_checkpoint_fn_errors_are_logged_not_raised():
    def bad(version, model):
        raise IOError("disk full")
    w, t = _worker(checkpoint_fn=bad)
    assert w.dispatch_control(ControlMsg.Checkpoint(5)) is False       # training goes on
    seen = []
    w2, _ = _worker(checkpoint_fn=lambda v, m: seen.append(v))
    w2.dispatch_control(ControlMsg.Checkpoint(7))
    assert seen == [7]


def test_epoch_fn_runs_once_per_epoch_and_can_set_the_learning_rate():
    x = torch.randn(64, 4)
    y = x.sum(1, keepdim=True)
    epochs = []

    def epoch_fn(epoch, worker):
        epochs.append(epoch)
        worker.set_lr(0.1 / (epoch + 1))
    h = (Trainer.builder(_model, lambda ps: nn.SGD(ps, 0.1), _train_fn).dataset(TensorDataSet(x, y)).batch_size(8)
         .num_epochs(3).devices(["cpu"]).epoch_fn(epoch_fn).run())
    h.join()
    assert epochs == [0, 1, 2]


def test_lr_is_the_same_whether_a_scheduler_runs_solo_or_inside_a_worker():
    """Cross-mode parity: scheduler(global step) * lr_scale drives the optimizer in the worker exactly as
    a plain loop would."""
    sched = nn.StepDecay(0.5, 3, 0.1)
    solo = [sched.lr(s) * 2.0 for s in range(6)]
    w, t = _worker()
    w.set_lr_scale(2.0)
    w.set_scheduler(nn.StepDecay(0.5, 3, 0.1))
    got = []
    x = torch.randn(8, 4)
    y = x.sum(1, keepdim=True)
    for _ in range(6):
        w.train_step([x, y], _train_fn)
        got.append(w.current_lr())
    assert got == pytest.approx(solo)


def test_worker_survives_an_averaging_collective_that_fails_because_a_peer_left():
    """The coordinator's `SyncNow` and a peer's exit can cross: the collective then ends with an error on the survivor. It
    keeps its own weights, acknowledges so that nobody waits, skips later averaging and goes on training."""
    from flodl_b200.parallel.ddp_run.messages import EpochPlan, TimingSyncAck
    w, t = _worker(total=64, batch=8)
    calls = {"n": 0}

    def broken(*a, **k):
        calls["n"] += 1
        raise RuntimeError("Connection closed by peer")
    w.engine.average_params = broken
    before = [p.t.detach().clone() for p in w.model().parameters()]
    assert w.dispatch_control(ControlMsg.SyncNow()) is False
    assert calls["n"] == 1 and w._averaging_broken
    assert all(torch.equal(a, p.t) for a, p in zip(before, w.model().parameters()))
    acks = []
    while True:
        m = t.box("tim0").try_recv()
        if m is None:
            break
        acks.append(m)
    assert any(isinstance(m, TimingSyncAck) for m in acks)
    assert w.dispatch_control(ControlMsg.SyncNow()) is False and calls["n"] == 1          # no second attempt
    assert w.run_epoch_plan(EpochPlan(0, 0, 64), _train_fn) is False and w.local_step() == 8


def test_engine_average_restores_the_weights_when_the_collective_fails(monkeypatch):
    from flodl_b200.parallel.engine import TrainEngine
    m = nn.Linear(4, 2)
    eng = TrainEngine(m, lambda ps: nn.SGD(ps, 0.1), grad_sync=False)
    eng.world, eng.rank = 2, 0                                  # pretend a second rank exists; the collective below fails
    eng.symm_stage = eng.symm_params = None
    before = eng.flat.params.clone()

    def boom(tensor, op=None):
        tensor.mul_(3.0)                                        # a half-done reduction
        raise RuntimeError("peer gone")
    monkeypatch.setattr(torch.distributed, "all_reduce", boom)
    with pytest.raises(RuntimeError, match="peer gone"):
        eng.average_params()
    assert torch.equal(eng.flat.params, before)
    with pytest.raises(RuntimeError):
        eng.average_params([0.5, 0.5])
    assert torch.equal(eng.flat.params, before)
