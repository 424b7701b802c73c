"""The public names of the reference are importable from this package, with the reference's call shapes
(flodl/src/lib.rs:54-108 root re-exports; ddp.rs, orchestrator.rs, worker.rs method lists)."""
import os

import pytest
import torch
import torch.nn.functional as F

import flodl_b200
from flodl_b200 import nn
from flodl_b200.autograd import Variable
from flodl_b200.graph import FlowBuilder, Graph

ROOT_NAMES = """
Verbosity set_verbosity verbosity cuda_available cuda_device_count cuda_memory_info cuda_memory_info_idx cuda_allocated_bytes
cuda_allocated_bytes_idx cuda_active_bytes cuda_active_bytes_idx cuda_peak_active_bytes cuda_peak_active_bytes_idx
cuda_peak_reserved_bytes cuda_peak_reserved_bytes_idx cuda_reset_peak_stats cuda_reset_peak_stats_idx cuda_empty_cache
cuda_utilization cuda_utilization_idx cuda_device_name cuda_device_name_idx cuda_devices cuda_compute_capability probe_device
usable_cuda_devices DeviceInfo set_current_cuda_device current_cuda_device cuda_synchronize hardware_summary set_cudnn_benchmark
manual_seed cuda_manual_seed_all malloc_trim live_tensor_count rss_kb Device DType Result Tensor TensorError TensorOptions Rng
Variable no_grad is_grad_enabled NoGradGuard max_pool2d adaptive_avg_pool2d grid_sample scaled_dot_product_attention embedding
embedding_bag Module NamedInputModule LoopBody TraceEmit forward_via_step Parameter Buffer Linear Optimizer Stateful SGD SGDBuilder
Adam AdamBuilder AdamW AdamWBuilder RMSprop RMSpropBuilder Adagrad AdagradBuilder RAdam NAdam save_checkpoint load_checkpoint
save_checkpoint_file load_checkpoint_file migrate_checkpoint migrate_checkpoint_file checkpoint_version checkpoint_keys LoadReport
MigrateReport GradScaler cast_parameters AutocastGuard autocast is_autocast_enabled Identity ReLU Sigmoid Tanh GELU GeluApprox SiLU
LeakyReLU ELU Softplus Mish SELU Hardswish Hardsigmoid PReLU Softmax LogSoftmax Flatten Dropout Dropout2d AlphaDropout ZeroPad2d
ReflectionPad2d LayerNorm RMSNorm Embedding EmbeddingBag GRUCell GRU LSTMCell LSTM Conv1d Conv1dBuilder Conv2d Conv2dBuilder
ConvTranspose1d ConvTranspose2d Conv3d Conv3dBuilder ConvTranspose3d GroupNorm BatchNorm BatchNorm2d InstanceNorm MaxPool2d AvgPool2d
MaxPool1d AvgPool1d AdaptiveMaxPool2d AdaptiveAvgPool2d PixelShuffle PixelUnshuffle Upsample Unfold Fold Bilinear
MultiheadAttention mse_loss cross_entropy_loss clip_grad_norm clip_grad_value walk_modules walk_modules_visited CudaGraph
FlowBuilder Graph GraphEpochIterator ActiveGraphEpochIterator Trend TrendGroup CpuWorker DataLoader DataLoaderBuilder EpochIterator
DistributedEpochIterator Batch DataSet BatchDataSet RandomSampler SequentialSampler Sampler Ddp Trainer HasGraph ElChe NcclComms
NcclRankComm NcclUniqueId NcclAbortHandle ReduceOp CudaEvent CudaEventFlags CudaStream StreamGuard DdpBuilder DdpHandle ApplyPolicy
AverageBackend DdpConfig DdpRunConfig EpochMetrics GpuWorker TrainedState Monitor modules
""".split()


@pytest.mark.parametrize("name", ROOT_NAMES)
def test_root_name_is_exported(name):
    assert hasattr(flodl_b200, name), name


def _has_all(obj, names):
    return [n for n in names.split() if not hasattr(obj, n)]


def test_trainer_ddp_graph_builder_and_handle_method_lists():
    from flodl_b200.parallel.ddp import Ddp, Trainer
    from flodl_b200.parallel.ddp_run import orchestrator, worker, messages
    assert not _has_all(Trainer, "setup setup_with builder setup_head setup_head_with")
    assert not _has_all(Ddp, "wrap sync_params all_reduce_gradients sync_buffers weighted_all_reduce_gradients world_size devices")
    assert not _has_all(Graph, """distribute auto_distribute set_optimizer set_scheduler set_lr_scale training_step step world_size
        is_distributed has_el_che chunk_ratios throughput shard_sizes devices set_lr set_data_loader set_loss_fn has_loss_fn epoch
        data_num_batches data_batch_size forward_batch forward_multi reset_state detach_state end_step end_sequence end_epoch
        set_device named_parameters named_buffers structural_hash save_checkpoint load_checkpoint snapshot_cpu subgraph parameters_at
        named_parameters_at named_buffers_at freeze thaw is_frozen load_subgraph_checkpoint set_training_at tagged_at collect_at
        record_at trend_at validate_path tagged collect collect_with record record_scalar flush flush_local trend trends traces
        traces_named traces_by_node eta dot svg plot_html export_trends write_log tree_summary profile flush_count""")
    assert not _has_all(FlowBuilder, """new from_ label internal verbose through fork also also_with tag tag_group input using split
        merge loop_body switch gate map build""")
    b = Trainer.builder(lambda d: None, lambda p: None, lambda m, batch: None)
    assert not _has_all(b, """dataset batch_size num_epochs policy backend overhead_target max_anchor anchor divergence_threshold
        no_divergence_guard max_batch_diff max_overshoot checkpoint_every progressive_dispatch max_grad_norm timeline lr_scale_ratio
        checkpoint_fn scheduler epoch_fn metrics_fn run""")
    assert not _has_all(orchestrator.DdpHandle, "world_size devices architecture_svg setup_monitor poll_metrics next_metrics join")
    assert not _has_all(worker.GpuWorker, """rank device local_step current_version current_epoch set_lr current_lr scale_lr set_lr_scale
        set_scheduler model train_step""")
    assert not _has_all(messages, "TimingMsg MetricsMsg ParamSnapshot EpochPlan AveragedParams ControlMsg WorkerConfig")


def _p(*shape):
    return nn.Parameter(Variable(torch.randn(*shape), requires_grad=True), "w")


def test_optimizer_builders_set_their_knobs_and_groups():
    a, b = _p(3), _p(3)
    opt = nn.Adam.with_groups().betas(0.8, 0.9).eps(1e-6).group([a], 0.1).group([b], 0.01).build()
    assert (opt.beta1, opt.beta2, opt.eps) == (0.8, 0.9, 1e-6) and len(opt.params) == 2
    assert isinstance(nn.Adam.with_groups(), nn.AdamBuilder)
    w = nn.AdamW.with_groups(0.05).group([a], 0.1).build()
    assert w.weight_decay == 0.05 and isinstance(w, nn.AdamW)
    s = nn.SGD.with_groups(0.9).weight_decay(1e-4).group([a], 0.1).build()
    assert (s.momentum, s.weight_decay) == (0.9, 1e-4) and isinstance(nn.SGD.with_groups(0.0), nn.SGDBuilder)
    r = nn.RMSprop.builder([a], 0.01).alpha(0.9).eps(1e-7).weight_decay(0.1).momentum(0.5).build()
    assert (r.alpha, r.eps, r.weight_decay, r.momentum, r.lr()) == (0.9, 1e-7, 0.1, 0.5, 0.01)
    g = nn.Adagrad.builder([a], 0.02).eps(1e-9).weight_decay(0.2).lr_decay(0.3).build()
    assert (g.eps, g.weight_decay, g.lr_decay) == (1e-9, 0.2, 0.3)
    for opt in (opt, w, s, r, g):                       # every built optimizer takes a step
        a.variable.t.grad = torch.ones(3)
        b.variable.t.grad = torch.ones(3)
        before = a.variable.t.detach().clone()
        opt.step()
        assert not torch.equal(before, a.variable.t.detach())


def test_conv_builder_alias_and_knobs():
    c = nn.Conv2d.configure(3, 8, 3).with_stride(2).with_padding(1).without_bias().done()
    assert isinstance(nn.Conv2d.configure(3, 8, 3), nn.Conv2dBuilder) and c.bias is None
    assert c.forward(Variable.wrap(torch.randn(2, 3, 8, 8))).t.shape == (2, 8, 4, 4)


def test_loop_body_and_named_input_bases():
    class Step(nn.LoopBody):
        def __init__(self): self.lin = nn.Linear(4, 4)
        def sub_modules(self): return [self.lin]
        def step(self, x, refs, emit):
            h = self.lin.forward(x)
            emit.publish("h", h)
            return h
    body = Step()
    x = Variable.wrap(torch.randn(2, 4))
    assert body.forward(x).t.shape == (2, 4) and body.as_loop_body() is body
    g = FlowBuilder.from_(nn.Linear(4, 4)).loop_body(body).for_n(3).build()
    g.forward(x)
    assert len(g.traces_named("h")) == 3

    class Mix(nn.NamedInputModule):
        def forward_named(self, x, refs):
            return x + refs["skip"] if "skip" in refs else x
    m = Mix()
    assert m.as_named_input() is m and torch.equal(m.forward(x).t, x.t)
    g2 = FlowBuilder.from_(nn.Linear(4, 4)).tag("skip").through(nn.GELU()).through(m).using("skip").build()
    assert g2.forward(x).t.shape == (2, 4)


def test_walk_modules_visited_shares_the_visited_set():
    shared = nn.Linear(2, 2)
    class Box(nn.Module):
        def __init__(self, *kids): self.kids = list(kids)
        def sub_modules(self): return self.kids
        def forward(self, x): return x
    a, b = Box(shared), Box(shared, nn.Linear(2, 2))
    seen, visited = [], set()
    flodl_b200.walk_modules_visited(a, visited, seen.append)
    flodl_b200.walk_modules_visited(b, visited, seen.append)
    assert len(seen) == 4 and seen.count(shared) == 1
    assert len(nn.collect_parameters([a, b])) == 2 + 4


def test_epoch_iterators_know_their_length():
    from flodl_b200.data import DataLoader, TensorDataSet
    ds = TensorDataSet(torch.arange(20.0).reshape(10, 2), torch.arange(10))
    loader = DataLoader.from_batch_dataset(ds).batch_size(3).shuffle(False).build()
    it = loader.epoch(0)
    assert isinstance(it, flodl_b200.EpochIterator) and len(it) == 3 and it.size_hint() == (3, 3)
    next(it)
    assert len(it) == 2
    assert len(list(it)) == 2 and len(it) == 0
    sharded = DataLoader.from_batch_dataset(ds).batch_size(2).shuffle(False).build().distributed(1, 2)
    it = sharded.epoch(0)
    assert isinstance(it, flodl_b200.DistributedEpochIterator) and (it.rank, it.world_size) == (1, 2)
    assert it.shard_bounds == (5, 10)
    first = next(it)
    assert first[1].tolist() == [5, 6]
    it.close()
    assert len(it) == 0


def test_graph_epoch_iterator_activates_lazily_and_counts():
    from flodl_b200.data import DataLoader, TensorDataSet
    g = FlowBuilder.from_(nn.Linear(2, 1)).build()
    ds = TensorDataSet(torch.randn(8, 2), torch.randn(8, 1))
    g.set_data_loader(DataLoader.from_batch_dataset(ds).batch_size(4).names(["x", "y"]).build(), "x")
    handle = g.epoch(0)
    assert isinstance(handle, flodl_b200.GraphEpochIterator) and handle._active is None
    active = handle.activate()
    assert isinstance(active, flodl_b200.ActiveGraphEpochIterator) and len(active) == 2
    assert len(list(handle)) == 2


def test_cuda_event_flags_and_device_queries_on_cpu():
    assert int(flodl_b200.CudaEventFlags.Default) == 0 and int(flodl_b200.CudaEventFlags.DisableTiming) == 1
    assert flodl_b200.cuda_active_bytes() == 0 or torch.cuda.is_available()
    assert flodl_b200.cuda_peak_reserved_bytes_idx(0) >= 0
    assert flodl_b200.current_cuda_device() == 0 or torch.cuda.is_available()


def test_snapshot_cpu_method_and_has_graph(tmp_path):
    g = FlowBuilder.from_(nn.Linear(2, 2)).build()
    snap = g.snapshot_cpu()
    path = os.path.join(tmp_path, "s.fdl")
    snap.save_file(path)
    assert flodl_b200.checkpoint_version(path) == 2 and len(snap.params) == 2
    from flodl_b200.parallel.ddp import _graph_of

    class Head(flodl_b200.HasGraph):
        def graph(self): return g
    assert _graph_of(Head()) is g and _graph_of(g) is g


# ---- constructor spellings and fluent knobs of the reference's layers -------------------------------------
def test_new_and_on_device_spellings_exist_on_every_module_class():
    assert isinstance(nn.ReLU.new(), nn.ReLU) and isinstance(nn.LeakyReLU.new(0.2), nn.LeakyReLU)
    assert nn.Softmax.new(-1).forward(Variable.wrap(torch.randn(2, 3))).t.sum().item() == pytest.approx(2.0, abs=1e-5)
    cell = nn.GRUCell.on_device(3, 5, "cpu")
    assert cell.parameters()[0].t.device.type == "cpu"
    assert isinstance(nn.StepDecay.new(0.1, 10, 0.5), nn.StepDecay) and nn.PlateauScheduler.new(0.1, 2, 0.5, 1e-4).current_lr == 0.1
    assert isinstance(nn.RAdam.new([_p(2)], 1e-3), nn.RAdam)
    g = flodl_b200.NoGradGuard.new()
    assert not torch.is_grad_enabled()
    g.release()
    assert torch.is_grad_enabled()


def test_pooling_knobs():
    x = Variable.wrap(torch.randn(1, 2, 9, 9))
    a = nn.MaxPool2d.new(3).padding(1).ceil_mode(True).forward(x).t
    assert torch.equal(a, F.max_pool2d(x.t, 3, 3, 1, 1, True))
    b = nn.AvgPool2d.with_stride(3, 2).padding(1).count_include_pad(False).forward(x).t
    torch.testing.assert_close(b, F.avg_pool2d(x.t, 3, 2, 1, False, False))
    x1 = Variable.wrap(torch.randn(1, 2, 10))
    assert torch.equal(nn.MaxPool1d.with_stride(3, 1).padding(1).forward(x1).t, F.max_pool1d(x1.t, 3, 1, 1))
    torch.testing.assert_close(nn.AvgPool1d.new(2).forward(x1).t, F.avg_pool1d(x1.t, 2))


def test_upsample_fold_unfold_and_padding_constructors():
    x = Variable.wrap(torch.randn(1, 2, 4, 4))
    up = nn.Upsample.new([8, 8], 1).align_corners(True).forward(x).t
    torch.testing.assert_close(up, F.interpolate(x.t, size=(8, 8), mode="bilinear", align_corners=True))
    assert nn.Upsample.new([8, 8], 0).align_corners(False).forward(x).t.shape == (1, 2, 8, 8)
    cols = nn.Unfold.new(3).padding([1, 1]).stride([1, 1]).forward(x).t
    assert cols.shape == (1, 18, 16)
    back = nn.Fold.with_kernel([4, 4], [3, 3]).padding([1, 1]).forward(Variable.wrap(cols)).t
    assert back.shape == (1, 2, 4, 4)
    assert nn.Unfold.with_kernel([2, 4]).forward(x).t.shape == (1, 16, 3)
    assert nn.ZeroPad2d.asymmetric(1, 2, 3, 4).forward(x).t.shape == (1, 2, 11, 7)
    assert nn.ReflectionPad2d.asymmetric(1, 0, 2, 0).forward(x).t.shape == (1, 2, 6, 5)
    bl = nn.Bilinear(3, 4, 5)
    assert bl.forward_bilinear(Variable.wrap(torch.randn(2, 3)), Variable.wrap(torch.randn(2, 4))).t.shape == (2, 5)


def test_tensor_error_and_device_info_helpers():
    e = flodl_b200.TensorError.new("CUDA out of memory. Tried to allocate 2 GiB")
    assert e.is_cuda_oom() and not flodl_b200.TensorError("shape mismatch").is_cuda_oom()
    assert flodl_b200.NcclAbortHandle().is_aborted() is False


# ---- timeline types ------------------------------------------------------------------------------------
def test_event_kind_variants_and_broadcast_type():
    from flodl_b200.monitor import EventKind, GpuTimelineSample, Timeline, TimelineBroadcast
    tl = Timeline.new(1000)
    tl.event(EventKind.SyncStart())
    tl.event(EventKind.SyncEnd(2.5))
    tl.event(EventKind.AnchorChanged(4, 8))
    tl.event(EventKind.Custom("eval"))
    tl.event("Throttle", rank=1)
    kinds = [e.kind for e in tl.events()]
    assert kinds == ["SyncStart", "SyncEnd", "AnchorChanged", "Custom", "Throttle"]
    assert tl.events()[2].fields == {"from": 4, "to": 8} and tl.events()[1].fields["duration_ms"] == 2.5
    assert EventKind.Throttle(1) == EventKind("Throttle", rank=1) and "Throttle" in repr(EventKind.Throttle(1))
    with pytest.raises(ValueError):
        EventKind("Nope")
    sub = tl.subscribe()
    tl.sample_once()
    tl._broadcast()
    msg = sub.get(timeout=1)
    assert isinstance(msg, TimelineBroadcast) and len(msg.events) == 5 and msg["samples"] == msg.samples
    assert tl.summary().sync_count == 1
    gs = tl.drain()[0][0].gpu_samples()
    assert all(isinstance(g, GpuTimelineSample) for g in gs)


# ---- coordinator / worker construction helpers ----------------------------------------------------------
def test_coordinator_builder_and_blocking_drain():
    from flodl_b200.parallel.ddp_run.channel import LocalTransport
    from flodl_b200.parallel.ddp_run.coordinator import Coordinator, CoordinatorBuilder
    from flodl_b200.parallel.ddp_run.messages import ApplyPolicy, AverageBackend, TimingBatch
    from flodl_b200.parallel.ddp_run.worker import GpuWorker
    tr = LocalTransport()
    el = flodl_b200.ElChe.new(2, 10)
    b = Coordinator.builder(tr, ApplyPolicy.Cadence, AverageBackend.Cpu, 2, 640, el)
    assert isinstance(b, CoordinatorBuilder)
    c = (b.batch_size(32).num_epochs(3).progressive(False).divergence_threshold(0.1).no_divergence_guard().checkpoint_every(5)
         .snapshot_timeout_secs(2).device_indices([0, 1]).partition_ratios([0.75, 0.25]).max_overshoot(3).overshoot_ceiling(9)
         .overhead_target(0.2).max_anchor(50).build())
    assert (c.batch_size, c.num_epochs, c.progressive, c.checkpoint_every, c.snapshot_timeout_secs) == (32, 3, False, 5, 2.0)
    assert c.partition_ratios == [0.75, 0.25] and c.max_overshoot == 3 and c.overshoot_ceiling == 9
    assert not c.convergence_guard.enabled and c.version == 0 and c.avg_count == 0 and c.abort_count == 0
    worker_side, coord_side = GpuWorker.channels(tr, 1)
    worker_side.timing_tx.send(TimingBatch(1, 12.5, 1, None, 0.7, None))
    assert c.drain_timing_blocking(0.5) is True and c.last_batch_ms[1] == 12.5 and c.steps_since_avg[1] == 1
    t0 = __import__("time").monotonic()
    assert c.drain_timing_blocking(0.05) is True and __import__("time").monotonic() - t0 < 1.0      # nothing queued: times out
    c.stop.set()
    assert c.drain_timing_blocking(0.01) is False
    coord_side.control_tx.send("x")
    assert worker_side.control_rx.try_recv() == "x"
    c.debug_state_dump(1)                                      # silent below debug verbosity


def test_prefetch_worker_distributed_mode_serves_requests_in_order():
    from flodl_b200.data import PrefetchWorker, TensorDataSet
    ds = TensorDataSet(torch.arange(20.0).reshape(10, 2), torch.arange(10))
    w = PrefetchWorker.new(ds, "cpu", 2)
    w.start_distributed_epoch()
    for idx in ([0, 1, 2], [7], [9, 8]):
        w.load_batch(idx)
    w.end_distributed_epoch()
    got = []
    while True:
        b = w.next()
        if b is None:
            break
        got.append(b[1].tolist())
    assert got == [[0, 1, 2], [7], [9, 8]]
    w.stop()
    with pytest.raises(RuntimeError):
        w.load_batch([1])
    w.start_epoch(list(range(10)), 5)                          # the ordinary mode still works afterwards
    assert w.next()[1].tolist() == [0, 1, 2, 3, 4]
    w.stop()


def test_monitor_log_accepts_a_graph_and_a_graph_with_extras():
    from flodl_b200.monitor import Metrics, Monitor
    g = FlowBuilder.from_(nn.Linear(2, 1)).tag("out").build()
    g.record_scalar("loss", 0.5)
    g.record_scalar("loss", 0.3)
    g.flush([])
    m = Monitor.new(2)
    line = m.log(0, 1.0, g)
    assert "loss=" in line and m.epochs[0].metrics[0][0] == "loss" and abs(m.epochs[0].metrics[0][1] - 0.4) < 1e-9
    m.log(1, 1.0, (g, [("lr", 0.01)]))
    assert [k for k, _ in m.epochs[1].metrics] == ["loss", "lr"]

    class Mine(Metrics):
        def into_metrics(self): return [("acc", 0.9)]
    m2 = Monitor.new(1)
    m2.log(0, 0.5, Mine())
    assert m2.epochs[0].metrics == [("acc", 0.9)] and m2.epochs[0].gpu_metrics == []


def test_ddp_handle_auto_runs_a_small_job_on_cpu():
    from flodl_b200.data import TensorDataSet
    from flodl_b200.parallel.ddp_run import ApplyPolicy, AverageBackend
    torch.manual_seed(0)
    x = torch.randn(64, 4)
    ds = TensorDataSet(x, x.sum(1, keepdim=True))
    h = flodl_b200.DdpHandle.auto(lambda dev: nn.Linear(4, 1, True, dev), lambda ps: nn.SGD(ps, 0.05),
                                  lambda m, batch: nn.mse_loss(m.forward(Variable.wrap(batch[0])), Variable.wrap(batch[1])),
                                  ds, 16, 2, ApplyPolicy.Sync, AverageBackend.Cpu)
    state = h.join()
    assert h.world_size() == 1 and len(state.params) == 2 and not h.errors()
    assert isinstance(flodl_b200.DdpHandle.builder(lambda d: None, lambda p: None, lambda m, b: None), flodl_b200.DdpBuilder)
