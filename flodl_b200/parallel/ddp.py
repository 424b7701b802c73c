"""Synchronous data parallelism: `Trainer`, `Ddp`, `DdpConfig`, `DistributedState`.

The reference keeps N replicas in ONE process, scatters each batch across them, and after
backward calls `ncclAllReduce` once per parameter, `ncclBroadcast` once per buffer, then N
optimizers (flodl/src/distributed/ddp.rs:83-369, flodl/src/graph/distributed.rs:239-452).
Here one process drives one GPU (`torchrun`); the same user-facing calls act on this process's
replica:

* `Trainer.setup(model, builder, optimizer)` / `Graph.distribute()` re-home the parameters into
  flat fp32 buffers (gradients in peer-mapped memory), broadcast rank 0's values with one P2P
  kernel and make `forward` take this rank's shard of the batch (`chunk_ratios`, as in
  graph/distributed.rs:767-839);
* `Graph.step()` averages gradients per ~25 MB bucket with the NVLink all-reduce kernels
  (weighted by shard size when shards are unequal, ddp.rs:206-225), broadcasts buffers in one
  packed message, runs the optimizer, zeroes gradients and feeds the auto-balancer
  (EMA alpha 0.3 of samples/ms, first rebalance after 10 steps then every 50, no rank below 5 %;
  ddp.rs:66-76, 232-319);
* with El Che (`DdpConfig`), every rank accumulates `el_che.batches(rank)` batches between two
  synchronisations and gradients are combined with weights `count_r / sum(count)`
  (graph/distributed.rs:254-404).

On CPU (gloo) the same code runs with `torch.distributed` collectives, which is what the
multi-process CPU tests exercise.
"""
from __future__ import annotations

import time
from typing import Callable, List, Optional, Sequence

import torch

from ..ops import core as _core_ops
import torch.distributed as dist

from ..nn.module import Module, Parameter
from ..tensor import TensorError
from . import comm as _comm
from .el_che import ElChe
from .flat import FlatParams, flat_of
from .grad_sync import GradSync

DEFAULT_CALIBRATION_STEPS = 10
DEFAULT_REBALANCE_INTERVAL = 50
EMA_ALPHA = 0.3
MIN_CHUNK_RATIO = 0.05


# ---- configuration -------------------------------------------------------------------------------
class DdpConfig:
    """Options of `Trainer.setup_with` (ddp.rs:1032-1118). `max_anchor`: None = El Che decides,
    0 = El Che off (plain per-batch DDP), n = anchor capped at n."""

    def __init__(self):
        self.speed_hint_: Optional[tuple] = None
        self.overhead_target_: Optional[float] = None
        self.max_anchor_: Optional[int] = None
        self.max_grad_norm_: Optional[float] = None
        self.timeline_ = None

    @classmethod
    def new(cls) -> "DdpConfig":
        return cls()

    def speed_hint(self, slow_rank: int, ratio: float) -> "DdpConfig":
        self.speed_hint_ = (int(slow_rank), float(ratio))
        return self

    def overhead_target(self, target: float) -> "DdpConfig":
        self.overhead_target_ = float(target)
        return self

    def max_anchor(self, max_anchor: Optional[int]) -> "DdpConfig":
        self.max_anchor_ = None if max_anchor is None else int(max_anchor)
        return self

    def max_grad_norm(self, max_norm: float) -> "DdpConfig":
        self.max_grad_norm_ = float(max_norm)
        return self

    def timeline(self, tl) -> "DdpConfig":
        self.timeline_ = tl
        return self


def rebalance_ratios(ema_throughput: Sequence[float]) -> Optional[List[float]]:
    """Chunk ratios proportional to throughput, no rank below `MIN_CHUNK_RATIO`, summing to 1
    (ddp.rs:271-319). None when nothing has been measured yet."""
    total = float(sum(ema_throughput))
    if total <= 0.0:
        return None
    n = len(ema_throughput)
    ratios = [t / total for t in ema_throughput]
    deficit, unclamped = 0.0, 0
    for i, r in enumerate(ratios):
        if r < MIN_CHUNK_RATIO:
            deficit += MIN_CHUNK_RATIO - r
            ratios[i] = MIN_CHUNK_RATIO
        else:
            unclamped += 1
    if deficit > 0.0 and unclamped > 0:
        free = sum(r for r in ratios if r > MIN_CHUNK_RATIO + 1e-9)
        if free > MIN_CHUNK_RATIO * n:
            ratios = [max(MIN_CHUNK_RATIO, r - deficit * (r / free)) if r > MIN_CHUNK_RATIO + 1e-9 else r for r in ratios]
    s = sum(ratios)
    return [r / s for r in ratios] if s > 0 else None


def shard_sizes_from_ratios(ratios: Sequence[float], batch: int) -> List[int]:
    """Integer shard sizes for `batch` samples: floor of the proportional share, the remainder to
    the last rank (ddp.rs:170-188)."""
    n = len(ratios)
    sizes, used = [], 0
    for i, r in enumerate(ratios):
        if i == n - 1:
            sizes.append(batch - used)
        else:
            s = int(batch * r)
            sizes.append(s)
            used += s
    return sizes


def broadcast_packed(tensors: Sequence[torch.Tensor], root: int = 0) -> None:
    """One broadcast for a whole list of (small) floating-point tensors instead of one per tensor
    (the reference issues one `ncclBroadcast` per buffer per step, ddp.rs:150-157)."""
    ts = [t for t in tensors if t.is_floating_point() and t.numel() > 0]
    if not ts or not dist.is_initialized() or dist.get_world_size() <= 1:
        return
    pack = torch.cat([t.detach().reshape(-1).float() for t in ts])
    dist.broadcast(pack, root)
    off = 0
    with torch.no_grad():
        for t in ts:
            t.copy_(pack[off:off + t.numel()].view(t.shape))
            off += t.numel()


# ---- the per-process replica state ---------------------------------------------------------------
class DistributedState:
    """What `Graph.distribute()` attaches to a graph (and what `Ddp` wraps around any module)."""

    def __init__(self, model: Module, *, scatter: bool = True, bucket_mb: float = 25.0, overlap: bool = True,
                 comm_backend: str = "symm", comm_blocks: int = 24, comm_timeout_s: float = 10.0,
                 config: Optional[DdpConfig] = None, sync: bool = True):
        self.model = model
        self.world_size, self.rank = _comm.world_size(), _comm.rank()
        params: List[Parameter] = model.parameters()
        if not params:
            raise TensorError("distribute(): the model has no parameters")
        tensors = [p.t for p in params]
        self.device = tensors[0].device
        self.scatter = bool(scatter)
        self._devices = self._gather_devices()
        self.symm_grads = self.symm_params = None
        self.flat = flat_of(tensors)
        if self.flat is None:
            grad_alloc = param_alloc = None
            if self.world_size > 1 and self.device.type == "cuda" and comm_backend == "symm":
                def grad_alloc(n):
                    self.symm_grads = _comm.SymmetricBuffer(n * 4, self.device.index, comm_timeout_s)
                    return self.symm_grads.view(torch.float32, 0, n)

                def param_alloc(n):
                    self.symm_params = _comm.SymmetricBuffer(n * 4, self.device.index, comm_timeout_s)
                    return self.symm_params.view(torch.float32, 0, n)
            from ..nn.module import walk_modules
            groups = [[p.t for p in g] for m in walk_modules(model) for g in m.fuse_groups()]
            self.flat = FlatParams(tensors, shadow=self.device.type == "cuda", grad_alloc=grad_alloc, param_alloc=param_alloc, groups=groups)
        backend = "symm" if self.symm_grads is not None else "nccl"
        # Overlapping a bucket's all-reduce with backward relies on knowing how many gradient
        # contributions each parameter gets per step. Data-dependent control flow (switch, while /
        # until loops) changes that from step to step and from rank to rank, so such models
        # exchange all gradients after backward instead.
        from ..nn.module import walk_modules as _walk
        if any(getattr(m, "dynamic", False) for m in _walk(model)):
            overlap = False
        _core_ops.set_eager_min_numel(0)      # flat buffers and direct gradient slots: native kernels for every size
        self.sync = GradSync(self.flat, self.symm_grads, int(bucket_mb * 1024 * 1024), overlap, comm_blocks, backend)
        # auto-balancer
        w = self.world_size
        self._ratios: List[float] = [1.0 / w] * w
        self._ema: List[float] = [0.0] * w
        self._local_ema = 0.0
        self.step_count = 0
        self.calibration_steps = DEFAULT_CALIBRATION_STEPS
        self.rebalance_interval = DEFAULT_REBALANCE_INTERVAL
        self._last_shards: List[int] = []
        self._t0 = None          # (start marker, local samples) of the step in flight
        self._pending_timing = None
        # El Che
        self.el_che: Optional[ElChe] = None
        self.max_grad_norm: Optional[float] = None
        self.timeline = None
        self._acc_batches = 0
        self._acc_wall_ms = 0.0
        self._last_sync_ms = 0.0
        if config is not None:
            self.configure_el_che(config)
        if sync and self.world_size > 1:
            self.sync_params()
            self.sync_buffers()

    # ---- construction helpers -----------------------------------------------------------------
    @classmethod
    def for_graph(cls, graph, factory: Optional[Callable] = None, **kw) -> "DistributedState":
        """`factory` is what builds one replica per device in the reference
        (graph/distributed.rs:34-127). With one process per GPU the replica already exists in
        every process, so it is accepted and not called."""
        return cls(graph, **kw)

    def _gather_devices(self) -> List[str]:
        me = str(self.device)
        if self.world_size <= 1:
            return [me]
        out = [None] * self.world_size
        dist.all_gather_object(out, me)
        return out

    def configure_el_che(self, config: DdpConfig) -> None:
        """Enable El Che cadence unless `max_anchor == 0` or the world is a single rank
        (ddp.rs:325-369). The speed hint also seeds the chunk ratios."""
        self.max_grad_norm = config.max_grad_norm_
        self.timeline = config.timeline_
        if self.world_size < 2 or config.max_anchor_ == 0:
            return
        e = ElChe(self.world_size, DEFAULT_CALIBRATION_STEPS)
        if config.overhead_target_ is not None:
            e.with_overhead_target(config.overhead_target_)
        if config.max_anchor_ is not None:
            e.with_max_anchor(config.max_anchor_)
        if config.speed_hint_ is not None:
            slow, ratio = config.speed_hint_
            e.with_speed_ratio(slow, ratio)
            raw = [1.0 if r == slow else ratio for r in range(self.world_size)]
            s = sum(raw)
            self._ratios = [x / s for x in raw]
        self.el_che = e
        # several backward passes per step: a bucket is complete only after the last one
        self.sync.overlap = False

    # ---- queries ------------------------------------------------------------------------------
    def intercepts_forward(self) -> bool:
        return self.world_size > 1 and self.scatter

    def devices(self) -> List[str]:
        return list(self._devices)

    def chunk_ratios(self) -> List[float]:
        return list(self._ratios)

    def throughput(self) -> List[float]:
        return list(self._ema)

    def is_balanced(self) -> bool:
        return all(abs(r - 1.0 / self.world_size) < 1e-9 for r in self._ratios)

    def shard_sizes(self, batch: int) -> List[int]:
        return shard_sizes_from_ratios(self._ratios, int(batch))

    compute_shard_sizes = shard_sizes

    def chunk_batches(self) -> int:
        """How many batches this rank runs before the next `step()` (1 without El Che)."""
        return self.el_che.batches(self.rank) if self.el_che is not None else 1

    # ---- forward ------------------------------------------------------------------------------
    def _mark(self):
        if self.device.type == "cuda":
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            return ev
        return time.perf_counter()

    def forward(self, graph, x):
        """Take this rank's rows of every input (dim 0) and run the graph on them."""
        from ..autograd import Variable
        xs = list(x) if isinstance(x, (list, tuple)) else [x]
        ts = [v.t if isinstance(v, Variable) else v for v in xs]
        batch = int(ts[0].shape[0])
        if batch < self.world_size:
            raise TensorError(f"distributed forward: batch {batch} is smaller than the world size {self.world_size}")
        sizes = self.shard_sizes(batch)
        start = sum(sizes[:self.rank])
        n = sizes[self.rank]
        self._last_shards = sizes
        # unequal shards: every bucket (also those reduced while backward still runs) must be
        # combined with the shard weights, so they are fixed before the step starts
        self.sync.set_weights(None if self.is_balanced() else [s / batch for s in sizes])
        shard = [Variable.wrap(t.narrow(0, start, n)) if t.dim() > 0 and t.shape[0] == batch else Variable.wrap(t) for t in ts]
        self.begin_batch(n)
        return graph.forward_impl(shard)

    def begin_batch(self, local_samples: int) -> None:
        """Mark the start of one forward/backward of `local_samples` samples (called by the
        scatter path; call it yourself when feeding pre-sharded batches)."""
        if self._acc_batches == 0:
            self.sync.begin_step()
            self._t0 = (self._mark(), 0)
        self._t0 = (self._t0[0], self._t0[1] + int(local_samples))
        self._acc_batches += 1

    # ---- gradient / buffer / parameter sync ---------------------------------------------------
    def sync_params(self, root: int = 0) -> None:
        if self.world_size <= 1:
            return
        if self.symm_params is not None:
            self.symm_params.broadcast(0, self.flat.total * 4, root, 96)
            torch.cuda.synchronize()
            self.symm_params.check()
        else:
            dist.broadcast(self.flat.params, root)
        self.flat.refresh_shadow()

    def sync_buffers(self, root: int = 0) -> None:
        if self.world_size > 1:
            broadcast_packed([b.get() for b in self.model.buffers()], root)

    def all_reduce_gradients(self) -> None:
        """Average gradients over all ranks (ddp.rs:133-147)."""
        self.sync.set_weights(None)
        self._finish_sync()

    def weighted_all_reduce_gradients(self, weights_or_counts: Sequence[float]) -> None:
        """Combine gradients as sum_r w_r * g_r with w = counts / sum(counts)
        (ddp.rs:206-225, 502-533)."""
        tot = float(sum(weights_or_counts))
        if tot <= 0:
            raise TensorError("weighted_all_reduce_gradients: weights sum to zero")
        self.sync.set_weights([float(c) / tot for c in weights_or_counts])
        self._finish_sync()
        self.sync.set_weights(None)

    def _finish_sync(self) -> None:
        if self.world_size <= 1:
            return
        if self.sync.active:
            self.sync.finish()
        else:
            self.sync.all_reduce_now()

    def guard_optimizer(self, optimizer) -> None:
        """Make sure gradients whose exchange gave up are never applied (`Graph.step()` calls this
        right before the optimizer). The fused optimizers read the collectives' status word on the
        device and leave the parameters alone when it is set; the exception is then raised by the
        next `check_async()` (start of the next step) without a host sync in between. Optimizers
        without a fused path are guarded by a blocking check here."""
        self.sync.guard(optimizer)

    def recover(self) -> None:
        """Collective: re-arm the symmetric buffers after a reported give-up."""
        for b in (self.symm_grads, self.symm_params):
            if b is not None:
                b.recover()
        self.sync.reset()

    # ---- Graph.step() hooks -------------------------------------------------------------------
    def before_optimizer(self) -> None:
        """Gradient combination + buffer broadcast for the step that is about to be applied."""
        if self.world_size <= 1:
            self._acc_batches = 0
            return
        t_sync = time.perf_counter()
        if self.el_che is not None:
            local = max(1, self._acc_batches)
            if self.max_grad_norm is not None:
                from ..nn.clip import clip_grad_norm
                clip_grad_norm(self.flat.tensors, self.max_grad_norm)
            counts = self._all_gather_floats([float(local)])
            counts = [c[0] for c in counts]
            if local > 1:
                self.flat.grads.div_(float(local))   # mean over this rank's batches
            self.weighted_all_reduce_gradients(counts)
            self._el_counts = [int(c) for c in counts]
        elif self.scatter and self._last_shards and self.sync.weights is not None:
            self._finish_sync()
        else:
            self.all_reduce_gradients()
        self.sync_buffers()
        self._last_sync_ms = (time.perf_counter() - t_sync) * 1e3
        if self._t0 is not None:
            self._pending_timing = (self._t0[0], self._mark(), self._t0[1])
            self._t0 = None
        self._acc_batches = 0

    def after_step(self) -> None:
        self.step_count += 1
        self._read_timing()
        if self.world_size <= 1:
            return
        if self.el_che is not None:
            if getattr(self, "_el_counts", None):
                walls = self._all_gather_floats([self._acc_wall_ms])
                self.el_che.report_timing([w[0] for w in walls], self._el_counts, self._last_sync_ms)
                self._acc_wall_ms = 0.0
            return
        if self.update_balance_due():
            self.rebalance()

    def _read_timing(self) -> None:
        pt = self._pending_timing
        if pt is None:
            return
        a, b, samples = pt
        if self.device.type == "cuda":
            if not b.query():
                return                       # not finished yet: read it after the next step
            ms = a.elapsed_time(b)
        else:
            ms = (b - a) * 1e3
        self._pending_timing = None
        self._acc_wall_ms += ms
        if ms > 0 and samples > 0:
            tp = samples / ms
            self._local_ema = tp if self._local_ema == 0.0 else EMA_ALPHA * tp + (1 - EMA_ALPHA) * self._local_ema

    def update_balance_due(self) -> bool:
        if self.step_count == self.calibration_steps:
            return True
        if self.step_count > self.calibration_steps:
            return (self.step_count - self.calibration_steps) % self.rebalance_interval == 0
        return False

    def update_balance(self) -> bool:
        """Count the step, read the last forward's timing into the throughput estimate and, when a
        rebalance is due, recompute the chunk ratios; true when they changed (ddp.rs:227-270).
        `Graph.step()` does the same through `after_step()`."""
        self.step_count += 1
        self._read_timing()
        if self.world_size <= 1 or self.el_che is not None or not self.update_balance_due():
            return False
        return self.rebalance()

    def rebalance(self) -> bool:
        """Exchange the per-rank throughput estimates and recompute the chunk ratios."""
        got = self._all_gather_floats([self._local_ema])
        self._ema = [g[0] for g in got]
        r = rebalance_ratios(self._ema) if all(e > 0 for e in self._ema) else None
        if r is None:
            return False
        self._ratios = r
        return True

    def _all_gather_floats(self, vals: Sequence[float]) -> List[List[float]]:
        if self.world_size <= 1:
            return [list(vals)]
        t = torch.tensor(list(vals), dtype=torch.float64, device=self.device if dist.get_backend() == "nccl" else "cpu")
        out = [torch.empty_like(t) for _ in range(self.world_size)]
        dist.all_gather(out, t)
        return [o.tolist() for o in out]


# ---- manual DDP ------------------------------------------------------------------------------------
class Ddp:
    """Manual DDP for custom loops (ddp.rs:382-542): wrap this process's replica, then call
    `all_reduce_gradients()` between backward and the optimizer step yourself."""

    def __init__(self, state: DistributedState):
        self.state = state

    @classmethod
    def wrap(cls, models, devices: Optional[Sequence] = None, **kw) -> "Ddp":
        """`models`: this process's replica (a `Module`), or a list whose entry `rank` is it - the
        reference passes one replica per device, here the other entries live in other processes."""
        if isinstance(models, (list, tuple)):
            if not models:
                raise TensorError("Ddp.wrap: no models")
            model = models[min(_comm.rank(), len(models) - 1)]
        else:
            model = models
        return cls(DistributedState(model, scatter=False, **kw))

    def sync_params(self) -> None: self.state.sync_params()
    def all_reduce_gradients(self) -> None: self.state.all_reduce_gradients()
    def sync_buffers(self) -> None: self.state.sync_buffers()
    def weighted_all_reduce_gradients(self, batch_counts: Sequence[float]) -> None: self.state.weighted_all_reduce_gradients(batch_counts)
    def world_size(self) -> int: return self.state.world_size
    def devices(self) -> List[str]: return self.state.devices()

    @staticmethod
    def is_heterogeneous() -> bool:
        """True when the ranks do not all sit on the same GPU model."""
        if _comm.world_size() <= 1 or not torch.cuda.is_available():
            return False
        names = [None] * _comm.world_size()
        dist.all_gather_object(names, torch.cuda.get_device_name(torch.cuda.current_device()))
        return len(set(names)) > 1

    @staticmethod
    def print_device_summary() -> None:
        from .. import log
        if _comm.rank() == 0:
            dev = torch.cuda.get_device_name(0) if torch.cuda.is_available() else "cpu"
            log.verbose(f"  ddp: {_comm.world_size()} rank(s), device {dev}")

    # deprecated aliases of the Trainer entry points (ddp.rs:551-639)
    @staticmethod
    def setup(model, builder, optimizer): return Trainer.setup(model, builder, optimizer)
    @staticmethod
    def setup_with(model, builder, optimizer, config): return Trainer.setup_with(model, builder, optimizer, config)
    @staticmethod
    def auto(model, builder, optimizer): return Trainer.setup(model, builder, optimizer)
    @staticmethod
    def auto_with(model, builder, optimizer, config): return Trainer.setup_with(model, builder, optimizer, config)
    @staticmethod
    def builder(model_factory, optim_factory, train_fn): return Trainer.builder(model_factory, optim_factory, train_fn)


def _native_ready() -> bool:
    from .. import ops as _ops
    try:
        return bool(_ops.native_enabled())
    except Exception:
        return False


def _graph_of(head):
    g = getattr(head, "graph", None)
    return g() if callable(g) else head        # a bare Graph stands for itself


class HasGraph:
    """Anything that wraps a training graph and hands it out with `.graph()`: what `Trainer.setup_head`
    accepts (the task heads of `flodl_b200.hf`; ddp.rs:974-981). A `Graph` is its own graph."""

    def graph(self):
        raise NotImplementedError


class Trainer:
    """One-call training setup (ddp.rs:742-952). Works for one rank or many: with a single
    process nothing is distributed and `model.step()` is a plain optimizer step."""

    @staticmethod
    def setup(model, builder: Optional[Callable], optimizer: Callable) -> None:
        Trainer.setup_with(model, builder, optimizer, None)

    @staticmethod
    def setup_with(model, builder: Optional[Callable], optimizer: Callable, config: Optional[DdpConfig], **kw) -> None:
        Ddp.print_device_summary()
        # One rank on a GPU still takes the distributed state: it moves parameters and gradients into the flat
        # buffers, so every op runs this library's kernels (gradients straight into their slots, one fused
        # optimizer launch); its collectives are no-ops in a world of one.
        on_gpu = any(p.t.is_cuda for p in model.parameters()[:1]) and _native_ready()
        if _comm.world_size() > 1 or on_gpu:
            model.distribute(builder, **kw)
            st: DistributedState = model._ddp
            if config is not None:
                st.configure_el_che(config)
            elif Ddp.is_heterogeneous():
                st.configure_el_che(DdpConfig())
        model.set_optimizer(optimizer)
        model.set_training(True)

    @staticmethod
    def setup_head(head, builder: Optional[Callable], optimizer: Callable) -> None:
        """`head`: an object with `.graph()` (the task heads of `flodl_b200.hf`), ddp.rs:900-923."""
        Trainer.setup_with(_graph_of(head), builder, optimizer, None)

    @staticmethod
    def setup_head_with(head, builder: Optional[Callable], optimizer: Callable, config: DdpConfig) -> None:
        Trainer.setup_with(_graph_of(head), builder, optimizer, config)

    @staticmethod
    def builder(model_factory: Callable, optim_factory: Callable, train_fn: Callable):
        """Asynchronous (Local-SGD) training: returns a `DdpBuilder` (ddp.rs:858-898)."""
        from .ddp_run import DdpBuilder
        return DdpBuilder(model_factory, optim_factory, train_fn)
