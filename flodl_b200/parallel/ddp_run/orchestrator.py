"""`DdpBuilder` / `DdpHandle`: launch asynchronous (Local-SGD) data-parallel training
(flodl/src/distributed/ddp_run/orchestrator.rs).

    state = (Trainer.builder(model_factory, optim_factory, train_fn)
             .dataset(ds).batch_size(32).num_epochs(5)
             .policy(ApplyPolicy.Cadence).backend(AverageBackend.Nccl)
             .run().join())

Three topologies, chosen at `run()`:

* one process per GPU (`torchrun`, process group initialised, world > 1): this process runs ONE
  worker thread; rank 0 also runs the coordinator thread; the control plane is a TCP store,
  parameter averaging is the fused peer-memory kernel (`AverageBackend.Nccl`) or host averaging
  through the coordinator (`AverageBackend.Cpu`);
* worker threads inside one process (`.devices([...])`): the reference's own layout
  (thread per device + coordinator thread); averaging goes through the host;
* a single device: a plain training loop, no coordination.
"""
from __future__ import annotations

import json
import queue
import threading
from typing import Callable, List, Optional, Sequence

import torch

from ... import log
from ...tensor import TensorError
from .. import comm as _comm
from ..el_che import ElChe
from .channel import LocalTransport, make_store_transport
from .coordinator import Coordinator
from .messages import (ApplyPolicy, AverageBackend, DdpRunConfig, EpochMetrics, TrainedState, WorkerConfig)
from .worker import GpuWorker

SEED = 42
DEFAULT_ANCHOR = 10
_RUN_COUNTER = [0]


class DdpHandle:
    """Running job: `join()` waits for it and returns the averaged `TrainedState`."""

    def __init__(self, workers: List[threading.Thread], coordinator: Optional[threading.Thread], devices: List, stop: threading.Event,
                 metrics: "queue.Queue", results: dict, is_root: bool, architecture_svg: Optional[str] = None,
                 graph_label: Optional[str] = None, graph_hash: Optional[str] = None, training_meta: Optional[dict] = None,
                 gpu_workers: Optional[List[GpuWorker]] = None, broadcast_final: bool = False):
        self._workers, self._coordinator = workers, coordinator
        self._devices, self._stop, self._metrics, self._results = devices, stop, metrics, results
        self._is_root = is_root
        self._svg, self._label, self._hash, self._meta = architecture_svg, graph_label, graph_hash, training_meta
        self._gpu_workers = gpu_workers if gpu_workers is not None else []
        self._broadcast_final = broadcast_final
        self._final: Optional[TrainedState] = None

    # ---- constructors kept from the reference (orchestrator.rs:90-215); `Trainer.builder` is the entry point
    @staticmethod
    def builder(model_factory: Callable, optim_factory: Callable, train_fn: Callable) -> "DdpBuilder":
        return DdpBuilder(model_factory, optim_factory, train_fn)

    @staticmethod
    def auto(model_factory, optim_factory, train_fn, dataset, batch_size: int, num_epochs: int,
             policy: ApplyPolicy = ApplyPolicy.Cadence, backend: AverageBackend = AverageBackend.Nccl) -> "DdpHandle":
        """Start a run with the default configuration (deprecated in the reference in favour of the builder)."""
        return DdpHandle.auto_with(model_factory, optim_factory, train_fn, dataset, batch_size, num_epochs, policy, backend, DdpRunConfig())

    @staticmethod
    def auto_with(model_factory, optim_factory, train_fn, dataset, batch_size: int, num_epochs: int,
                  policy: ApplyPolicy, backend: AverageBackend, config: DdpRunConfig) -> "DdpHandle":
        return (DdpBuilder(model_factory, optim_factory, train_fn).dataset(dataset).batch_size(batch_size).num_epochs(num_epochs)
                .policy(policy).backend(backend).config(config).run())

    def world_size(self) -> int: return len(self._devices)
    def devices(self) -> List: return list(self._devices)
    def architecture_svg(self) -> Optional[str]: return self._svg
    def training_meta(self) -> Optional[dict]: return self._meta

    def errors(self) -> List[BaseException]:
        """Exceptions raised by this process's workers or coordinator so far."""
        return [v for k, v in self._results.items() if k.startswith("worker_err") or k == "coord_err"]

    def setup_monitor(self, monitor) -> None:
        """Hand the model's picture, identity and the run's metadata to a `Monitor`."""
        if self._svg is not None and hasattr(monitor, "set_architecture_svg"):
            monitor.set_architecture_svg(self._svg)
        if hasattr(monitor, "set_identity"):
            monitor.set_identity(self._label, self._hash)
        if self._meta is not None and hasattr(monitor, "set_metadata"):
            monitor.set_metadata(self._meta)

    def poll_metrics(self) -> List[EpochMetrics]:
        out = []
        while True:
            try:
                out.append(self._metrics.get_nowait())
            except queue.Empty:
                return out

    def next_metrics(self, timeout: Optional[float] = None) -> Optional[EpochMetrics]:
        """Blocks until the next epoch has been aggregated. None once the job is over (the coordinator has finished and
        nothing is queued), or when `timeout` seconds pass without a new epoch."""
        import time
        deadline = None if timeout is None else time.monotonic() + float(timeout)
        while True:
            try:
                return self._metrics.get(timeout=0.1)
            except queue.Empty:
                if self._coordinator is None or not self._coordinator.is_alive():
                    try:
                        return self._metrics.get_nowait()
                    except queue.Empty:
                        return None
                if deadline is not None and time.monotonic() >= deadline:
                    return None

    def _abort_collectives(self) -> None:
        for w in self._gpu_workers:
            w.abort_collectives()

    def join(self) -> TrainedState:
        if self._final is not None:
            return self._final
        first_err = None
        for th in self._workers:
            th.join()
        for k, v in list(self._results.items()):
            if k.startswith("worker_err") and first_err is None:
                first_err = v
                self._stop.set()
                self._abort_collectives()
        if self._coordinator is not None:
            if first_err is not None:
                self._stop.set()
            self._coordinator.join()
        state = self._results.get("state")
        cerr = self._results.get("coord_err")
        if self._broadcast_final:
            state = _share_final_state(state)
        if state is not None:
            if first_err is not None:
                log.msg(f"  ddp: WARNING: training state recovered but a worker failed: {first_err!r}")
            self._final = state
            return state
        err = first_err or cerr
        if err is not None:
            raise err
        raise TensorError("join: no trained state available")


def _share_final_state(state: Optional[TrainedState]) -> Optional[TrainedState]:
    """Multi-process runs: rank 0 holds the averaged result; every rank's `join()` returns it."""
    import torch.distributed as dist
    box = [state]
    dist.broadcast_object_list(box, src=0)
    return box[0]


class DdpBuilder:
    def __init__(self, model_factory: Callable, optim_factory: Callable, train_fn: Callable):
        self.model_factory, self.optim_factory, self.train_fn = model_factory, optim_factory, train_fn
        self._dataset = None
        self._batch_size: Optional[int] = None
        self._num_epochs: Optional[int] = None
        self._policy = ApplyPolicy.Cadence
        self._backend = AverageBackend.Nccl
        self._cfg = DdpRunConfig()
        self._checkpoint_fn = None
        self._scheduler_fn = None
        self._epoch_fn = None
        self._metrics_fn = None
        self._devices: Optional[List] = None
        self._cuda_graph = False

    # ---- configuration (orchestrator.rs:1117-1359) ----------------------------------------------
    def dataset(self, ds): self._dataset = ds; return self
    def batch_size(self, n): self._batch_size = int(n); return self
    def num_epochs(self, n): self._num_epochs = int(n); return self
    def policy(self, p: ApplyPolicy): self._policy = p; return self
    def backend(self, b: AverageBackend): self._backend = b; return self
    def overhead_target(self, t): self._cfg.overhead_target = float(t); return self
    def max_anchor(self, m): self._cfg.max_anchor = int(m); return self
    def anchor(self, a): self._cfg.anchor = int(a); return self
    def divergence_threshold(self, t): self._cfg.divergence_threshold = float(t); return self
    def no_divergence_guard(self): self._cfg.no_divergence_guard = True; return self
    def max_batch_diff(self, d): self._cfg.max_batch_diff = int(d); return self
    def max_overshoot(self, n): self._cfg.max_overshoot = int(n); return self
    def checkpoint_every(self, n): self._cfg.checkpoint_every = int(n); return self
    def progressive_dispatch(self, on): self._cfg.progressive_dispatch = bool(on); return self
    def max_grad_norm(self, n): self._cfg.max_grad_norm = float(n); return self
    def timeline(self, tl): self._cfg.timeline = tl; return self
    def lr_scale_ratio(self, r): self._cfg.lr_scale_ratio = float(r); return self
    def partition_ratios(self, r): self._cfg.partition_ratios = list(r); return self
    def snapshot_timeout(self, secs): self._cfg.snapshot_timeout_secs = float(secs); return self
    def config(self, cfg: DdpRunConfig): self._cfg = cfg; return self
    def checkpoint_fn(self, f): self._checkpoint_fn = f; return self
    def scheduler(self, f): self._scheduler_fn = f; return self
    def epoch_fn(self, f): self._epoch_fn = f; return self
    def metrics_fn(self, f): self._metrics_fn = f; return self

    def devices(self, devs: Sequence):
        """Run one worker THREAD per listed device inside this process (the reference's layout)."""
        self._devices = [torch.device(d) for d in devs]
        return self

    def cuda_graph(self, on: bool = True):
        """Capture each worker's training step (forward, backward, clip, optimizer) as one CUDA
        graph; batches must then keep one shape."""
        self._cuda_graph = bool(on)
        return self

    # ---- launch ---------------------------------------------------------------------------------
    def _el_che(self, world: int) -> ElChe:
        e = ElChe(max(2, world), self._cfg.anchor if self._cfg.anchor is not None else DEFAULT_ANCHOR)   # a lone device never consults it
        if self._cfg.overhead_target is not None:
            e.with_overhead_target(self._cfg.overhead_target)
        if self._cfg.max_anchor is not None:
            e.with_max_anchor(self._cfg.max_anchor)
        if self._cfg.max_batch_diff is not None:
            e.with_max_batch_diff(self._cfg.max_batch_diff)
        return e

    def _fixed_cadence(self, collective: bool) -> Optional[int]:
        """`anchor(k)` together with `max_anchor(k)` pins the cadence; with the collective backend
        the workers then average every k local steps on their own, without a round trip."""
        c = self._cfg
        if collective and self._policy == ApplyPolicy.Cadence and c.anchor is not None and c.anchor == c.max_anchor:
            return int(c.anchor)
        return None

    def _lr_factor(self, world: int) -> float:
        if world > 1 and self._cfg.lr_scale_ratio > 0.0:
            f = 1.0 + (world - 1) * self._cfg.lr_scale_ratio
            log.verbose(f"  ddp: LR scaled by {f:.2f}x (ratio={self._cfg.lr_scale_ratio:.2f}, world_size={world}). Adjust with .lr_scale_ratio()")
            return f
        return 1.0

    def _meta(self, devices: List, progressive: bool, total: int) -> dict:
        c = self._cfg
        names = [torch.cuda.get_device_name(d) if torch.device(d).type == "cuda" and torch.cuda.is_available() else str(d) for d in devices]
        return {"gpus": len(devices), "gpu_names": names, "policy": self._policy.value, "backend": self._backend.value,
                "batch_size": self._batch_size, "num_epochs": self._num_epochs, "total_samples": total,
                "progressive_dispatch": progressive, "anchor": c.anchor, "max_anchor": c.max_anchor,
                "overhead_target": c.overhead_target, "max_batch_diff": c.max_batch_diff, "max_grad_norm": c.max_grad_norm,
                "lr_scale_ratio": c.lr_scale_ratio}

    def run(self) -> DdpHandle:
        if self._dataset is None:
            raise TensorError("DdpBuilder: dataset is required")
        if not self._batch_size:
            raise TensorError("DdpBuilder: batch_size is required")
        if not self._num_epochs:
            raise TensorError("DdpBuilder: num_epochs is required")
        multi_process = _comm.world_size() > 1 and self._devices is None
        if multi_process:
            return self._run_processes()
        devices = self._devices
        if devices is None:
            devices = [torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")]
        return self._run_threads(devices)

    def _coordinator(self, transport, world: int, total: int, metrics_q, fixed: Optional[int], backend: AverageBackend,
                     device_indices: List[int]) -> Coordinator:
        c = self._cfg
        progressive = c.progressive_dispatch
        if fixed is not None:
            progressive = False
        return Coordinator(transport, self._policy, backend, world, total, self._el_che(world), batch_size=self._batch_size,
                           num_epochs=self._num_epochs, progressive=progressive,
                           divergence_threshold=c.divergence_threshold if c.divergence_threshold is not None else 0.05,
                           divergence_guard=not c.no_divergence_guard, checkpoint_every=c.checkpoint_every,
                           snapshot_timeout_secs=c.snapshot_timeout_secs, partition_ratios=c.partition_ratios,
                           max_overshoot=c.max_overshoot, device_indices=device_indices, metrics_fn=self._metrics_fn,
                           epoch_metrics_sink=metrics_q, timeline=c.timeline, fixed_cadence=fixed)

    def _describe(self, model):
        g = model.as_graph() if hasattr(model, "as_graph") else None
        if g is None:
            return None, None, None
        svg = None
        try:
            svg = g.svg()
            svg = svg.decode() if isinstance(svg, (bytes, bytearray)) else svg
        except Exception:
            svg = None
        return svg, g.label(), g.structural_hash()

    def _worker_thread(self, wcfg: WorkerConfig, transport, collective: bool, stop: threading.Event, results: dict,
                       lr_factor: float, registry: List[GpuWorker], name: str) -> threading.Thread:
        # Autocast state is per thread (PyTorch's and this package's): the workers inherit the state of the thread
        # that calls run(), so `with AutocastGuard(bf16): builder.run().join()` trains in bf16.
        from ... import ops as _ops_mod
        inherited = _ops_mod.FLAGS.autocast

        def body():
            guard = None
            try:
                if wcfg.device.type == "cuda":
                    torch.cuda.set_device(wcfg.device)
                if inherited is not None:
                    from ...nn.amp import AutocastGuard
                    guard = AutocastGuard(inherited, wcfg.device.type)
                w = GpuWorker(wcfg, self.model_factory, self.optim_factory, self._dataset, transport, self._checkpoint_fn, collective)
                registry.append(w)
                sched = self._scheduler_fn(wcfg.world_size) if self._scheduler_fn is not None else None
                if lr_factor > 1.0:
                    if sched is not None:
                        w.set_lr_scale(lr_factor)
                    else:
                        w.scale_lr(lr_factor)
                if sched is not None:
                    w.set_scheduler(sched)
                w.run(self.train_fn, self._epoch_fn, stop)
            except BaseException as e:
                log.msg(f"  ddp: worker {wcfg.rank} error: {e!r}")
                results[f"worker_err{wcfg.rank}"] = e
                try:
                    from .messages import TimingExiting
                    transport.box(f"tim{wcfg.rank}").send(TimingExiting(wcfg.rank, repr(e)))
                except Exception:
                    pass
                stop.set()
            finally:
                if guard is not None:
                    guard.release()
        return threading.Thread(target=body, name=name, daemon=True)

    def _coord_thread(self, coord: Coordinator, stop: threading.Event, results: dict) -> threading.Thread:
        def body():
            try:
                coord.stop = stop
                results["state"] = coord.run()
                if coord.error is not None:
                    results["coord_err"] = coord.error
            except BaseException as e:
                results["coord_err"] = e
                stop.set()
        return threading.Thread(target=body, name="ddp-coordinator", daemon=True)

    def _run_threads(self, devices: List[torch.device]) -> DdpHandle:
        world = len(devices)
        total = len(self._dataset)
        tmp = self.model_factory(devices[0])
        init_p = [p.t.detach().to("cpu", copy=True) for p in tmp.parameters()]
        init_b = [b.get().detach().to("cpu", copy=True) for b in tmp.buffers()]
        svg, label, ghash = self._describe(tmp)
        del tmp
        transport = LocalTransport()
        stop = threading.Event()
        results: dict = {}
        metrics_q: "queue.Queue" = queue.Queue()
        backend = AverageBackend.Cpu       # threads of one process cannot run a cross-process collective
        policy = self._policy if world > 1 else ApplyPolicy.Sync
        coord = self._coordinator(transport, world, total, metrics_q, None, backend, [d.index or 0 for d in devices])
        if world == 1:
            coord.policy = policy
            coord.progressive = False
            log.verbose(f"  ddp: single device ({devices[0]}) | no coordination")
        lr_factor = self._lr_factor(world)
        registry: List[GpuWorker] = []
        workers = []
        for rank, dev in enumerate(devices):
            wcfg = WorkerConfig(rank, world, dev, init_p, init_b, total, self._batch_size, SEED, self._cfg.max_grad_norm,
                                self._cfg.timeline, policy, None, self._cuda_graph)
            workers.append(self._worker_thread(wcfg, transport, False, stop, results, lr_factor, registry, f"ddp-gpu-{rank}"))
        cth = self._coord_thread(coord, stop, results)
        cth.start()
        for th in workers:
            th.start()
        progressive = coord.progressive
        return DdpHandle(workers, cth, devices, stop, metrics_q, results, True, svg, label, ghash,
                         self._meta(devices, progressive, total), registry)

    def _run_processes(self) -> DdpHandle:
        import torch.distributed as dist
        world, rank = _comm.world_size(), _comm.rank()
        total = len(self._dataset)
        dev = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() and dist.get_backend() == "nccl" else torch.device("cpu")
        _RUN_COUNTER[0] += 1
        transport = make_store_transport(f"ddp{_RUN_COUNTER[0]}")
        all_devs = [None] * world
        dist.all_gather_object(all_devs, str(dev))
        stop = threading.Event()
        results: dict = {}
        metrics_q: "queue.Queue" = queue.Queue()
        collective = self._backend == AverageBackend.Nccl
        fixed = self._fixed_cadence(collective)
        cth = None
        progressive = False
        if rank == 0:
            coord = self._coordinator(transport, world, total, metrics_q, fixed, self._backend, list(range(world)))
            progressive = coord.progressive
            cth = self._coord_thread(coord, stop, results)
        lr_factor = self._lr_factor(world)
        registry: List[GpuWorker] = []
        wcfg = WorkerConfig(rank, world, dev, None, None, total, self._batch_size, SEED, self._cfg.max_grad_norm, self._cfg.timeline,
                            self._policy, fixed, self._cuda_graph)
        # the worker thread allocates the peer-mapped buffers (a collective step over the default
        # process group): do not issue collectives from other threads until the first epoch runs
        wth = self._worker_thread(wcfg, transport, collective, stop, results, lr_factor, registry, f"ddp-gpu-{rank}")
        if cth is not None:
            cth.start()
        wth.start()
        return DdpHandle([wth], cth, all_devs, stop, metrics_q, results, rank == 0, None, None, None,
                         self._meta(all_devs, progressive, total) if rank == 0 else None, registry, broadcast_final=True)
