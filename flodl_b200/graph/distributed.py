"""Graph-level data parallelism hooks (flodl/src/graph/distributed.rs). The methods are mixed
into `Graph`; the machinery lives in `flodl_b200.parallel.ddp`."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional


@dataclass
class LossContext:
    """What a loss function bound with `set_loss_fn` receives for every batch
    (flodl/src/graph/mod.rs:60-69): the live forward output, the batch with all named fields,
    the tagged outputs and the loop traces of this forward pass."""
    output: object
    batch: object
    tags: Dict[str, object] = field(default_factory=dict)
    traces: Dict[str, list] = field(default_factory=dict)


class GraphEpochIterator:
    """Handle on one epoch of the bound loader (`Graph.epoch(n)`); iteration starts with `activate()`
    or with the first `next()` (flodl/src/graph/graph.rs:1150-1230). With a loss function bound
    (`set_loss_fn`) each item has already been run: forward on the batch's input field, loss,
    backward; the item is then `(batch, loss)`. Without one the item is the `Batch`."""

    def __init__(self, graph, epoch: int):
        self.graph, self.epoch_index = graph, epoch
        self._active = None

    def activate(self) -> "ActiveGraphEpochIterator":
        if self._active is None:
            self._active = ActiveGraphEpochIterator(self.graph, self.epoch_index)
        return self._active

    def __iter__(self):
        return self.activate()

    def __next__(self):
        return next(self.activate())

    def __len__(self) -> int:
        return len(self.activate())


class ActiveGraphEpochIterator:
    """The running form of `GraphEpochIterator`. Knows how many batches are left. When it ends (or is
    closed) on an El Che cadence with gradients accumulated and not yet combined, it calls
    `graph.step()` so that the epoch's last batches are not lost (graph.rs:1232-1250)."""

    def __init__(self, graph, epoch: int):
        self.graph, self.epoch_index = graph, epoch
        loader, self.input_name = graph._data_binding
        self._it = loader.epoch(epoch)
        self._done = False

    def __iter__(self):
        return self

    def __len__(self) -> int:
        return len(self._it) if hasattr(self._it, "__len__") else 0

    def size_hint(self):
        n = len(self)
        return n, n

    def __next__(self):
        try:
            batch = next(self._it)
        except StopIteration:
            self.close()
            raise
        g = self.graph
        if g._loss_fn is None:
            return batch
        x = batch[self.input_name] if hasattr(batch, "has") and batch.has(self.input_name) else batch[0]
        if g._ddp is not None and not g._ddp.scatter:
            g._ddp.begin_batch(int(x.shape[0]))
        out = g.forward(x)
        tags = {n: g.tagged(n) for n in g.tag_names_list()} if hasattr(g, "tag_names_list") else {}
        loss = g._loss_fn(LossContext(out, batch, tags, {}))
        loss.backward()
        return batch, loss

    def close(self) -> None:
        if self._done:
            return
        self._done = True
        if hasattr(self._it, "close"):
            self._it.close()
        g = self.graph
        if g.has_el_che() and getattr(g._ddp, "_acc_batches", 0) > 0 and g._optimizer is not None:
            g.step()


class DistributedMixin:
    def _init_distributed(self) -> None:
        self._ddp = None            # parallel.ddp.DistributedState once distribute() ran
        self._optimizer = None
        self._scheduler = None
        self._lr_scale = 1.0
        self._training_step = 0
        self._data_binding = None
        self._loss_fn = None

    # ---- setup ----------------------------------------------------------------------------------
    def distribute(self, factory: Optional[Callable] = None, **kw):
        from ..parallel import ddp
        self._ddp = ddp.DistributedState.for_graph(self, factory, **kw)
        return self

    def auto_distribute(self, factory: Optional[Callable] = None, **kw):
        from ..parallel import comm
        if comm.world_size() > 1:
            self.distribute(factory, **kw)
        return self

    def is_distributed(self) -> bool:
        return self._ddp is not None and self._ddp.intercepts_forward()

    def world_size(self) -> int:
        return self._ddp.world_size if self._ddp is not None else 1

    def devices(self) -> List:
        return self._ddp.devices() if self._ddp is not None else [p.t.device for p in self.parameters()[:1]]

    def has_el_che(self) -> bool:
        return self._ddp is not None and self._ddp.el_che is not None

    def chunk_ratios(self) -> List[float]:
        return self._ddp.chunk_ratios() if self._ddp is not None else [1.0]

    def throughput(self) -> List[float]:
        return self._ddp.throughput() if self._ddp is not None else []

    def shard_sizes(self, batch: int) -> List[int]:
        return self._ddp.shard_sizes(batch) if self._ddp is not None else [batch]

    def forward_distributed(self, x):
        return self._ddp.forward(self, x)

    # ---- optimizer / schedule -------------------------------------------------------------------
    def set_optimizer(self, factory: Callable) -> None:
        """`factory(parameters) -> Optimizer`; one optimizer per replica (here: per process)."""
        self._optimizer = factory(self.parameters())

    def optimizer(self):
        return self._optimizer

    def set_scheduler(self, scheduler) -> None:
        self._scheduler = scheduler

    def set_lr_scale(self, scale: float) -> None:
        self._lr_scale = float(scale)

    def set_lr(self, lr: float) -> None:
        if self._optimizer is not None:
            self._optimizer.set_lr(lr)

    def training_step(self) -> int:
        return self._training_step

    def step(self) -> None:
        """All-reduce gradients (when distributed), sync buffers, apply the scheduled learning
        rate, optimizer step, zero gradients (graph/distributed.rs:239-452)."""
        if self._optimizer is None:
            from ..tensor import TensorError
            raise TensorError("step(): call set_optimizer first")
        if self._ddp is not None:
            self._ddp.before_optimizer()
        if self._scheduler is not None:
            self._optimizer.set_lr(self._scheduler.lr(self._training_step) * self._lr_scale)
        if self._ddp is not None:
            self._ddp.guard_optimizer(self._optimizer)
        self._optimizer.step()
        self._optimizer.zero_grad()
        self._training_step += 1
        if self._ddp is not None:
            self._ddp.after_step()

    # ---- data binding ---------------------------------------------------------------------------
    def set_data_loader(self, loader, input_name: str = "input") -> None:
        """Bind a `DataLoader`; in a multi-rank job the loader is restricted to this rank's shard
        and the forward pass no longer scatters (the data arrives pre-sharded,
        flodl/src/graph/distributed.rs:843-939)."""
        from ..parallel import comm
        if comm.world_size() > 1 and hasattr(loader, "distributed"):
            loader.distributed(comm.rank(), comm.world_size())
            if self._ddp is not None:
                self._ddp.scatter = False
                loader.set_shard_ratios(None if self._ddp.is_balanced() else self._ddp.chunk_ratios())
        self._data_binding = (loader, input_name)

    def set_loss_fn(self, f: Callable) -> None:
        self._loss_fn = f

    def has_loss_fn(self) -> bool:
        return self._loss_fn is not None

    def data_num_batches(self) -> int:
        return self._data_binding[0].num_batches() if self._data_binding else 0

    def data_batch_size(self) -> int:
        return self._data_binding[0].batch_size if self._data_binding else 0

    def epoch(self, epoch: int) -> "GraphEpochIterator":
        """Batches of `epoch` from the bound loader (see `GraphEpochIterator`)."""
        if self._data_binding is None:
            from ..tensor import TensorError
            raise TensorError("epoch(): call set_data_loader first")
        return GraphEpochIterator(self, epoch)

    def forward_batch(self, batch):
        from ..autograd import Variable
        x = batch[0] if isinstance(batch, (list, tuple)) else batch
        return self.forward(x if isinstance(x, Variable) else Variable.wrap(x))
