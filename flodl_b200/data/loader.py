"""`DataLoader`: batches for an epoch, resident on the device or streamed
(flodl/src/data/loader.rs).

Mode selection (`build()`): a dataset whose tensors fit into the device's free memory under the
usage cap (default 90 % of total) is copied there once and batches are device-side row gathers;
otherwise (or with `.streaming()`, or if the resident copy runs out of memory) batches come from
a `PrefetchWorker`, whose depth is re-derived from free memory at every epoch. On 180 GB parts
almost every benchmark dataset is resident.

`DataLoader.distributed(rank, world)` restricts every epoch to this rank's shard of the global
order (equal shards by default, `set_shard_ratios` for unequal ones).
"""
from __future__ import annotations

from typing import Iterator, List, Optional, Sequence

import torch

from ..tensor import TensorError
from .dataset import Batch, BatchDataSet, DataSet, DataSetAdapter, TensorDataSet
from .prefetch import PrefetchWorker
from .sampler import RandomSampler, Sampler, SequentialSampler

VRAM_MAX_USAGE = 0.90
BOOTSTRAP_PREFETCH = 4


def _mem_info(device: torch.device):
    try:
        return torch.cuda.mem_get_info(device)
    except Exception:
        return None


def can_fit_resident(n: int, per_sample_bytes: int, device: torch.device, max_usage: float = VRAM_MAX_USAGE) -> bool:
    """CPU: always. CUDA: the dataset must fit between current usage and `max_usage` of total."""
    if device.type != "cuda":
        return True
    info = _mem_info(device)
    if info is None:
        return False
    free, total = info
    budget = max(0, int(total * max_usage) - (total - free))
    return per_sample_bytes * n < budget


def prefetch_depth_from_vram(per_sample_bytes: int, batch_size: int, device, max_usage: float = VRAM_MAX_USAGE,
                             activation_reserve: int = 0) -> int:
    """How many batches may wait on the device: the gap between current usage (+ a reserve for
    activations) and the usage cap, in batches. CPU targets double-buffer."""
    device = torch.device(device)
    batch_bytes = per_sample_bytes * batch_size
    if device.type != "cuda" or batch_bytes == 0:
        return 2
    info = _mem_info(device)
    if info is None:
        return 2
    free, total = info
    cap = int(total * min(0.99, max(0.5, max_usage)))
    budget = max(0, cap - ((total - free) + activation_reserve))
    return budget // batch_bytes


class DataLoaderBuilder:
    def __init__(self, dataset: BatchDataSet):
        self._ds = dataset
        self._batch_size: Optional[int] = None
        self._device = torch.device("cpu")
        self._seed = 42
        self._shuffle = True
        self._sampler: Optional[Sampler] = None
        self._prefetch: Optional[int] = None
        self._max_usage = VRAM_MAX_USAGE
        self._streaming = False
        self._names: Optional[List[str]] = None
        self._drop_last = True

    def batch_size(self, n: int): self._batch_size = int(n); return self
    def device(self, d): self._device = torch.device(d.torch if hasattr(d, "torch") else d); return self
    def seed(self, s: int): self._seed = int(s); return self
    def shuffle(self, on: bool): self._shuffle = bool(on); return self
    def sampler(self, s: Sampler): self._sampler = s; return self
    def prefetch(self, depth: int): self._prefetch = int(depth); return self
    def vram_max_usage(self, f: float): self._max_usage = float(f); return self
    def streaming(self): self._streaming = True; return self
    def names(self, names: Sequence[str]): self._names = list(names); return self
    def drop_last(self, on: bool): self._drop_last = bool(on); return self

    def build(self) -> "DataLoader":
        if not self._batch_size or self._batch_size <= 0:
            raise TensorError("DataLoader: batch_size is required and must be > 0")
        n = len(self._ds)
        if n == 0:
            raise TensorError("DataLoader: dataset is empty")
        sampler = self._sampler or (RandomSampler(n, self._seed) if self._shuffle else SequentialSampler(n))
        probe = self._ds.get_batch([0])
        per_sample = sum(t.numel() * t.element_size() for t in probe)
        if self._names is not None and len(self._names) != len(probe):
            raise TensorError(f"DataLoader: {len(self._names)} names for {len(probe)} tensors per sample")
        resident = None
        if not self._streaming and can_fit_resident(n, per_sample, self._device, self._max_usage):
            try:
                if isinstance(self._ds, TensorDataSet):
                    resident = [t.to(self._device) for t in self._ds.tensors()]
                else:
                    resident = [t.to(self._device) for t in self._ds.get_batch(list(range(n)))]
            except torch.cuda.OutOfMemoryError:
                resident = None               # fall back to streaming
                torch.cuda.empty_cache()
        return DataLoader(self._ds, self._batch_size, self._device, sampler, resident, per_sample,
                          self._prefetch, self._max_usage, self._names, self._drop_last)


class DataLoader:
    def __init__(self, dataset, batch_size, device, sampler, resident, per_sample_bytes, prefetch, max_usage, names, drop_last):
        self._ds, self.batch_size, self._device, self._sampler = dataset, int(batch_size), device, sampler
        self._resident = resident
        self._per_sample = per_sample_bytes
        self._user_prefetch = prefetch
        self._max_usage = max_usage
        self._names = names
        self._drop_last = drop_last
        self._worker: Optional[PrefetchWorker] = None
        self._depth = prefetch if prefetch is not None else BOOTSTRAP_PREFETCH
        self._rank, self._world = 0, 1
        self._shard_ratios: Optional[List[float]] = None

    # ---- constructors ---------------------------------------------------------------------------
    @staticmethod
    def from_dataset(dataset: DataSet) -> DataLoaderBuilder:
        return DataLoaderBuilder(DataSetAdapter(dataset))

    @staticmethod
    def from_batch_dataset(dataset: BatchDataSet) -> DataLoaderBuilder:
        return DataLoaderBuilder(dataset)

    # ---- queries --------------------------------------------------------------------------------
    def __len__(self) -> int: return len(self._ds)
    def len(self) -> int: return len(self._ds)
    def is_empty(self) -> bool: return len(self._ds) == 0
    def device(self): return self._device
    def is_resident(self) -> bool: return self._resident is not None
    def names(self) -> List[str]: return list(self._names or [])
    def is_distributed(self) -> bool: return self._world > 1
    def prefetch_depth(self) -> int: return 0 if self.is_resident() else self._depth
    def dataset(self) -> BatchDataSet: return self._ds

    def num_batches(self) -> int:
        n = self._shard_len()
        return n // self.batch_size if self._drop_last else -(-n // self.batch_size)

    def set_prefetch_depth(self, depth: int) -> None:
        self._depth = max(1, int(depth))
        self._user_prefetch = self._depth

    def auto_resize(self) -> int:
        """Re-derive the prefetch depth from the memory that is free right now."""
        if self.is_resident():
            return 0
        self._depth = max(2, min(prefetch_depth_from_vram(self._per_sample, self.batch_size, self._device, self._max_usage), self.num_batches() or 1))
        return self._depth

    # ---- distribution ---------------------------------------------------------------------------
    def distributed(self, rank: int, world: int) -> "DataLoader":
        self._rank, self._world = int(rank), int(world)
        return self

    def set_shard_ratios(self, ratios: Optional[Sequence[float]]) -> None:
        self._shard_ratios = None if ratios is None else list(ratios)

    def _shard_bounds(self, n: int):
        if self._world <= 1:
            return 0, n
        if self._shard_ratios is None:
            base, rem = divmod(n, self._world)
            sizes = [base + (1 if r < rem else 0) for r in range(self._world)]
        else:
            s = sum(self._shard_ratios)
            sizes = [int(n * r / s) for r in self._shard_ratios]
            sizes[-1] = n - sum(sizes[:-1])
        start = sum(sizes[:self._rank])
        return start, start + sizes[self._rank]

    def _shard_len(self) -> int:
        a, b = self._shard_bounds(len(self._ds))
        return b - a

    # ---- iteration ------------------------------------------------------------------------------
    def epoch(self, epoch: int) -> "EpochIterator":
        order = self._sampler.indices(epoch)
        a, b = self._shard_bounds(len(order))
        order = order[a:b]
        gen = self._iter_resident(order) if self._resident is not None else self._iter_streaming(order)
        if self._world > 1:
            return DistributedEpochIterator(gen, self.num_batches(), self._rank, self._world, (a, b))
        return EpochIterator(gen, self.num_batches())

    def _iter_resident(self, order: List[int]) -> Iterator[Batch]:
        idx_all = torch.as_tensor(order, dtype=torch.long).to(self._device)
        bs = self.batch_size
        nb = self.num_batches()
        for b in range(nb):
            idx = idx_all[b * bs:(b + 1) * bs]
            yield Batch([t.index_select(0, idx) for t in self._resident], self._names)

    def _iter_streaming(self, order: List[int]) -> Iterator[Batch]:
        if self._user_prefetch is None:
            self.auto_resize()
        if self._worker is None:
            self._worker = PrefetchWorker(self._ds, self._device, self._depth)
        self._worker.set_prefetch_depth(self._depth)
        self._worker.start_epoch(order, self.batch_size, self._drop_last)
        try:
            while True:
                batch = self._worker.next()
                if batch is None:
                    return
                if self._device.type == "cpu":
                    batch = [t for t in batch]
                yield Batch(batch, self._names)
        finally:
            self._worker.stop()


class EpochIterator:
    """The batches of one epoch (`DataLoader.epoch`), already on the loader's device. Knows how many
    batches are left (`len(it)`, `size_hint()`); dropping or `close()`-ing it mid-epoch stops the
    prefetch worker of a streaming loader (flodl/src/data/loader.rs:861-900)."""

    def __init__(self, gen, num_batches: int):
        self._gen, self._remaining = gen, int(num_batches)

    def __iter__(self):
        return self

    def __next__(self) -> Batch:
        try:
            batch = next(self._gen)
        except StopIteration:
            self._remaining = 0
            raise
        self._remaining = max(0, self._remaining - 1)
        return batch

    def __len__(self) -> int:
        return self._remaining

    def size_hint(self):
        return self._remaining, self._remaining

    def close(self) -> None:
        self._gen.close()
        self._remaining = 0

    def __del__(self):
        try:
            self._gen.close()
        except Exception:
            pass


class DistributedEpochIterator(EpochIterator):
    """Epoch iterator of a loader that was sharded with `DataLoader.distributed(rank, world)`: this
    rank's slice `[lo, hi)` of the epoch's global permutation, cut by the current shard ratios
    (flodl/src/data/loader.rs:1180-1275; one process per GPU here, so each rank iterates its own)."""

    def __init__(self, gen, num_batches: int, rank: int, world: int, bounds):
        super().__init__(gen, num_batches)
        self.rank, self.world_size, self.shard_bounds = rank, world, tuple(bounds)
