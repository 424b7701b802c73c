"""Datasets, samplers and loaders (flodl/src/data/).

* `DataSet` - per-item access (`len`, `get(i) -> [tensors]`); `BatchDataSet` - batched access
  (`get_batch(indices) -> [tensors]`). A `DataSet` is adapted by stacking position-wise.
* `RandomSampler` (seeded per epoch) / `SequentialSampler`.
* `DataLoader` - resident (the whole dataset lives on the device, batches are `index_select`s) or
  streaming (a background worker gathers rows into pinned memory and copies them on its own
  stream, `PrefetchWorker`); chosen from free device memory unless forced.
"""
from .dataset import Batch, BatchDataSet, DataSet, DataSetAdapter, TensorDataSet  # noqa: F401
from .loader import DataLoader, DataLoaderBuilder, DistributedEpochIterator, EpochIterator, prefetch_depth_from_vram  # noqa: F401
from .prefetch import PrefetchWorker  # noqa: F401
from .sampler import RandomSampler, Sampler, SequentialSampler  # noqa: F401
