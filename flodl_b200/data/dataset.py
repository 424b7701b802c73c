"""Dataset protocols and the named `Batch` (flodl/src/data/mod.rs:88-340)."""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Union

import torch

from ..tensor import TensorError


class DataSet:
    """Per-item dataset: `len()` and `get(index) -> [tensor, ...]` (one sample, no batch dim)."""

    def __len__(self) -> int:  # pragma: no cover - interface
        raise NotImplementedError

    def len(self) -> int:
        return len(self)

    def get(self, index: int) -> List[torch.Tensor]:  # pragma: no cover - interface
        raise NotImplementedError

    def is_empty(self) -> bool:
        return len(self) == 0


class BatchDataSet:
    """Batched dataset: `get_batch(indices) -> [tensor, ...]`, each with a leading batch dim."""

    def __len__(self) -> int:  # pragma: no cover - interface
        raise NotImplementedError

    def len(self) -> int:
        return len(self)

    def get_batch(self, indices: Sequence[int]) -> List[torch.Tensor]:  # pragma: no cover - interface
        raise NotImplementedError

    def is_empty(self) -> bool:
        return len(self) == 0


class DataSetAdapter(BatchDataSet):
    """Turns a `DataSet` into a `BatchDataSet` by stacking the i-th tensors of every sample
    (mod.rs:140-180). An empty index list gives an empty batch list."""

    def __init__(self, inner: DataSet):
        self.inner = inner

    def __len__(self) -> int:
        return len(self.inner)

    def get_batch(self, indices: Sequence[int]) -> List[torch.Tensor]:
        if len(indices) == 0:
            return []
        items = [self.inner.get(int(i)) for i in indices]
        return [torch.stack([it[k] for it in items]) for k in range(len(items[0]))]


class TensorDataSet(BatchDataSet):
    """Whole-dataset tensors sharing dim 0; batches are row gathers. The loaders' fast paths
    (device-resident `index_select`, native pinned-memory prefetch) key on this class."""

    def __init__(self, *tensors: torch.Tensor):
        if not tensors:
            raise TensorError("TensorDataSet: at least one tensor")
        n = tensors[0].shape[0]
        for t in tensors:
            if t.shape[0] != n:
                raise TensorError("TensorDataSet: tensors disagree on dim 0")
        self._tensors = list(tensors)

    def tensors(self) -> List[torch.Tensor]:
        return self._tensors

    def __len__(self) -> int:
        return int(self._tensors[0].shape[0])

    def get_batch(self, indices: Sequence[int]) -> List[torch.Tensor]:
        idx = torch.as_tensor(list(indices) if not isinstance(indices, torch.Tensor) else indices, dtype=torch.long,
                              device=self._tensors[0].device)
        return [t.index_select(0, idx) for t in self._tensors]


class Batch:
    """One batch: tensors addressable by position or by name (`batch[0]`, `batch["image"]`).
    Unnamed batches get the names "0", "1", ... (mod.rs:242-330)."""

    def __init__(self, tensors: Sequence[torch.Tensor], names: Optional[Sequence[str]] = None):
        self._tensors = list(tensors)
        self._names = list(names) if names else [str(i) for i in range(len(self._tensors))]
        if len(self._names) != len(self._tensors):
            raise TensorError(f"Batch: {len(self._names)} names for {len(self._tensors)} tensors")
        self._index: Dict[str, int] = {n: i for i, n in enumerate(self._names)}

    def get(self, index: int) -> torch.Tensor:
        return self._tensors[index]

    def len(self) -> int:
        return len(self._tensors)

    def get_named(self, name: str) -> Optional[torch.Tensor]:
        i = self._index.get(name)
        return None if i is None else self._tensors[i]

    def has(self, name: str) -> bool:
        return name in self._index

    def names(self) -> List[str]:
        return list(self._names)

    def __len__(self) -> int:
        return len(self._tensors)

    def is_empty(self) -> bool:
        return not self._tensors

    def into_vec(self) -> List[torch.Tensor]:
        return list(self._tensors)

    def into_parts(self):
        return list(self._names), list(self._tensors)

    def __getitem__(self, key: Union[int, str]) -> torch.Tensor:
        if isinstance(key, str):
            if key not in self._index:
                raise KeyError(f"Batch has no tensor named {key!r} (names: {self._names})")
            return self._tensors[self._index[key]]
        return self._tensors[key]

    def __iter__(self):
        return iter(self._tensors)

    def __repr__(self) -> str:
        parts = ", ".join(f"{n}: {list(t.shape)}" for n, t in zip(self._names, self._tensors))
        return f"Batch({parts})"
