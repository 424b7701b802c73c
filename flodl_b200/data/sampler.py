"""Index samplers (flodl/src/data/sampler.rs): a new order per epoch, reproducible per seed."""
from __future__ import annotations

from typing import List

from .. import _ext


class Sampler:
    def __len__(self) -> int:  # pragma: no cover - interface
        raise NotImplementedError

    def len(self) -> int:
        return len(self)

    def is_empty(self) -> bool:
        return len(self) == 0

    def indices(self, epoch: int) -> List[int]:  # pragma: no cover - interface
        raise NotImplementedError


class RandomSampler(Sampler):
    """Permutation of 0..n drawn from a generator seeded with `seed + epoch`."""

    def __init__(self, n: int, seed: int = 42):
        self.n, self.seed = int(n), int(seed)

    @classmethod
    def new(cls, n: int, seed: int) -> "RandomSampler":
        return cls(n, seed)

    def __len__(self) -> int:
        return self.n

    def indices(self, epoch: int) -> List[int]:
        return list(_ext.require().Rng(self.seed + int(epoch)).permutation(self.n))


class SequentialSampler(Sampler):
    def __init__(self, n: int):
        self.n = int(n)

    @classmethod
    def new(cls, n: int) -> "SequentialSampler":
        return cls(n)

    def __len__(self) -> int:
        return self.n

    def indices(self, epoch: int) -> List[int]:
        return list(range(self.n))
