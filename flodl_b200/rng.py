"""Host-side random numbers independent of the tensor library's generator: Xoshiro256++ seeded
through SplitMix64, implemented in the C++ runtime (flodl/src/rng.rs). Used by samplers, the
DDP partitioner and anything that must shuffle identically on every rank."""
from __future__ import annotations

from typing import List, MutableSequence, Sequence, TypeVar

from . import _ext

T = TypeVar("T")


class Rng:
    def __init__(self, seed: int):
        self._r = _ext.require().Rng(int(seed) & 0xFFFFFFFFFFFFFFFF)

    @classmethod
    def seed(cls, seed: int) -> "Rng":
        return cls(seed)

    @classmethod
    def from_entropy(cls) -> "Rng":
        import os
        return cls(int.from_bytes(os.urandom(8), "little"))

    def usize(self, n: int) -> int:
        """Uniform integer in [0, n)."""
        return self._r.usize(int(n))

    def f32(self) -> float:
        return self._r.f32()

    def f64(self) -> float:
        return self._r.f64()

    def bernoulli(self, p: float) -> bool:
        return self._r.bernoulli(float(p))

    def range(self, lo: int, hi: int) -> int:
        """Uniform integer in [lo, hi)."""
        return self._r.range(int(lo), int(hi))

    def normal(self, mean: float = 0.0, std: float = 1.0) -> float:
        return self._r.normal(float(mean), float(std))

    def permutation(self, n: int) -> List[int]:
        return list(self._r.permutation(int(n)))

    def shuffle(self, items: MutableSequence[T]) -> None:
        """In place, Fisher-Yates."""
        perm = self._r.permutation(len(items))
        snapshot = list(items)
        for i, j in enumerate(perm):
            items[i] = snapshot[j]

    def choice(self, items: Sequence[T]) -> T:
        return items[self.usize(len(items))]
