"""Character-level language-modelling windows from a text: vocabulary = sorted unique characters,
non-overlapping windows of `seq_len`, target = input shifted by one character."""
from __future__ import annotations

from typing import List, Sequence, Tuple

import torch

from ...tensor import TensorError
from ..dataset import TensorDataSet


class Shakespeare(TensorDataSet):
    def __init__(self, data: torch.Tensor, targets: torch.Tensor, idx_to_char: List[str]):
        super().__init__(data, targets)
        self.data, self.targets = data, targets
        self.idx_to_char = idx_to_char
        self.char_to_idx: List[Tuple[str, int]] = [(c, i) for i, c in enumerate(idx_to_char)]
        self.vocab_size = len(idx_to_char)

    @classmethod
    def parse(cls, text: str, seq_len: int) -> "Shakespeare":
        if len(text) < seq_len + 1:
            raise TensorError(f"Shakespeare: text length {len(text)} too short for seq_len {seq_len}")
        vocab = sorted(set(text))
        lut = {c: i for i, c in enumerate(vocab)}
        enc = torch.tensor([lut[c] for c in text], dtype=torch.long)
        n = (enc.numel() - 1) // seq_len
        if n == 0:
            raise TensorError("Shakespeare: not enough text for even one sequence")
        data = enc[:n * seq_len].view(n, seq_len).clone()
        targets = enc[1:n * seq_len + 1].view(n, seq_len).clone()
        return cls(data, targets, vocab)

    @classmethod
    def from_file(cls, path: str, seq_len: int) -> "Shakespeare":
        with open(path, "r", encoding="utf-8") as f:
            return cls.parse(f.read(), seq_len)

    def decode(self, indices: Sequence[int]) -> str:
        return "".join(self.idx_to_char[int(i)] if 0 <= int(i) < self.vocab_size else "?" for i in indices)
