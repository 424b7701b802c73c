"""MNIST from its IDX files (big-endian headers; images magic 2051, labels magic 2049), raw or
gzip-compressed. Images become float32 `[N,1,rows,cols]` in [0,1], labels int64 `[N]`."""
from __future__ import annotations

import gzip
import struct
from typing import List, Sequence

import numpy as np
import torch

from ...tensor import TensorError
from ..dataset import TensorDataSet


def _maybe_gunzip(raw: bytes) -> bytes:
    return gzip.decompress(raw) if raw[:2] == b"\x1f\x8b" else raw


class Mnist(TensorDataSet):
    def __init__(self, images: torch.Tensor, labels: torch.Tensor):
        super().__init__(images, labels)
        self.images, self.labels = images, labels

    @classmethod
    def parse(cls, images_gz: bytes, labels_gz: bytes) -> "Mnist":
        img, lab = _maybe_gunzip(images_gz), _maybe_gunzip(labels_gz)
        if len(img) < 16:
            raise TensorError("MNIST images: file too short for header")
        magic, n, rows, cols = struct.unpack(">IIII", img[:16])
        if magic != 2051:
            raise TensorError(f"MNIST images: bad magic {magic}, expected 2051")
        count = n * rows * cols
        if len(img) < 16 + count:
            raise TensorError(f"MNIST images: expected {count} pixels, got {len(img) - 16}")
        if len(lab) < 8:
            raise TensorError("MNIST labels: file too short for header")
        lmagic, nl = struct.unpack(">II", lab[:8])
        if lmagic != 2049:
            raise TensorError(f"MNIST labels: bad magic {lmagic}, expected 2049")
        if nl != n:
            raise TensorError(f"MNIST: {n} images but {nl} labels")
        if len(lab) < 8 + n:
            raise TensorError("MNIST labels: truncated")
        px = np.frombuffer(img, dtype=np.uint8, count=count, offset=16).astype(np.float32) / 255.0
        images = torch.from_numpy(px).view(n, 1, rows, cols)
        labels = torch.from_numpy(np.frombuffer(lab, dtype=np.uint8, count=n, offset=8).astype(np.int64))
        return cls(images, labels)

    @classmethod
    def from_files(cls, images_path: str, labels_path: str) -> "Mnist":
        with open(images_path, "rb") as f, open(labels_path, "rb") as g:
            return cls.parse(f.read(), g.read())
