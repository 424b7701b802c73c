"""CIFAR-10 from its binary batch files: 10 000 records of 1 label byte + 3072 pixel bytes
(already channel-major). Images become float32 `[N,3,32,32]` in [0,1], labels int64 `[N]`."""
from __future__ import annotations

from typing import Sequence

import numpy as np
import torch

from ...tensor import TensorError
from ..dataset import TensorDataSet

IMAGES_PER_BATCH = 10_000
PIXELS_PER_IMAGE = 3 * 32 * 32
BYTES_PER_RECORD = 1 + PIXELS_PER_IMAGE


class Cifar10(TensorDataSet):
    def __init__(self, images: torch.Tensor, labels: torch.Tensor):
        super().__init__(images, labels)
        self.images, self.labels = images, labels

    @classmethod
    def parse(cls, batches: Sequence[bytes]) -> "Cifar10":
        if not batches:
            raise TensorError("CIFAR-10: no batch data provided")
        imgs, labs = [], []
        for bi, raw in enumerate(batches):
            expected = IMAGES_PER_BATCH * BYTES_PER_RECORD
            if len(raw) != expected:
                raise TensorError(f"CIFAR-10 batch {bi}: expected {expected} bytes, got {len(raw)}")
            rec = np.frombuffer(raw, dtype=np.uint8).reshape(IMAGES_PER_BATCH, BYTES_PER_RECORD)
            lab = rec[:, 0].astype(np.int64)
            if lab.max() > 9:
                bad = int(np.argmax(lab > 9))
                raise TensorError(f"CIFAR-10 batch {bi} image {bad}: invalid label {int(lab[bad])}")
            labs.append(lab)
            imgs.append(rec[:, 1:].astype(np.float32) / 255.0)
        images = torch.from_numpy(np.concatenate(imgs)).view(-1, 3, 32, 32)
        labels = torch.from_numpy(np.concatenate(labs))
        return cls(images, labels)

    @classmethod
    def from_files(cls, paths: Sequence[str]) -> "Cifar10":
        blobs = []
        for p in paths:
            with open(p, "rb") as f:
                blobs.append(f.read())
        return cls.parse(blobs)
