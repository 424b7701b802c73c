"""Weight initialisers (flodl/src/nn/init.rs:8-103). Draw order matters for reproducibility:
each layer draws its weight first, then its bias, in construction order, from PyTorch's global
generator (`manual_seed` controls it)."""
from __future__ import annotations

import math
from typing import Sequence

import torch

from ..tensor import Device


def _dev(device):
    return Device.of(device).torch if device is not None else torch.device("cpu")


def uniform(shape: Sequence[int], low: float, high: float, device=None) -> torch.Tensor:
    return torch.rand(tuple(shape), device=_dev(device)) * (high - low) + low


def normal(shape: Sequence[int], mean: float, std: float, device=None) -> torch.Tensor:
    return torch.randn(tuple(shape), device=_dev(device)) * std + mean


def kaiming_uniform(shape: Sequence[int], fan_in: int, a: float = math.sqrt(5.0), device=None) -> torch.Tensor:
    gain = math.sqrt(2.0 / (1.0 + a * a))
    bound = math.sqrt(3.0) * gain / math.sqrt(max(fan_in, 1))
    return torch.rand(tuple(shape), device=_dev(device)) * (2 * bound) - bound


def kaiming_normal(shape: Sequence[int], fan_in: int, a: float = 0.0, device=None) -> torch.Tensor:
    gain = math.sqrt(2.0 / (1.0 + a * a))
    return torch.randn(tuple(shape), device=_dev(device)) * (gain / math.sqrt(max(fan_in, 1)))


def xavier_uniform(shape: Sequence[int], fan_in: int, fan_out: int, device=None) -> torch.Tensor:
    bound = math.sqrt(6.0 / (fan_in + fan_out))
    return torch.rand(tuple(shape), device=_dev(device)) * (2 * bound) - bound


def xavier_normal(shape: Sequence[int], fan_in: int, fan_out: int, device=None) -> torch.Tensor:
    return torch.randn(tuple(shape), device=_dev(device)) * math.sqrt(2.0 / (fan_in + fan_out))


def uniform_bias(fan_in: int, shape: Sequence[int], device=None) -> torch.Tensor:
    bound = 1.0 / math.sqrt(max(fan_in, 1))
    return torch.rand(tuple(shape), device=_dev(device)) * (2 * bound) - bound


def trunc_normal(shape: Sequence[int], mean: float = 0.0, std: float = 1.0, a: float = -2.0, b: float = 2.0, device=None) -> torch.Tensor:
    t = torch.empty(tuple(shape), device=_dev(device))
    torch.nn.init.trunc_normal_(t, mean, std, a, b)
    return t


def orthogonal(shape: Sequence[int], gain: float = 1.0, device=None) -> torch.Tensor:
    """Gram-Schmidt (QR) on a random normal matrix, done on the host."""
    rows = shape[0]
    cols = int(torch.tensor(list(shape[1:])).prod().item()) if len(shape) > 1 else 1
    flat = torch.randn(max(rows, cols), min(rows, cols))
    q, r = torch.linalg.qr(flat)
    q = q * torch.sign(torch.diagonal(r))
    if rows < cols:
        q = q.t()
    return (q[:rows, :cols] * gain).reshape(tuple(shape)).to(_dev(device))
