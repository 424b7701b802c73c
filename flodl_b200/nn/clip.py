"""Gradient clipping (flodl/src/nn/clip.rs:10-27, flodl-sys/ops_training.cpp:769-800).

`clip_grad_norm` returns the PRE-clip global L2 norm and scales every gradient by
`max_norm / (total + 1e-6)` when the total exceeds `max_norm`. On CUDA with gradients in a flat
buffer the norm is one fused reduction (`fb_grad_norm`) and the scaling one pass; the device-side
variant `clip_grad_norm_fused` avoids the host sync altogether by handing the coefficient to the
optimizer kernel as a device scalar.
"""
from __future__ import annotations

from typing import Sequence

import torch

from .. import _ext
from ..parallel import flat as _flat
from .module import Parameter


def _tensors(params):
    return [p.t if isinstance(p, Parameter) else p for p in params]


def clip_grad_norm_fused(params: Sequence, max_norm: float) -> torch.Tensor:
    """Device-resident result: fp32 [2] = {pre-clip norm, clip coefficient}. No host sync. The
    gradients are NOT modified; pass `out[1:2]` to `Optimizer.set_grad_scale`. Requires the
    gradients to live in one flat buffer on CUDA."""
    ts = _tensors(params)
    rng = _flat.contiguous_range(ts)
    if rng is None or not ts[0].is_cuda:
        raise ValueError("clip_grad_norm_fused needs CUDA parameters re-homed by FlatParams")
    flat, a, b = rng
    from .. import ops
    ops.core._launched(2)
    return _ext.require().grad_norm(flat.grads[a:b], float(max_norm), 1.0)


def clip_grad_norm(params: Sequence, max_norm: float) -> float:
    ts = [t for t in _tensors(params) if t.grad is not None]
    if not ts:
        return 0.0
    from .. import ops
    rng = _flat.contiguous_range(ts) if ts[0].is_cuda and ops.native_enabled() else None
    if rng is not None:
        flat, a, b = rng
        out = _ext.require().grad_norm(flat.grads[a:b], float(max_norm), 1.0)
        total, coef = out.tolist()
        if coef != 1.0:
            flat.grads[a:b].mul_(coef)
        return float(total)
    norms = torch._foreach_norm([t.grad for t in ts])
    total = float(torch.stack([n.float() for n in norms]).norm().item())
    if total > max_norm:
        torch._foreach_mul_([t.grad for t in ts], max_norm / (total + 1e-6))
    return total


def clip_grad_value(params: Sequence, max_val: float) -> float:
    """Clamp every gradient element to [-max_val, max_val]; returns the largest |g| seen before."""
    peak = 0.0
    for t in _tensors(params):
        if t.grad is None:
            continue
        peak = max(peak, float(t.grad.abs().max().item()))
        t.grad.clamp_(-max_val, max_val)
    return peak
