"""Flat parameter / gradient storage.

All parameters of a model live in ONE fp32 buffer, their gradients in ONE fp32 buffer with the
same layout, and (for the tensor cores) a bf16 shadow of the parameters in a third. That turns
what the reference does per tensor into single launches over a range:

* gradient all-reduce per ~25 MB bucket instead of one NCCL call per parameter
  (flodl/src/distributed/ddp.rs:133-147),
* one fused optimizer kernel per step (flodl/src/nn/optim/adam.rs:152-198,
  flodl/src/nn/optim/sgd.rs:132-172),
* one global-norm reduction (flodl-sys/ops_training.cpp:769-800),
* one broadcast for the initial parameter sync (ddp.rs:160-167).

The gradient buffer can be placed in peer-mapped ("symmetric") memory so the collectives in
`csrc/comm` can read it from other GPUs directly.
"""
from __future__ import annotations

from typing import Callable, Dict, List, Optional, Sequence

import torch

ALIGN = 64  # elements; keeps every slot 256-byte aligned in fp32 and 128-byte aligned in bf16


def _align(n: int) -> int:
    return (n + ALIGN - 1) // ALIGN * ALIGN


def _slot_view(buf: torch.Tensor, offset: int, like: torch.Tensor) -> torch.Tensor:
    """View of `buf[offset : offset + numel]` shaped like `like`. 4-D tensors flagged
    `_fb_channels_last` (2-D convolution filters) are stored K-R-S-C, i.e. the view has channels-last
    strides: the tensor-core convolutions then take the bf16 shadow as it is, and the filter
    gradient they produce adds into the slot without a layout change. Element-wise consumers (the
    optimizer, norms, collectives) work on the flat range and never see the difference."""
    n = like.numel()
    flat = buf[offset:offset + n]
    if like.dim() == 4 and getattr(like, "_fb_channels_last", False):
        co, ci, kh, kw = like.shape
        return flat.view(co, kh, kw, ci).permute(0, 3, 1, 2)
    return flat.view(like.shape)


class FlatParams:
    """Re-homes `tensors` (leaf parameter tensors) into flat buffers.

    After construction each tensor `p`:
      * `p.data` is a view into `self.params` (fp32),
      * `p.grad` is a view into `self.grads` (fp32, same offsets) that is never replaced,
      * `p._fb_grad` is that same view (ops write / accumulate gradients into it directly),
      * `p._fb_bf16` is a view into `self.shadow` (bf16 copy of the value), if `shadow=True`,
      * `p._fb_flat = (self, offset, numel)`.
    """

    def __init__(self, tensors: Sequence[torch.Tensor], shadow: bool = True, grad_alloc: Optional[Callable[[int], torch.Tensor]] = None,
                 param_alloc: Optional[Callable[[int], torch.Tensor]] = None, groups: Optional[Sequence[Sequence[torch.Tensor]]] = None):
        # `groups`: lists of tensors that must sit back to back (e.g. the Q, K, V weights of an
        # attention block, so one GEMM can address them as a single operand)
        follow = {}
        for g in groups or ():
            g = list(g)
            for t in g[1:]:
                follow[id(t)] = True
            follow[("head", id(g[0]))] = g
        uniq, seen = [], set()
        for t in tensors:
            if id(t) in seen or follow.get(id(t)):
                continue
            chain = follow.get(("head", id(t)), [t])
            for c in chain:
                if id(c) not in seen:
                    seen.add(id(c))
                    uniq.append(c)
        for t in tensors:   # grouped tensors whose head was not in `tensors`
            if id(t) not in seen:
                seen.add(id(t))
                uniq.append(t)
        if not uniq:
            raise ValueError("FlatParams needs at least one parameter")
        dev = uniq[0].device
        self.tensors: List[torch.Tensor] = uniq
        self.offsets: List[int] = []
        off = 0
        for t in uniq:
            if t.device != dev:
                raise ValueError("all parameters must live on one device")
            self.offsets.append(off)
            off += _align(t.numel())
        self.total = off
        self.device = dev
        self.params = param_alloc(off) if param_alloc else torch.zeros(off, dtype=torch.float32, device=dev)
        self.grads = grad_alloc(off) if grad_alloc else torch.zeros(off, dtype=torch.float32, device=dev)
        self.shadow = torch.zeros(off, dtype=torch.bfloat16, device=dev) if shadow and dev.type == "cuda" else None
        with torch.no_grad():
            for t, o in zip(uniq, self.offsets):
                n = t.numel()
                view = _slot_view(self.params, o, t)
                view.copy_(t.detach().float())
                rg = t.requires_grad
                t.data = view
                t.requires_grad_(rg)
                g = _slot_view(self.grads, o, t)
                t.grad = g
                t._fb_grad = g
                t._fb_flat = (self, o, n)
                if self.shadow is not None:
                    t._fb_bf16 = _slot_view(self.shadow, o, t)
        self.refresh_shadow()

    # ---- maintenance --------------------------------------------------------------------------
    def refresh_shadow(self) -> None:
        if self.shadow is not None:
            self.shadow.copy_(self.params)

    def zero_grad(self) -> None:
        self.grads.zero_()

    def restore_grad_views(self) -> None:
        """Re-attach `.grad` after something set it to None (e.g. a foreign `zero_grad(set_to_none)`)."""
        for t, o in zip(self.tensors, self.offsets):
            if t.grad is None or t.grad.data_ptr() != self.grads.data_ptr() + 4 * o:
                t.grad = _slot_view(self.grads, o, t)

    def range_of(self, t: torch.Tensor):
        _, o, n = t._fb_flat
        return o, n

    # ---- buckets --------------------------------------------------------------------------------
    def buckets(self, bucket_bytes: int = 25 * 1024 * 1024) -> List[Dict]:
        """Contiguous ranges of about `bucket_bytes` of gradient, cut at parameter boundaries,
        listed from the END of the buffer (the last layers' gradients are produced first)."""
        elems = max(1, bucket_bytes // 4)
        out, hi = [], self.total
        members: List[int] = []
        for i in range(len(self.tensors) - 1, -1, -1):
            members.append(i)
            lo = self.offsets[i]
            if hi - lo >= elems or i == 0:
                out.append({"start": lo, "end": hi, "members": list(members)})
                hi, members = lo, []
        return out


def flat_of(tensors: Sequence[torch.Tensor]) -> Optional[FlatParams]:
    """The FlatParams that holds ALL of `tensors`, or None."""
    owner = None
    for t in tensors:
        f = getattr(t, "_fb_flat", None)
        if f is None:
            return None
        if owner is None:
            owner = f[0]
        elif owner is not f[0]:
            return None
    return owner


def contiguous_range(tensors: Sequence[torch.Tensor]):
    """(flat, start, end) if `tensors` cover one gap-free range of a FlatParams (up to alignment padding)."""
    flat = flat_of(tensors)
    if flat is None:
        return None
    spans = sorted((t._fb_flat[1], t._fb_flat[1] + _align(t._fb_flat[2])) for t in {id(t): t for t in tensors}.values())
    for (a0, a1), (b0, b1) in zip(spans, spans[1:]):
        if a1 != b0:
            return None
    return flat, spans[0][0], spans[-1][1]
