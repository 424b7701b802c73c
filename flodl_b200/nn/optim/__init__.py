"""Optimizers (flodl/src/nn/optim/*.rs): Adam, AdamW, SGD, RMSprop, Adagrad, RAdam, NAdam.

`Optimizer` contract: `step, zero_grad, lr, set_lr, set_group_lr, scale_lr`
(flodl/src/nn/optim/mod.rs:27-45); `Stateful`: `save_state/load_state` (+ files, gzip by
extension; mod.rs:55-93) with the reference's byte layout so optimizer checkpoints interchange.

Adam/AdamW and SGD run this library's fused kernels on CUDA: one launch over the whole flat
buffer when the parameters were re-homed by `flodl_b200.parallel.flat.FlatParams`, one launch
per tensor otherwise. Parameters whose gradient is None are skipped, as in the reference.
"""
from __future__ import annotations

import gzip
import io
import math
import struct
from typing import Tuple, List, Optional, Sequence

import torch

from ... import _ext
from ...parallel import flat as _flat
from ...tensor import TensorError
from ..module import Parameter


def _pt(p) -> torch.Tensor:
    return p.t if isinstance(p, Parameter) else p


class _Group:
    def __init__(self, lr: float, start: int, end: int):
        self.lr, self.start, self.end = lr, start, end


class Stateful:
    def save_state(self, w) -> None:  # pragma: no cover - interface
        raise NotImplementedError

    def load_state(self, r) -> None:  # pragma: no cover - interface
        raise NotImplementedError

    def save_state_file(self, path: str) -> None:
        opener = gzip.open if path.endswith(".gz") else open
        with opener(path, "wb") as f:
            self.save_state(f)

    def load_state_file(self, path: str) -> None:
        opener = gzip.open if path.endswith(".gz") else open
        with opener(path, "rb") as f:
            self.load_state(f)

    def state_bytes(self) -> bytes:
        b = io.BytesIO()
        self.save_state(b)
        return b.getvalue()


def write_tensor_state(w, t: Optional[torch.Tensor]) -> None:
    """u8 present + tensor record (same record as the .fdl entries; checkpoint.rs:323-350)."""
    w.write(_ext.require().pack_tensor_record(t))


def read_tensor_state(r, device) -> Optional[torch.Tensor]:
    present = r.read(1)
    if not present or present == b"\x00":
        return None
    ndim = struct.unpack("<I", r.read(4))[0]
    shape = struct.unpack(f"<{ndim}q", r.read(8 * ndim)) if ndim else ()
    tag = r.read(1)[0]
    nbytes = struct.unpack("<Q", r.read(8))[0]
    dt = {1: torch.float16, 2: torch.bfloat16, 3: torch.float32, 4: torch.float64, 5: torch.int32, 6: torch.int64}[tag]
    raw = bytearray(r.read(nbytes))
    t = torch.frombuffer(raw, dtype=dt).reshape(shape).clone() if nbytes else torch.empty(shape, dtype=dt)
    return t.to(device)


class Optimizer(Stateful):
    @classmethod
    def new(cls, *args, **kw):
        return cls(*args, **kw)

    def __init__(self, params: Sequence, lr: float):
        self.params: List[torch.Tensor] = [_pt(p) for p in params]
        self._lr = float(lr)
        self.groups: List[_Group] = []
        self.grad_scale: Optional[torch.Tensor] = None   # device scalar multiplied into every gradient
        self.skip_flag: int = 0    # device address of a word that, when non-zero, turns the fused update into a no-op
        self._hyper = None
        self._hyper_host = None

    # builder-style groups: Opt.with_groups(...).group(params, lr).group(...).build()
    def _add_group(self, params, lr):
        start = len(self.params)
        self.params.extend(_pt(p) for p in params)
        self.groups.append(_Group(float(lr), start, len(self.params)))

    def _group_ranges(self):
        if self.groups:
            return [(g.lr, g.start, g.end) for g in self.groups]
        return [(self._lr, 0, len(self.params))]

    def lr(self) -> float:
        return self._lr

    def set_lr(self, lr: float) -> None:
        self._lr = float(lr)
        for g in self.groups:
            g.lr = float(lr)

    def set_group_lr(self, group: int, lr: float) -> None:
        if self.groups:
            if 0 <= group < len(self.groups):
                self.groups[group].lr = float(lr)
        else:
            self.set_lr(lr)

    def scale_lr(self, factor: float) -> None:
        if self.groups:
            for g in self.groups:
                g.lr *= factor
        self._lr *= factor

    def zero_grad(self) -> None:
        flat = _flat.flat_of(self.params)
        if flat is not None:
            flat.zero_grad()
            return
        for p in self.params:
            p.grad = None

    def set_grad_scale(self, scale: Optional[torch.Tensor]) -> None:
        """Device-resident multiplier for all gradients (clip coefficient, 1/loss-scale)."""
        self.grad_scale = scale

    @property
    def fused(self) -> bool:
        """True when `step()` runs this library's fused kernels (which honour `set_skip_flag`)."""
        return False

    def set_skip_flag(self, address: int) -> None:
        """Device-visible int the fused kernels read first: non-zero means "leave the parameters
        alone" (the symmetric collectives raise their status word when a wait gave up, so
        un-reduced gradients are never applied). 0 removes the guard."""
        self.skip_flag = int(address)

    def _sync_shadow(self) -> None:
        """After an update that wrote the fp32 parameters without the fused kernels: bring the
        bf16 copies the GEMMs and convolutions read up to date."""
        flat = _flat.flat_of(self.params)
        if flat is not None:
            flat.refresh_shadow()
            return
        with torch.no_grad():
            for p in self.params:
                sh = getattr(p, "_fb_bf16", None)
                if sh is not None:
                    sh.copy_(p.data)

    # hyper-parameters travel through a pinned host buffer -> device tensor, so a captured CUDA
    # graph replays the optimizer kernel with fresh values and no host sync
    def _hyper_tensor(self, device, values: Sequence[float], slot: int = 0) -> torch.Tensor:
        if self._hyper is None or self._hyper.device != device:
            self._hyper = torch.zeros(64, 4, dtype=torch.float32, device=device)
        if not torch.cuda.is_current_stream_capturing() if device.type == "cuda" else True:
            # pageable source: the driver stages the 16 bytes before returning, so the next step
            # may overwrite them at once; inside a capture the owner of the graph refreshes the
            # device tensor before each replay instead
            self._hyper[slot].copy_(torch.tensor(list(values) + [0.0] * (4 - len(values)), dtype=torch.float32))
        return self._hyper[slot]

    def hyper_values(self):
        """(device tensor [64,4], list of per-group value lists) for graph owners that refresh
        hyper-parameters between replays."""
        return self._hyper

    def _save_groups(self, w):
        w.write(struct.pack("<I", len(self.groups)))
        for g in self.groups:
            w.write(struct.pack("<dqq", g.lr, g.start, g.end))

    def _load_groups(self, r):
        ng = struct.unpack("<I", r.read(4))[0]
        self.groups = []
        for _ in range(ng):
            lr, s, e = struct.unpack("<dqq", r.read(24))
            self.groups.append(_Group(lr, s, e))


def _native(p: torch.Tensor) -> bool:
    from ... import ops
    return p.is_cuda and ops.native_enabled() and p.dtype == torch.float32


class _GroupBuilder:
    """Fluent construction of an optimizer: hyper-parameters by name, then one `group(params, lr)` per
    learning-rate group (or the `(params, lr)` given to `Opt.builder`), then `build()`."""
    KNOBS = ()

    def __init__(self, cls, **kw):
        self.cls, self.kw, self.gs = cls, kw, []

    def group(self, params, lr):
        self.gs.append((list(params), lr))
        return self

    def _set(self, key, value):
        self.kw[key] = value
        return self

    def build(self):
        opt = self.cls([], self.gs[0][1] if self.gs else 1e-3, **self.kw)
        for ps, lr in self.gs:
            opt._add_group(ps, lr)
        opt._init_state()
        return opt


class AdamBuilder(_GroupBuilder):
    """`Adam.with_groups().betas(0.9, 0.98).eps(1e-6).group(ps, lr).build()` (adam.rs:58-100)."""
    def betas(self, beta1, beta2): return self._set("betas", (beta1, beta2))
    def eps(self, eps): return self._set("eps", eps)


class AdamWBuilder(AdamBuilder):
    """`AdamW.with_groups(weight_decay)`, same knobs as `AdamBuilder` (adam.rs:268-310)."""
    def weight_decay(self, wd): return self._set("weight_decay", wd)


class SGDBuilder(_GroupBuilder):
    """`SGD.with_groups(momentum).weight_decay(wd).group(ps, lr).build()` (sgd.rs:62-110)."""
    def momentum(self, m): return self._set("momentum", m)
    def weight_decay(self, wd): return self._set("weight_decay", wd)


class RMSpropBuilder(_GroupBuilder):
    """`RMSprop.builder(ps, lr).alpha(a).eps(e).weight_decay(wd).momentum(m).build()` (rmsprop.rs:100-125)."""
    def alpha(self, a): return self._set("alpha", a)
    def eps(self, eps): return self._set("eps", eps)
    def weight_decay(self, wd): return self._set("weight_decay", wd)
    def momentum(self, m): return self._set("momentum", m)


class AdagradBuilder(_GroupBuilder):
    """`Adagrad.builder(ps, lr).eps(e).weight_decay(wd).lr_decay(d).build()` (adagrad.rs:30-50)."""
    def eps(self, eps): return self._set("eps", eps)
    def weight_decay(self, wd): return self._set("weight_decay", wd)
    def lr_decay(self, d): return self._set("lr_decay", d)


# -------------------------------------------------------------------------------------------- Adam
class Adam(Optimizer):
    """Adam with libtorch `_fused_adamw_` semantics and weight_decay 0 (no L2 knob, as in the
    reference: adam.rs:124-126). State: fp32 m, v per parameter (lazy), one step counter."""

    def __init__(self, params, lr: float = 1e-3, betas=(0.9, 0.999), eps: float = 1e-8, weight_decay: float = 0.0):
        super().__init__(params, lr)
        self.beta1, self.beta2, self.eps, self.weight_decay = betas[0], betas[1], eps, weight_decay
        self.t = 0
        self._init_state()

    @classmethod
    def new(cls, params, lr): return cls(params, lr)
    @classmethod
    def with_groups(cls, **kw): return AdamBuilder(cls, **kw)

    def _init_state(self):
        self.m: List[Optional[torch.Tensor]] = [None] * len(self.params)
        self.v: List[Optional[torch.Tensor]] = [None] * len(self.params)
        self._flat_m = self._flat_v = None

    def _flat_state(self, flat):
        if self._flat_m is None or self._flat_m.numel() != flat.total:
            self._flat_m = torch.zeros(flat.total, dtype=torch.float32, device=flat.device)
            self._flat_v = torch.zeros(flat.total, dtype=torch.float32, device=flat.device)
            for i, p in enumerate(self.params):   # per-tensor views keep save/load working
                o, n = flat.range_of(p)
                self.m[i] = self._flat_m[o:o + n].view(p.shape)
                self.v[i] = self._flat_v[o:o + n].view(p.shape)
        return self._flat_m, self._flat_v

    def advance(self) -> None:
        """Host half of a step: bump the counter and upload {lr, 1-b1^t, 1-b2^t, wd} per group.
        A CUDA-graph owner calls this before each replay; `apply` is the capturable half."""
        self.t += 1
        self._cur = []
        bc1, bc2 = 1 - self.beta1 ** self.t, 1 - self.beta2 ** self.t
        for gi, (lr, s, e) in enumerate(self._group_ranges()):
            self._cur.append((lr, bc1, bc2))
            if e > s and _native(self.params[s]):
                self._hyper_tensor(self.params[s].device, [lr, bc1, bc2, self.weight_decay], gi)

    @property
    def fused(self) -> bool:
        return bool(self.params) and _native(self.params[0])

    def step(self) -> None:
        self.advance()
        self.apply()

    def apply(self, window: Optional[Tuple[int, int]] = None) -> None:
        """The capturable half of a step. `window = (lo, hi)` restricts a flat-buffer update to the
        elements [lo, hi) of the buffer (a trainer applies the part whose gradients have arrived
        while the rest is still being exchanged); it needs every group to sit in one flat range."""
        for gi, (_, s, e) in enumerate(self._group_ranges()):
            lr, bc1, bc2 = self._cur[gi]
            ps = self.params[s:e]
            if not ps:
                continue
            if _native(ps[0]):
                C = _ext.require()
                hyper = self._hyper[gi]
                rng = _flat.contiguous_range(ps)
                if window is not None and rng is None:
                    raise TensorError("apply(window=...) needs parameters in one flat range")
                if rng is not None:
                    flat, a, b = rng
                    if window is not None:
                        a, b = max(a, int(window[0])), min(b, int(window[1]))
                        if b <= a:
                            continue
                    m, v = self._flat_state(flat)
                    C.adam_step(flat.params[a:b], flat.grads[a:b], m[a:b], v[a:b],
                                None if flat.shadow is None else flat.shadow[a:b], hyper, self.beta1, self.beta2, self.eps, self.grad_scale,
                                self.skip_flag)
                    from ... import ops
                    ops.core._launched()
                    continue
                plist, glist, mlist, vlist, shlist = [], [], [], [], []
                for i in range(s, e):
                    p = self.params[i]
                    if p.grad is None:
                        continue
                    if self.m[i] is None:
                        self.m[i], self.v[i] = torch.zeros_like(p.data), torch.zeros_like(p.data)
                    if not p.data.is_contiguous():
                        raise TensorError("Adam: non-contiguous parameter")
                    sh = getattr(p, "_fb_bf16", None)
                    plist.append(p.data.view(-1))
                    glist.append(p.grad.contiguous().view(-1))
                    mlist.append(self.m[i].view(-1))
                    vlist.append(self.v[i].view(-1))
                    shlist.append(None if sh is None else sh.view(-1))
                if plist:
                    C.adam_step_multi(plist, glist, mlist, vlist, shlist, hyper, self.beta1, self.beta2, self.eps, self.grad_scale, self.skip_flag)
                continue
            with torch.no_grad():
                for i in range(s, e):
                    p = self.params[i]
                    if p.grad is None:
                        continue
                    g = p.grad.to(p.dtype)
                    if self.grad_scale is not None:
                        g = g * self.grad_scale.to(g.device, g.dtype)
                    if self.m[i] is None:
                        self.m[i], self.v[i] = torch.zeros_like(p.data), torch.zeros_like(p.data)
                    if self.weight_decay:
                        p.mul_(1 - lr * self.weight_decay)
                    self.m[i].mul_(self.beta1).add_(g, alpha=1 - self.beta1)
                    self.v[i].mul_(self.beta2).addcmul_(g, g, value=1 - self.beta2)
                    denom = (self.v[i] / bc2).sqrt_().add_(self.eps)
                    p.addcdiv_(self.m[i], denom, value=-(lr / bc1))
                    sh = getattr(p, "_fb_bf16", None)
                    if sh is not None:
                        sh.copy_(p.data)

    def save_state(self, w) -> None:
        w.write(struct.pack("<Idq", len(self.params), self._lr, self.t))
        for i in range(len(self.params)):
            write_tensor_state(w, self.m[i])
            write_tensor_state(w, self.v[i])
        self._save_groups(w)

    def load_state(self, r) -> None:
        n, lr, t = struct.unpack("<Idq", r.read(20))
        if n != len(self.params):
            raise TensorError(f"Adam: param count mismatch: checkpoint={n} optimizer={len(self.params)}")
        self._lr, self.t = lr, t
        for i, p in enumerate(self.params):
            m, v = read_tensor_state(r, p.device), read_tensor_state(r, p.device)
            if self.m[i] is not None and m is not None:
                self.m[i].copy_(m)
                self.v[i].copy_(v)
            else:
                self.m[i], self.v[i] = m, v
        self._load_groups(r)


class AdamW(Adam):
    """Adam with decoupled weight decay: `p *= 1 - lr*wd` before the update."""

    def __init__(self, params, lr: float = 1e-3, weight_decay: float = 0.01, betas=(0.9, 0.999), eps: float = 1e-8):
        super().__init__(params, lr, betas, eps, weight_decay)

    @classmethod
    def new(cls, params, lr, weight_decay): return cls(params, lr, weight_decay)
    @classmethod
    def with_groups(cls, weight_decay=0.01, **kw): return AdamWBuilder(cls, weight_decay=weight_decay, **kw)


# --------------------------------------------------------------------------------------------- SGD
class SGD(Optimizer):
    """g += wd*p; v = g on the first step else mu*v + g; p -= lr*v (no dampening / nesterov;
    flodl/src/nn/optim/sgd.rs:132-172)."""

    def __init__(self, params, lr: float, momentum: float = 0.0, weight_decay: float = 0.0):
        super().__init__(params, lr)
        self.momentum, self.weight_decay = momentum, weight_decay
        self._init_state()

    @classmethod
    def new(cls, params, lr, momentum=0.0): return cls(params, lr, momentum)
    @classmethod
    def with_groups(cls, momentum=0.0, **kw): return SGDBuilder(cls, momentum=momentum, **kw)
    def with_weight_decay(self, wd): self.weight_decay = wd; return self

    def _init_state(self):
        self.velocity: List[Optional[torch.Tensor]] = [None] * len(self.params)
        self._flat_v = None
        self._steps = 0

    def advance(self) -> None:
        first = self._steps == 0
        self._steps += 1
        self._cur = []
        for gi, (lr, s, e) in enumerate(self._group_ranges()):
            self._cur.append((lr, first))
            if e > s and _native(self.params[s]):
                self._hyper_tensor(self.params[s].device, [lr, self.momentum, self.weight_decay, 1.0 if first else 0.0], gi)

    @property
    def fused(self) -> bool:
        return bool(self.params) and _native(self.params[0])

    def step(self) -> None:
        self.advance()
        self.apply()

    def apply(self, window: Optional[Tuple[int, int]] = None) -> None:
        for gi, (_, s, e) in enumerate(self._group_ranges()):
            lr, first = self._cur[gi]
            ps = self.params[s:e]
            if not ps:
                continue
            if _native(ps[0]):
                C = _ext.require()
                rng = _flat.contiguous_range(ps)
                if window is not None and rng is None:
                    raise TensorError("apply(window=...) needs parameters in one flat range")
                if rng is not None:
                    flat, a, b = rng
                    if window is not None:
                        a, b = max(a, int(window[0])), min(b, int(window[1]))
                        if b <= a:
                            continue
                    if self.momentum and (self._flat_v is None or self._flat_v.numel() != flat.total):
                        self._flat_v = torch.zeros(flat.total, dtype=torch.float32, device=flat.device)
                        for i, p in enumerate(self.params):
                            o, n = flat.range_of(p)
                            self.velocity[i] = self._flat_v[o:o + n].view(p.shape)
                    C.sgd_step(flat.params[a:b], flat.grads[a:b], self._flat_v[a:b] if self.momentum else None,
                               None if flat.shadow is None else flat.shadow[a:b], self._hyper[gi], self.grad_scale, self.skip_flag)
                    from ... import ops
                    ops.core._launched()
                    continue
                for i in range(s, e):
                    p = self.params[i]
                    if p.grad is None:
                        continue
                    fresh = self.velocity[i] is None
                    if self.momentum and fresh:
                        self.velocity[i] = torch.zeros_like(p.data)
                    hyper = self._hyper_tensor(p.device, [lr, self.momentum, self.weight_decay, 1.0 if fresh else 0.0], 32 + (1 if fresh else 0))
                    sh = getattr(p, "_fb_bf16", None)
                    C.sgd_step(p.data.view(-1), p.grad.contiguous().view(-1), self.velocity[i].view(-1) if self.momentum else None,
                               None if sh is None else sh.view(-1), hyper, self.grad_scale, self.skip_flag)
                continue
            with torch.no_grad():
                for i in range(s, e):
                    p = self.params[i]
                    if p.grad is None:
                        continue
                    g = p.grad.to(p.dtype)
                    if self.grad_scale is not None:
                        g = g * self.grad_scale.to(g.device, g.dtype)
                    if self.weight_decay:
                        g = g + self.weight_decay * p
                    if self.momentum:
                        if self.velocity[i] is None:
                            self.velocity[i] = g.clone()
                        else:
                            self.velocity[i].mul_(self.momentum).add_(g)
                        g = self.velocity[i]
                    p.sub_(g, alpha=lr)
                    sh = getattr(p, "_fb_bf16", None)
                    if sh is not None:
                        sh.copy_(p.data)

    def save_state(self, w) -> None:
        w.write(struct.pack("<Idd", len(self.params), self._lr, self.weight_decay))
        for v in self.velocity:
            write_tensor_state(w, v)
        self._save_groups(w)

    def load_state(self, r) -> None:
        n, lr, wd = struct.unpack("<Idd", r.read(20))
        if n != len(self.params):
            raise TensorError(f"SGD: param count mismatch: checkpoint={n} optimizer={len(self.params)}")
        self._lr, self.weight_decay = lr, wd
        for i, p in enumerate(self.params):
            v = read_tensor_state(r, p.device)
            if self.velocity[i] is not None and v is not None:
                self.velocity[i].copy_(v)
            else:
                self.velocity[i] = v
            if v is not None:
                self._steps = max(self._steps, 1)
        self._load_groups(r)


# ----------------------------------------------------------------------------------------- RMSprop
class RMSprop(Optimizer):
    """alpha 0.99, eps 1e-8; first step v = (1-alpha) g^2; denom = sqrt(v)+eps; optional momentum
    buffer (flodl/src/nn/optim/rmsprop.rs:137-190)."""

    def __init__(self, params, lr: float = 1e-2, alpha: float = 0.99, eps: float = 1e-8, weight_decay: float = 0.0, momentum: float = 0.0):
        super().__init__(params, lr)
        self.alpha, self.eps, self.weight_decay, self.momentum = alpha, eps, weight_decay, momentum
        self._init_state()

    @classmethod
    def with_groups(cls, **kw): return RMSpropBuilder(cls, **kw)
    @classmethod
    def builder(cls, params, lr): return RMSpropBuilder(cls).group(params, lr)

    def _init_state(self):
        self.sq = [None] * len(self.params)
        self.buf = [None] * len(self.params)

    def step(self) -> None:
        with torch.no_grad():
            for lr, s, e in self._group_ranges():
                for i in range(s, e):
                    p = self.params[i]
                    if p.grad is None:
                        continue
                    g = p.grad.to(p.dtype)
                    if self.weight_decay:
                        g = g + self.weight_decay * p
                    if self.sq[i] is None:
                        self.sq[i] = (1 - self.alpha) * g * g
                    else:
                        self.sq[i].mul_(self.alpha).addcmul_(g, g, value=1 - self.alpha)
                    denom = self.sq[i].sqrt().add_(self.eps)
                    if self.momentum > 0:
                        if self.buf[i] is None:
                            self.buf[i] = g / denom
                        else:
                            self.buf[i].mul_(self.momentum).addcdiv_(g, denom)
                        p.sub_(self.buf[i], alpha=lr)
                    else:
                        p.addcdiv_(g, denom, value=-lr)
        self._sync_shadow()

    def save_state(self, w) -> None:
        w.write(struct.pack("<Id", len(self.params), self._lr))
        for a, b in zip(self.sq, self.buf):
            write_tensor_state(w, a)
            write_tensor_state(w, b)
        self._save_groups(w)

    def load_state(self, r) -> None:
        n, lr = struct.unpack("<Id", r.read(12))
        if n != len(self.params):
            raise TensorError(f"RMSprop: param count mismatch: checkpoint={n} optimizer={len(self.params)}")
        self._lr = lr
        for i, p in enumerate(self.params):
            self.sq[i], self.buf[i] = read_tensor_state(r, p.device), read_tensor_state(r, p.device)
        self._load_groups(r)




# ----------------------------------------------------------------------------------------- Adagrad
class Adagrad(Optimizer):
    """clr = lr / (1 + (t-1) lr_decay); ss += g^2; p -= clr g / (sqrt(ss)+eps)
    (flodl/src/nn/optim/adagrad.rs:84-106)."""

    def __init__(self, params, lr: float = 1e-2, lr_decay: float = 0.0, eps: float = 1e-10, weight_decay: float = 0.0):
        super().__init__(params, lr)
        self.lr_decay, self.eps, self.weight_decay = lr_decay, eps, weight_decay
        self.t = 0
        self._init_state()

    @classmethod
    def with_groups(cls, **kw): return AdagradBuilder(cls, **kw)
    @classmethod
    def builder(cls, params, lr): return AdagradBuilder(cls).group(params, lr)

    def _init_state(self):
        self.ss = [None] * len(self.params)

    def step(self) -> None:
        self.t += 1
        with torch.no_grad():
            for lr, s, e in self._group_ranges():
                clr = lr / (1 + (self.t - 1) * self.lr_decay)
                for i in range(s, e):
                    p = self.params[i]
                    if p.grad is None:
                        continue
                    g = p.grad.to(p.dtype)
                    if self.weight_decay:
                        g = g + self.weight_decay * p
                    if self.ss[i] is None:
                        self.ss[i] = torch.zeros_like(p.data)
                    self.ss[i].addcmul_(g, g)
                    p.addcdiv_(g, self.ss[i].sqrt().add_(self.eps), value=-clr)
        self._sync_shadow()

    def save_state(self, w) -> None:
        w.write(struct.pack("<Idq", len(self.params), self._lr, self.t))
        for a in self.ss:
            write_tensor_state(w, a)
        self._save_groups(w)

    def load_state(self, r) -> None:
        n, lr, t = struct.unpack("<Idq", r.read(20))
        if n != len(self.params):
            raise TensorError(f"Adagrad: param count mismatch: checkpoint={n} optimizer={len(self.params)}")
        self._lr, self.t = lr, t
        for i, p in enumerate(self.params):
            self.ss[i] = read_tensor_state(r, p.device)
        self._load_groups(r)




# ------------------------------------------------------------------------------------ RAdam / NAdam
class _AdamLike(Optimizer):
    def __init__(self, params, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0):
        super().__init__(params, lr)
        self.beta1, self.beta2, self.eps, self.weight_decay = betas[0], betas[1], eps, weight_decay
        self.t = 0
        self._init_state()

    def _init_state(self):
        self.m = [None] * len(self.params)
        self.v = [None] * len(self.params)

    def _moments(self, i, p):
        g = p.grad.to(p.dtype)
        if self.weight_decay:
            g = g + self.weight_decay * p
        if self.m[i] is None:
            self.m[i], self.v[i] = torch.zeros_like(p.data), torch.zeros_like(p.data)
        self.m[i].mul_(self.beta1).add_(g, alpha=1 - self.beta1)
        self.v[i].mul_(self.beta2).addcmul_(g, g, value=1 - self.beta2)
        return g

    def save_state(self, w) -> None:
        w.write(struct.pack("<Idq", len(self.params), self._lr, self.t))
        for a, b in zip(self.m, self.v):
            write_tensor_state(w, a)
            write_tensor_state(w, b)
        self._save_groups(w)

    def load_state(self, r) -> None:
        n, lr, t = struct.unpack("<Idq", r.read(20))
        if n != len(self.params):
            raise TensorError(f"{type(self).__name__}: param count mismatch: checkpoint={n} optimizer={len(self.params)}")
        self._lr, self.t = lr, t
        for i, p in enumerate(self.params):
            self.m[i], self.v[i] = read_tensor_state(r, p.device), read_tensor_state(r, p.device)
        self._load_groups(r)


class RAdam(_AdamLike):
    """Rectified Adam: rho_inf = 2/(1-b2) - 1; rectified step when rho_t > 5, else p -= lr * m_hat
    (flodl/src/nn/optim/radam.rs:45-96)."""

    def step(self) -> None:
        self.t += 1
        t = self.t
        rho_inf = 2.0 / (1.0 - self.beta2) - 1.0
        b2t = self.beta2 ** t
        rho_t = rho_inf - 2.0 * t * b2t / (1.0 - b2t)
        bc1 = 1 - self.beta1 ** t
        with torch.no_grad():
            for lr, s, e in self._group_ranges():
                for i in range(s, e):
                    p = self.params[i]
                    if p.grad is None:
                        continue
                    self._moments(i, p)
                    m_hat = self.m[i] / bc1
                    if rho_t > 5.0:
                        r = math.sqrt(((rho_t - 4) * (rho_t - 2) * rho_inf) / ((rho_inf - 4) * (rho_inf - 2) * rho_t))
                        v_hat = (self.v[i] / (1 - b2t)).sqrt_().add_(self.eps)
                        p.addcdiv_(m_hat, v_hat, value=-lr * r)
                    else:
                        p.sub_(m_hat, alpha=lr)
        self._sync_shadow()

class NAdam(_AdamLike):
    """m_hat = b1*m/(1-b1^(t+1)) + (1-b1) g/(1-b1^t); no momentum-decay schedule
    (flodl/src/nn/optim/nadam.rs:50-91)."""

    def step(self) -> None:
        self.t += 1
        t = self.t
        bc1, bc1n, bc2 = 1 - self.beta1 ** t, 1 - self.beta1 ** (t + 1), 1 - self.beta2 ** t
        with torch.no_grad():
            for lr, s, e in self._group_ranges():
                for i in range(s, e):
                    p = self.params[i]
                    if p.grad is None:
                        continue
                    g = self._moments(i, p)
                    m_hat = self.m[i] * (self.beta1 / bc1n) + g * ((1 - self.beta1) / bc1)
                    p.addcdiv_(m_hat, (self.v[i] / bc2).sqrt_().add_(self.eps), value=-lr)
        self._sync_shadow()
