"""`Module`, `Parameter`, `Buffer` and module-tree walking.

Same contract as the reference's `Module` trait (flodl/src/nn/mod.rs:123-235), `Parameter`
(flodl/src/nn/parameter.rs) and `Buffer` (flodl/src/nn/buffer.rs): a module maps one `Variable`
to one `Variable`; leaf modules list their own parameters/buffers, containers list
`sub_modules()` and inherit de-duplicated collection; optional capabilities
(`forward_named` for `.using()` refs, `step` for named loop traces, `as_graph`) are discovered
by the graph builder.
"""
from __future__ import annotations

from typing import Callable, Dict, List, Optional, Sequence

import torch

from ..autograd import Variable
from ..tensor import Device


class Parameter:
    """A named trainable `Variable` (flodl/src/nn/parameter.rs)."""

    __slots__ = ("variable", "name")

    def __init__(self, data, name: str):
        if isinstance(data, Variable):
            self.variable = data
            if not data.t.requires_grad and data.t.is_floating_point():
                data.t.requires_grad_(True)
        else:
            self.variable = Variable(data, requires_grad=True)
        self.name = name

    @classmethod
    def new(cls, data, name: str) -> "Parameter":
        return cls(data, name)

    @property
    def t(self) -> torch.Tensor:
        return self.variable.t

    def freeze(self) -> None:
        self.variable.t.requires_grad_(False)

    def unfreeze(self) -> None:
        self.variable.t.requires_grad_(True)

    def is_frozen(self) -> bool:
        return not self.variable.t.requires_grad

    def to_device(self, device) -> None:
        d = Device.of(device).torch
        if self.variable.t.device != d:
            rg = self.variable.t.requires_grad
            self.variable.t.data = self.variable.t.data.to(d)
            if self.variable.t.grad is not None:
                self.variable.t.grad = None
            self.variable.t.requires_grad_(rg)

    def shape(self) -> List[int]:
        return list(self.variable.t.shape)

    def numel(self) -> int:
        return self.variable.t.numel()

    def key(self) -> int:
        return id(self.variable.t)

    def __repr__(self) -> str:
        return f"Parameter({self.name}, shape={self.shape()})"


class Buffer:
    """A named non-trainable tensor with shared identity (running statistics, masks)."""

    __slots__ = ("_t", "name")

    def __init__(self, tensor: torch.Tensor, name: str):
        self._t = tensor.detach()
        self.name = name

    @classmethod
    def new(cls, tensor: torch.Tensor, name: str) -> "Buffer":
        return cls(tensor, name)

    def get(self) -> torch.Tensor:
        return self._t

    @property
    def t(self) -> torch.Tensor:
        return self._t

    def set(self, tensor: torch.Tensor) -> None:
        with torch.no_grad():
            if tensor.shape == self._t.shape and tensor.device == self._t.device and tensor.dtype == self._t.dtype:
                self._t.copy_(tensor)
            else:
                self._t.data = tensor.detach()

    def to_device(self, device) -> None:
        d = Device.of(device).torch
        if self._t.device != d:
            self._t.data = self._t.data.to(d)

    def shape(self) -> List[int]:
        return list(self._t.shape)

    def device(self) -> Device:
        return Device.of(self._t)

    def key(self) -> int:
        return id(self._t)


class Module:
    """Base class of every layer, activation, container and `Graph`."""

    training: bool = True

    # ---- the reference's constructor spellings: `X::new(args)` and `X::on_device(args, device)` ------
    @classmethod
    def new(cls, *args, **kw):
        return cls(*args, **kw)

    @classmethod
    def on_device(cls, *args, **kw):
        """Like `new`, with the device as the last argument (classes whose constructor takes `device=`)."""
        *rest, device = args
        return cls(*rest, device=device, **kw)

    # ---- to be provided by subclasses -----------------------------------------------------------
    def forward(self, input: Variable) -> Variable:  # pragma: no cover - abstract
        raise NotImplementedError

    def name(self) -> str:
        return "module"

    def sub_modules(self) -> List["Module"]:
        return []

    def own_parameters(self) -> List[Parameter]:
        """Parameters held directly by this module (leaf modules override)."""
        return []

    def own_buffers(self) -> List[Buffer]:
        return []

    def fuse_groups(self) -> List[List[Parameter]]:
        """Groups of parameters a flat-buffer engine should place back to back so one kernel can
        treat them as a single operand (e.g. the Q, K, V projection weights)."""
        return []

    # ---- collection -----------------------------------------------------------------------------
    def parameters(self) -> List[Parameter]:
        out, seen = [], set()
        for m in walk_modules(self):
            for p in m.own_parameters():
                if p.key() not in seen:
                    seen.add(p.key())
                    out.append(p)
        return out

    def buffers(self) -> List[Buffer]:
        out, seen = [], set()
        for m in walk_modules(self):
            for b in m.own_buffers():
                if b.key() not in seen:
                    seen.add(b.key())
                    out.append(b)
        return out

    # ---- state ----------------------------------------------------------------------------------
    def move_to_device(self, device) -> None:
        for p in self.parameters():
            p.to_device(device)
        for b in self.buffers():
            b.to_device(device)
        for m in walk_modules(self):
            m._on_device_change(device)

    def _on_device_change(self, device) -> None:
        pass

    def set_training(self, training: bool) -> None:
        for m in walk_modules(self):
            m.training = training

    def train(self) -> None:
        self.set_training(True)

    def eval(self) -> None:
        self.set_training(False)

    # ---- optional capabilities ------------------------------------------------------------------
    def trace(self) -> Optional[Variable]:
        """Per-iteration side output collected by loop nodes (legacy trace)."""
        return None

    def as_named_input(self):
        """Return self if the module implements `forward_named(input, refs)`."""
        return self if callable(getattr(self, "forward_named", None)) else None

    def as_loop_body(self):
        """Return self if the module implements `step(state, refs, emit)` for named loop traces."""
        return self if callable(getattr(self, "step", None)) else None

    def as_graph(self):
        return None

    def structural_hash(self) -> Optional[str]:
        return None

    def reset(self) -> None:
        """Clear per-forward state (called by loops before iterating)."""

    def detach_state(self) -> None:
        """Cut the autograd history of carried state (truncated BPTT)."""

    def __call__(self, x):
        return self.forward(x if isinstance(x, Variable) else Variable.wrap(x))


def walk_modules(root: Module) -> List[Module]:
    """Depth-first, de-duplicated list of `root` and everything reachable via `sub_modules()`
    (`walk_modules_visited`, flodl/src/nn/mod.rs)."""
    out, seen, stack = [], set(), [root]
    while stack:
        m = stack.pop()
        if id(m) in seen:
            continue
        seen.add(id(m))
        out.append(m)
        stack.extend(reversed(m.sub_modules()))
    return out


def walk_modules_visited(module: Module, visited: set, f) -> None:
    """Call `f` on `module` and everything below it, skipping what `visited` (a set the caller owns,
    of `id()`s) already holds: share one set over several roots to see a shared sub-module once
    (flodl/src/nn/mod.rs:408-420)."""
    if id(module) in visited:
        return
    visited.add(id(module))
    f(module)
    for child in module.sub_modules():
        walk_modules_visited(child, visited, f)


def collect_parameters(mods) -> list:
    """Parameters of several modules, concatenated without de-duplication (flodl/src/nn/mod.rs:422-436)."""
    out = []
    for m in mods:
        out.extend(m.parameters())
    return out


def modules(*mods: Module) -> List[Module]:
    """`modules![a, b, c]` (flodl/src/lib.rs:47-52)."""
    return list(mods)


class LoopBodyEmit:
    """Collector handed to `LoopBody.step`: `emit("name", value)` publishes a named trace."""

    def __init__(self):
        self.values: Dict[str, List[Variable]] = {}

    def __call__(self, name: str, value: Variable) -> None:
        self.values.setdefault(name, []).append(value)

    publish = __call__

    @classmethod
    def discard(cls) -> "LoopBodyEmit":
        """An emitter whose values nobody reads (what `forward_via_step` hands to `step`)."""
        return cls()


TraceEmit = LoopBodyEmit


class NamedInputModule(Module):
    """A module that takes extra named inputs wired by `FlowBuilder.using()`: implement
    `forward_named(input, refs)` with `refs` a dict from tag name to the tag's current value
    (flodl/src/nn/mod.rs:281-290). Any module with a `forward_named` method is accepted by the
    builder; this base states the contract and defaults `forward` to empty refs."""

    def forward_named(self, input: Variable, refs: Dict[str, Variable]) -> Variable:
        raise NotImplementedError

    def forward(self, x):
        return self.forward_named(x, {})


class LoopBody(Module):
    """A loop body with named per-iteration traces: implement `step(input, refs, emit)` and call
    `emit.publish(name, value)`; the loop collects them under `Graph.traces_named(name)`
    (flodl/src/nn/mod.rs:374-384). `forward` runs one step with a discarding emitter."""

    def step(self, input: Variable, refs: Dict[str, Variable], emit: LoopBodyEmit) -> Variable:
        raise NotImplementedError

    def as_loop_body(self):
        return self

    def forward(self, x):
        return forward_via_step(self, x)


def forward_via_step(body: Module, input: Variable) -> Variable:
    """Default `forward` for step-style loop bodies (flodl/src/nn/mod.rs:299-393)."""
    return body.step(input, {}, LoopBodyEmit())
