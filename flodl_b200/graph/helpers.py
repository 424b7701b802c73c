"""Ready-made routers, halting conditions and small utility modules for the graph builder
(flodl/src/graph/router.rs, halt.rs, state.rs, reshape.rs)."""
from __future__ import annotations

from typing import Dict, Sequence

import torch

from ..autograd import Variable
from ..nn.layers import Linear
from ..nn.module import Module


def _add_refs(x: Variable, refs: Dict[str, Variable]) -> Variable:
    for v in refs.values():
        x = x.add(v)
    return x


class SoftmaxRouter(Module):
    """Linear -> softmax over experts; refs are added to the input before routing."""
    def __init__(self, input_dim: int, num_experts: int, device=None): self.proj = Linear(input_dim, num_experts, True, device)
    @classmethod
    def on_device(cls, i, n, device): return cls(i, n, device)
    def name(self): return "softmax_router"
    def sub_modules(self): return [self.proj]
    def forward(self, x): return self.proj.forward(x).softmax(-1)
    def forward_named(self, x, refs): return self.forward(_add_refs(x, refs))


class SigmoidRouter(Module):
    def __init__(self, input_dim: int, num_experts: int, device=None): self.proj = Linear(input_dim, num_experts, True, device)
    @classmethod
    def on_device(cls, i, n, device): return cls(i, n, device)
    def name(self): return "sigmoid_router"
    def sub_modules(self): return [self.proj]
    def forward(self, x): return self.proj.forward(x).sigmoid()
    def forward_named(self, x, refs): return self.forward(_add_refs(x, refs))


class FixedSelector(Module):
    def __init__(self, index: int): self.index = float(index)
    def name(self): return "fixed_selector"
    def forward(self, x): return Variable(torch.tensor([self.index], device=x.t.device))


class ArgmaxSelector(Module):
    def __init__(self, input_dim: int, num_branches: int, device=None): self.proj = Linear(input_dim, num_branches, True, device)
    @classmethod
    def on_device(cls, i, n, device): return cls(i, n, device)
    def name(self): return "argmax_selector"
    def sub_modules(self): return [self.proj]
    def forward(self, x):
        logits = self.proj.forward(x).data().reshape(-1)
        return Variable(torch.tensor([float(int(logits.argmax().item()))], device=x.t.device))


class ThresholdHalt(Module):
    """Positive (= halt) when the largest element of the state exceeds the threshold."""
    def __init__(self, threshold: float): self.threshold = threshold
    def name(self): return "threshold_halt"
    def forward(self, x): return Variable((x.data().float().max() - self.threshold).reshape(1))


class LearnedHalt(Module):
    def __init__(self, input_dim: int, device=None): self.proj = Linear(input_dim, 1, True, device)
    @classmethod
    def on_device(cls, i, device): return cls(i, device)
    def name(self): return "learned_halt"
    def sub_modules(self): return [self.proj]
    def forward(self, x): return self.proj.forward(x)


class StateAdd(Module):
    """Identity that adds every ref to its input: the usual consumer of a forward reference."""
    def name(self): return "state_add"
    def forward(self, x): return x
    def forward_named(self, x, refs): return _add_refs(x, refs)


class Reshape(Module):
    def __init__(self, shape: Sequence[int]): self.shape = list(shape)
    def name(self): return "reshape"
    def forward(self, x): return x.reshape(self.shape)
