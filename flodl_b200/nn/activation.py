"""Activation modules (flodl/src/nn/activation.rs): 17 stateless (or one-parameter) layers."""
from __future__ import annotations

from enum import Enum

import torch
import torch.nn.functional as F

from .. import ops as _ops
from ..autograd import Variable
from .module import Module, Parameter

W = Variable.wrap


class GeluApprox(Enum):
    Exact = "none"
    Tanh = "tanh"


def _simple(cls_name, mod_name, fn):
    def forward(self, x):
        return W(fn(x.t))
    return type(cls_name, (Module,), {"name": lambda self: mod_name, "forward": forward,
                                      "new": classmethod(lambda cls: cls())})


Identity = _simple("Identity", "identity", lambda t: t)
ReLU = _simple("ReLU", "relu", torch.relu)
Sigmoid = _simple("Sigmoid", "sigmoid", torch.sigmoid)
Tanh = _simple("Tanh", "tanh", torch.tanh)
SiLU = _simple("SiLU", "silu", F.silu)
Mish = _simple("Mish", "mish", F.mish)
SELU = _simple("SELU", "selu", F.selu)
Hardswish = _simple("Hardswish", "hardswish", F.hardswish)
Hardsigmoid = _simple("Hardsigmoid", "hardsigmoid", F.hardsigmoid)


class GELU(Module):
    """erf form by default; `GELU.tanh()` / `GELU.with_approximate(GeluApprox.Tanh)` for the tanh form
    (flodl/src/nn/activation.rs:123-215)."""

    def __init__(self, approximate: GeluApprox = GeluApprox.Exact):
        self.approximate = approximate

    @classmethod
    def new(cls): return cls()
    @classmethod
    def tanh(cls): return cls(GeluApprox.Tanh)
    @classmethod
    def with_approximate(cls, approx): return cls(approx)
    def name(self): return "gelu"
    def forward(self, x): return W(_ops.gelu(x.t, self.approximate.value))


class LeakyReLU(Module):
    def __init__(self, negative_slope: float = 0.01): self.slope = negative_slope
    def name(self): return "leaky_relu"
    def forward(self, x): return W(F.leaky_relu(x.t, self.slope))


class ELU(Module):
    def __init__(self, alpha: float = 1.0): self.alpha = alpha
    def name(self): return "elu"
    def forward(self, x): return W(F.elu(x.t, self.alpha))


class Softplus(Module):
    def __init__(self, beta: float = 1.0, threshold: float = 20.0): self.beta, self.threshold = beta, threshold
    def name(self): return "softplus"
    def forward(self, x): return W(F.softplus(x.t, self.beta, self.threshold))


class Softmax(Module):
    def __init__(self, dim: int = -1): self.dim = dim
    def name(self): return "softmax"
    def forward(self, x): return W(torch.softmax(x.t, self.dim))


class LogSoftmax(Module):
    def __init__(self, dim: int = -1): self.dim = dim
    def name(self): return "log_softmax"
    def forward(self, x): return W(torch.log_softmax(x.t, self.dim))


class Flatten(Module):
    def __init__(self, start_dim: int = 1, end_dim: int = -1): self.s, self.e = start_dim, end_dim
    def name(self): return "flatten"
    def forward(self, x): return W(x.t.flatten(self.s, self.e))


class PReLU(Module):
    def __init__(self, num_parameters: int = 1, init: float = 0.25, device=None):
        from ..tensor import Device
        d = Device.of(device).torch if device is not None else None
        self.weight = Parameter(torch.full((num_parameters,), init, device=d), "weight")
    def name(self): return "prelu"
    def own_parameters(self): return [self.weight]
    def forward(self, x): return W(F.prelu(x.t, self.weight.t.to(x.t.dtype)))
