"""`Variable`: a shared handle on a tensor that records operations for backward.

Mirrors flodl/src/autograd/variable.rs:34-204 and the op surface of flodl/src/autograd/ops.rs.
The autograd graph is PyTorch's (as libtorch's is in the reference); a `Variable` holds the
`torch.Tensor` in `.t`, is cheap to copy (copies share the tensor, like `Rc<RefCell<Tensor>>`),
and exposes the reference's method names. Ops that have a native sm_100a kernel route through
`flodl_b200.ops`.
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch
import torch.nn.functional as F

from .. import ops as _ops
from ..tensor import Device, DType, TensorError


def _t(x):
    return x.t if isinstance(x, Variable) else x


class Variable:
    __slots__ = ("t", "__weakref__")

    def __init__(self, data, requires_grad: bool = False):
        if isinstance(data, Variable):
            data = data.t
        if not isinstance(data, torch.Tensor):
            data = torch.as_tensor(data)
        if requires_grad and not data.requires_grad:
            if not data.is_leaf:
                data = data.detach()
            data.requires_grad_(True)
        self.t = data

    # ---- construction ---------------------------------------------------------------------------
    @staticmethod
    def new(data: torch.Tensor, requires_grad: bool = False) -> "Variable":
        return Variable(data, requires_grad)

    @staticmethod
    def wrap(t: torch.Tensor) -> "Variable":
        v = Variable.__new__(Variable)
        v.t = t
        return v

    # ---- accessors ------------------------------------------------------------------------------
    def data(self) -> torch.Tensor:
        return self.t.detach()

    def grad(self) -> Optional[torch.Tensor]:
        return self.t.grad

    def set_grad(self, grad: torch.Tensor) -> None:
        self.t.grad = grad

    def requires_grad(self) -> bool:
        return self.t.requires_grad

    def set_requires_grad(self, flag: bool) -> None:
        if not self.t.is_leaf and not flag:
            raise TensorError("set_requires_grad(false) on a non-leaf variable; use detach()")
        self.t.requires_grad_(flag)

    def is_leaf(self) -> bool:
        return self.t.is_leaf

    def shape(self) -> List[int]:
        return list(self.t.shape)

    def dtype(self) -> DType:
        return DType.from_torch(self.t.dtype)

    def device(self) -> Device:
        return Device.of(self.t)

    def numel(self) -> int:
        return self.t.numel()

    def item(self) -> float:
        if self.t.numel() != 1:
            raise TensorError(f"item() needs a one-element tensor, got shape {list(self.t.shape)}")
        return float(self.t.item())

    def zero_grad(self) -> None:
        if self.t.grad is not None:
            self.t.grad.zero_()

    def zero_grad_set_to_none(self) -> None:
        self.t.grad = None

    def detach(self) -> "Variable":
        return Variable.wrap(self.t.detach())

    def detach_(self) -> None:
        self.t = self.t.detach()

    def to_device(self, device) -> "Variable":
        return Variable.wrap(self.t.to(Device.of(device).torch))

    def to_dtype(self, dtype) -> "Variable":
        return Variable.wrap(self.t.to(dtype.torch if isinstance(dtype, DType) else dtype))

    def set_data(self, data: torch.Tensor) -> None:
        """Replace the value, keep identity and `requires_grad` (checkpoint loads, device moves)."""
        rg = self.t.requires_grad
        with torch.no_grad():
            if self.t.shape == data.shape and self.t.dtype == data.dtype and self.t.device == data.device:
                self.t.copy_(data)
            else:
                self.t.data = data.detach()
        self.t.requires_grad_(rg)

    def autograd_node_count(self) -> int:
        """Number of autograd nodes reachable from this variable (ops_training.cpp:891-912)."""
        fn = self.t.grad_fn
        if fn is None:
            return 0
        seen, stack = set(), [fn]
        while stack:
            f = stack.pop()
            if f is None or f in seen:
                continue
            seen.add(f)
            stack.extend(n for n, _ in f.next_functions)
        return len(seen)

    def ensure_grad_accumulator(self):
        """Materialise the AccumulateGrad node now (the reference pins it to the training stream,
        ops_training.cpp:62-77); returns an opaque handle that keeps it alive."""
        if not self.t.requires_grad or not self.t.is_leaf:
            return None
        return self.t.view_as(self.t).grad_fn.next_functions[0][0]

    def backward(self) -> None:
        """Backpropagate from a scalar, then drop the graph (`tensor.backward()` + `detach_()`)."""
        if self.t.numel() != 1:
            raise TensorError("backward() needs a scalar loss")
        self.t.backward()
        self.t = self.t.detach()

    # ---- arithmetic -----------------------------------------------------------------------------
    def _bin(self, other, fn):
        return Variable.wrap(fn(self.t, _t(other)))

    def add(self, o): return self._bin(o, torch.add)
    def sub(self, o): return self._bin(o, torch.sub)
    def mul(self, o): return self._bin(o, torch.mul)
    def div(self, o): return self._bin(o, torch.div)
    def matmul(self, o): return self._bin(o, torch.matmul)
    def mul_scalar(self, s: float): return Variable.wrap(self.t * s)
    def div_scalar(self, s: float): return Variable.wrap(self.t / s)
    def add_scalar(self, s: float): return Variable.wrap(self.t + s)
    def neg(self): return Variable.wrap(-self.t)
    def atan2(self, o): return self._bin(o, torch.atan2)
    def maximum(self, o): return self._bin(o, torch.maximum)
    def minimum(self, o): return self._bin(o, torch.minimum)
    __add__ = add
    __sub__ = sub
    __mul__ = lambda self, o: self.mul(o) if isinstance(o, (Variable, torch.Tensor)) else self.mul_scalar(o)
    __truediv__ = lambda self, o: self.div(o) if isinstance(o, (Variable, torch.Tensor)) else self.div_scalar(o)
    __neg__ = neg
    __matmul__ = matmul
    __radd__ = lambda self, o: Variable.wrap(_t(o) + self.t)
    __rsub__ = lambda self, o: Variable.wrap(_t(o) - self.t)
    __rmul__ = lambda self, o: Variable.wrap(_t(o) * self.t)
    __rtruediv__ = lambda self, o: Variable.wrap(_t(o) / self.t)
    __pow__ = lambda self, e: Variable.wrap(self.t.pow(_t(e)))

    # ---- activations ----------------------------------------------------------------------------
    def relu(self): return Variable.wrap(torch.relu(self.t))
    def sigmoid(self): return Variable.wrap(torch.sigmoid(self.t))
    def tanh(self): return Variable.wrap(torch.tanh(self.t))
    def gelu(self): return Variable.wrap(_ops.gelu(self.t, "none"))
    def gelu_tanh(self): return Variable.wrap(_ops.gelu(self.t, "tanh"))
    def silu(self): return Variable.wrap(F.silu(self.t))
    def leaky_relu(self, slope: float = 0.01): return Variable.wrap(F.leaky_relu(self.t, slope))
    def elu(self, alpha: float = 1.0): return Variable.wrap(F.elu(self.t, alpha))
    def softplus(self, beta: float = 1.0, threshold: float = 20.0): return Variable.wrap(F.softplus(self.t, beta, threshold))
    def mish(self): return Variable.wrap(F.mish(self.t))
    def selu(self): return Variable.wrap(F.selu(self.t))
    def hardswish(self): return Variable.wrap(F.hardswish(self.t))
    def hardsigmoid(self): return Variable.wrap(F.hardsigmoid(self.t))
    def prelu(self, weight): return Variable.wrap(F.prelu(self.t, _t(weight)))

    # ---- reductions -----------------------------------------------------------------------------
    def sum(self): return Variable.wrap(self.t.sum())
    def mean(self): return Variable.wrap(self.t.mean())
    def sum_dim(self, dim: int, keepdim: bool = False): return Variable.wrap(self.t.sum(dim, keepdim))
    def mean_dim(self, dim: int, keepdim: bool = False): return Variable.wrap(self.t.mean(dim, keepdim))
    def prod(self): return Variable.wrap(self.t.prod())
    def prod_dim(self, dim: int, keepdim: bool = False): return Variable.wrap(self.t.prod(dim, keepdim))
    def cumsum(self, dim: int): return Variable.wrap(self.t.cumsum(dim))
    def logsumexp(self, dim: int, keepdim: bool = False): return Variable.wrap(torch.logsumexp(self.t, dim, keepdim))
    def min(self): return Variable.wrap(self.t.min())
    def max(self): return Variable.wrap(self.t.max())
    def min_dim(self, dim: int, keepdim: bool = False): return Variable.wrap(self.t.min(dim, keepdim).values)
    def max_dim(self, dim: int, keepdim: bool = False): return Variable.wrap(self.t.max(dim, keepdim).values)
    def var(self): return Variable.wrap(self.t.var())
    def std(self): return Variable.wrap(self.t.std())
    def var_dim(self, dim: int, keepdim: bool = False): return Variable.wrap(self.t.var(dim, keepdim=keepdim))
    def std_dim(self, dim: int, keepdim: bool = False): return Variable.wrap(self.t.std(dim, keepdim=keepdim))
    def softmax(self, dim: int): return Variable.wrap(torch.softmax(self.t, dim))
    def log_softmax(self, dim: int): return Variable.wrap(torch.log_softmax(self.t, dim))
    def argmax(self, dim: int, keepdim: bool = False): return Variable.wrap(self.t.argmax(dim, keepdim))

    # ---- elementwise math -----------------------------------------------------------------------
    def exp(self): return Variable.wrap(self.t.exp())
    def log(self): return Variable.wrap(self.t.log())
    def sqrt(self): return Variable.wrap(self.t.sqrt())
    def abs(self): return Variable.wrap(self.t.abs())
    def pow_scalar(self, e: float): return Variable.wrap(self.t.pow(e))
    def triu(self, diagonal: int = 0): return Variable.wrap(self.t.triu(diagonal))
    def tril(self, diagonal: int = 0): return Variable.wrap(self.t.tril(diagonal))
    def sin(self): return Variable.wrap(self.t.sin())
    def cos(self): return Variable.wrap(self.t.cos())
    def sign(self): return Variable.wrap(self.t.sign())
    def floor(self): return Variable.wrap(self.t.floor())
    def ceil(self): return Variable.wrap(self.t.ceil())
    def round(self): return Variable.wrap(self.t.round())
    def reciprocal(self): return Variable.wrap(self.t.reciprocal())
    def clamp(self, lo: float, hi: float): return Variable.wrap(self.t.clamp(lo, hi))
    def clamp_min(self, lo: float): return Variable.wrap(self.t.clamp_min(lo))
    def clamp_max(self, hi: float): return Variable.wrap(self.t.clamp_max(hi))
    def log1p(self): return Variable.wrap(self.t.log1p())
    def expm1(self): return Variable.wrap(self.t.expm1())
    def log2(self): return Variable.wrap(self.t.log2())
    def log10(self): return Variable.wrap(self.t.log10())
    def masked_fill(self, mask, value: float): return Variable.wrap(self.t.masked_fill(_t(mask).bool(), value))
    def normalize(self, p: float = 2.0, dim: int = -1, eps: float = 1e-12): return Variable.wrap(F.normalize(self.t, p, dim, eps))
    def cosine_similarity(self, other, dim: int = -1, eps: float = 1e-8): return Variable.wrap(F.cosine_similarity(self.t, _t(other), dim, eps))

    # ---- shape ----------------------------------------------------------------------------------
    def reshape(self, shape: Sequence[int]): return Variable.wrap(self.t.reshape(tuple(shape)))
    def transpose(self, d0: int, d1: int): return Variable.wrap(self.t.transpose(d0, d1))
    def permute(self, dims: Sequence[int]): return Variable.wrap(self.t.permute(tuple(dims)))
    def squeeze(self, dim: int): return Variable.wrap(self.t.squeeze(dim))
    def unsqueeze(self, dim: int): return Variable.wrap(self.t.unsqueeze(dim))

    def unsqueeze_many(self, dims: Sequence[int]):
        t = self.t
        for d in dims:
            t = t.unsqueeze(d)
        return Variable.wrap(t)

    def flatten(self, start: int = 0, end: int = -1): return Variable.wrap(self.t.flatten(start, end))
    def expand(self, shape: Sequence[int]): return Variable.wrap(self.t.expand(tuple(shape)))
    def narrow(self, dim: int, start: int, length: int): return Variable.wrap(self.t.narrow(dim, start, length))
    def select(self, dim: int, index: int): return Variable.wrap(self.t.select(dim, index))
    def index_select(self, dim: int, index): return Variable.wrap(self.t.index_select(dim, _t(index)))
    def gather(self, dim: int, index): return Variable.wrap(self.t.gather(dim, _t(index)))
    def cat(self, other, dim: int = 0): return Variable.wrap(torch.cat((self.t, _t(other)), dim))
    def chunk(self, chunks: int, dim: int = 0): return [Variable.wrap(c) for c in self.t.chunk(chunks, dim)]
    def repeat(self, repeats: Sequence[int]): return Variable.wrap(self.t.repeat(tuple(repeats)))
    def pad(self, padding: Sequence[int], value: float = 0.0): return Variable.wrap(F.pad(self.t, tuple(padding), value=value))
    def contiguous(self): return Variable.wrap(self.t.contiguous())

    def topk(self, k: int, dim: int = -1, largest: bool = True, sorted_: bool = True):
        r = self.t.topk(k, dim, largest, sorted_)
        return Variable.wrap(r.values), r.indices

    def sort(self, dim: int = -1, descending: bool = False):
        r = self.t.sort(dim, descending)
        return Variable.wrap(r.values), r.indices

    @staticmethod
    def cat_many(vs: Sequence["Variable"], dim: int = 0) -> "Variable":
        return Variable.wrap(torch.cat([_t(v) for v in vs], dim))

    @staticmethod
    def stack(vs: Sequence["Variable"], dim: int = 0) -> "Variable":
        return Variable.wrap(torch.stack([_t(v) for v in vs], dim))

    def __repr__(self) -> str:
        return f"Variable(shape={list(self.t.shape)}, dtype={self.t.dtype}, device={self.t.device}, requires_grad={self.t.requires_grad})"


# the comparison / query / math-extension ops of the reference's surface, by the reference's names
from .. import tensor_ops as _tensor_ops  # noqa: E402

_tensor_ops.install_variable_methods(Variable)
