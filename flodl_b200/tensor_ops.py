"""The reference's tensor-op surface by its own names, over `torch.Tensor`.

The reference wraps libtorch tensors in an owned `Tensor` with about three hundred chainable
methods, each a call through its C shim (flodl-sys/shim.h, implemented in `ops_tensor.cpp`,
`ops_math_ext.cpp`, `ops_nn.cpp`). Here the tensor type is `torch.Tensor` itself; this module
gives the operations whose reference name or convention differs from PyTorch's (float 0/1 masks
from comparisons, `*_scalar` / `*_tensor` pairs, `sum_dims`, `norm_p_dim`, `cat2`, ...) and the
math-extension set (`median`, `searchsorted`, `nonzero`, `cumprod`, `multinomial`, `isclose`,
`addmm`, `scatter_add`, `movedim`, `flip`, `argsort`, `randperm`, `one_hot`, `meshgrid`, `cdist`,
...), as plain functions. `Variable` exposes every differentiable one as a method (installed by
`install_variable_methods`), so `v.median_dim(1)` or `v.scatter_add(0, idx, src)` read as in the
reference.

Conventions kept from the shim: comparison and predicate ops return masks in the input's floating
dtype (fp32 for integer inputs) with 0.0 / 1.0 entries; `any` / `all` return a 0-dim mask; index
results are int64; ops returning several tensors return tuples.
"""
from __future__ import annotations

from typing import Callable, Dict, List, Optional, Sequence, Tuple

import torch
import torch.nn.functional as F

from .tensor import TensorError

T = torch.Tensor


def _mask(b: T, like: T) -> T:
    return b.to(like.dtype if like.is_floating_point() else torch.float32)


def _bool(m: T) -> T:
    return m if m.dtype == torch.bool else m != 0


# ---- comparisons / predicates (float masks; ops_tensor.cpp "Comparison", "Boolean / detection") ----
def gt_scalar(t: T, s: float) -> T: return _mask(t > s, t)
def ge_scalar(t: T, s: float) -> T: return _mask(t >= s, t)
def le_scalar(t: T, s: float) -> T: return _mask(t <= s, t)
def lt_scalar(t: T, s: float) -> T: return _mask(t < s, t)
def eq_scalar(t: T, s: float) -> T: return _mask(t == s, t)
def ne_scalar(t: T, s: float) -> T: return _mask(t != s, t)
def gt_tensor(a: T, b: T) -> T: return _mask(a > b, a)
def lt_tensor(a: T, b: T) -> T: return _mask(a < b, a)
def ge_tensor(a: T, b: T) -> T: return _mask(a >= b, a)
def le_tensor(a: T, b: T) -> T: return _mask(a <= b, a)
def eq_tensor(a: T, b: T) -> T: return _mask(a == b, a)
def ne_tensor(a: T, b: T) -> T: return _mask(a != b, a)
def isnan(t: T) -> T: return _mask(torch.isnan(t), t)
def isinf(t: T) -> T: return _mask(torch.isinf(t), t)
def logical_and(a: T, b: T) -> T: return _mask(_bool(a) & _bool(b), a)
def logical_or(a: T, b: T) -> T: return _mask(_bool(a) | _bool(b), a)
def logical_not(t: T) -> T: return _mask(~_bool(t), t)
def any(t: T) -> T: return _mask(_bool(t).any(), t)        # noqa: A001  (the reference's name)
def all(t: T) -> T: return _mask(_bool(t).all(), t)        # noqa: A001
def isclose(a: T, b: T, rtol: float = 1e-5, atol: float = 1e-8) -> T: return _mask(torch.isclose(a, b, rtol, atol), a)
def all_finite(t: T) -> bool: return bool(torch.isfinite(t).all().item())


# ---- reductions and queries (ops_math_ext.cpp) --------------------------------------------------------
def norm(t: T) -> T: return t.norm()
def norm_p_dim(t: T, p: float, dim: int, keepdim: bool = False) -> T: return t.norm(p, dim, keepdim)
def sum_dims(t: T, dims: Sequence[int], keepdim: bool = False) -> T: return t.sum(tuple(int(d) for d in dims), keepdim)
def cumprod(t: T, dim: int) -> T: return t.cumprod(dim)
def median(t: T) -> T: return t.median()
def median_dim(t: T, dim: int, keepdim: bool = False) -> Tuple[T, T]:
    r = t.median(dim, keepdim)
    return r.values, r.indices
def count_nonzero(t: T) -> T: return torch.count_nonzero(t)
def count_nonzero_dim(t: T, dim: int) -> T: return torch.count_nonzero(t, dim)
def argmin(t: T, dim: int, keepdim: bool = False) -> T: return t.argmin(dim, keepdim)
def nonzero(t: T) -> T: return torch.nonzero(t)
def unique(t: T, sorted_: bool = True, return_inverse: bool = False) -> Tuple[T, Optional[T]]:
    if return_inverse:
        out, inv = torch.unique(t, sorted=sorted_, return_inverse=True)
        return out, inv
    return torch.unique(t, sorted=sorted_), None
def searchsorted(sorted_seq: T, values: T) -> T: return torch.searchsorted(sorted_seq, values)


# ---- element-wise math ------------------------------------------------------------------------------
def tan(t): return t.tan()
def asin(t): return t.asin()
def acos(t): return t.acos()
def atan(t): return t.atan()
def erf(t): return t.erf()
def erfc(t): return t.erfc()
def trunc(t): return t.trunc()
def frac(t): return t.frac()
def fmod_scalar(t, s: float): return t.fmod(s)
def fmod_tensor(a, b): return a.fmod(b)
def remainder_scalar(t, s: float): return t.remainder(s)
def remainder_tensor(a, b): return a.remainder(b)
def lerp(a, b, weight: float): return torch.lerp(a, b, float(weight))
def lerp_tensor(a, b, weight: T): return torch.lerp(a, b, weight)
def addmm(bias, mat1, mat2, beta: float = 1.0, alpha: float = 1.0): return torch.addmm(bias, mat1, mat2, beta=beta, alpha=alpha)
def addcmul(t, t1, t2, value: float = 1.0): return torch.addcmul(t, t1, t2, value=value)
def addcdiv(t, t1, t2, value: float = 1.0): return torch.addcdiv(t, t1, t2, value=value)
def where(condition, x, y): return torch.where(_bool(condition), x, y)


# ---- indexing / scatter -----------------------------------------------------------------------------
def scatter(t, dim: int, index, src): return t.scatter(dim, index, src)
def scatter_add(t, dim: int, index, src): return t.scatter_add(dim, index, src)
def index_add(t, dim: int, index, src): return t.index_add(dim, index, src)
def select_scatter(t, src, dim: int, index: int): return torch.select_scatter(t, src, dim, index)
def narrow_scatter(t, src, dim: int, start: int): return torch.slice_scatter(t, src, dim, start, start + src.shape[dim])
def argsort(t, dim: int = -1, descending: bool = False): return t.argsort(dim, descending)


# ---- shape --------------------------------------------------------------------------------------------
def diagonal(t, offset: int = 0, dim1: int = 0, dim2: int = 1): return t.diagonal(offset, dim1, dim2)
def movedim(t, src: int, dst: int): return t.movedim(src, dst)
def tile(t, reps: Sequence[int]): return t.tile(tuple(reps))
def flip(t, dims: Sequence[int]): return t.flip(tuple(dims))
def roll(t, shift: int, dim: int): return t.roll(shift, dim)
def split(t, split_size: int, dim: int = 0) -> List[T]: return list(t.split(split_size, dim))
def unbind(t, dim: int = 0) -> List[T]: return list(t.unbind(dim))
def cat2(a, b, dim: int = 0): return torch.cat((a, b), dim)
def meshgrid(tensors: Sequence[T]) -> List[T]: return list(torch.meshgrid(*tensors, indexing="ij"))
_PAD_MODES = {0: "constant", 1: "reflect", 2: "replicate", 3: "circular"}
def pad_mode(t, padding: Sequence[int], mode: int = 0, value: float = 0.0):
    if mode not in _PAD_MODES:
        raise TensorError(f"pad_mode: unknown mode {mode} (0 constant, 1 reflect, 2 replicate, 3 circular)")
    return F.pad(t, list(padding), _PAD_MODES[mode], value if mode == 0 else None) if mode == 0 else F.pad(t, list(padding), _PAD_MODES[mode])
_INTERP = {0: "nearest", 1: "bilinear", 2: "bicubic", 3: "trilinear"}
def interpolate(t, output_size: Sequence[int], mode: int = 0, align_corners: bool = False):
    if mode not in _INTERP:
        raise TensorError(f"interpolate: unknown mode {mode}")
    return F.interpolate(t, size=list(output_size), mode=_INTERP[mode], align_corners=None if mode == 0 else bool(align_corners))


# ---- distances / creation / sampling ---------------------------------------------------------------------
def cdist(x, y, p: float = 2.0): return torch.cdist(x, y, p)
def one_hot(t, num_classes: int): return F.one_hot(t.long(), num_classes).to(torch.float32)
def bernoulli(t): return torch.bernoulli(t)
def multinomial(probs, num_samples: int, replacement: bool = False): return torch.multinomial(probs, num_samples, replacement)
def randperm(n: int, dtype=torch.int64, device=None): return torch.randperm(n, dtype=dtype, device=device)
def eye(n: int, dtype=torch.float32, device=None): return torch.eye(n, dtype=dtype, device=device)
def linspace(start: float, end: float, steps: int, dtype=torch.float32, device=None): return torch.linspace(start, end, steps, dtype=dtype, device=device)
def randint(low: int, high: int, shape: Sequence[int], dtype=torch.int64, device=None): return torch.randint(low, high, tuple(shape), dtype=dtype, device=device)
def zeros_like(t): return torch.zeros_like(t)
def ones_like(t): return torch.ones_like(t)
def full_like(t, value: float): return torch.full_like(t, value)
def rand_like(t): return torch.rand_like(t)
def randn_like(t): return torch.randn_like(t)


# ---- multi-tensor ("foreach") helpers used by the optimizers and Local SGD (ops_training.cpp) ---------
def foreach_add_scalar_(ts: Sequence[T], s: float) -> None: torch._foreach_add_(list(ts), s)
def foreach_mul_scalar_(ts: Sequence[T], s: float) -> None: torch._foreach_mul_(list(ts), s)
def foreach_zero_(ts: Sequence[T]) -> None: torch._foreach_zero_(list(ts))
def foreach_add_list_(a: Sequence[T], b: Sequence[T], alpha: float = 1.0) -> None: torch._foreach_add_(list(a), list(b), alpha=alpha)
def foreach_norm(ts: Sequence[T], ord: float = 2.0) -> List[T]: return list(torch._foreach_norm(list(ts), ord))   # noqa: A002
def foreach_lerp_scalar_(a: Sequence[T], b: Sequence[T], weight: float) -> None: torch._foreach_lerp_(list(a), list(b), weight)
def foreach_sqrt_(ts: Sequence[T]) -> None: torch._foreach_sqrt_(list(ts))


# Differentiable (or index-producing) ops that `Variable` gains as methods. The first argument is the
# receiver; other Variable arguments are unwrapped; tensor results are wrapped again.
VARIABLE_METHODS: Tuple[str, ...] = (
    "gt_scalar", "ge_scalar", "le_scalar", "lt_scalar", "eq_scalar", "ne_scalar", "gt_tensor", "lt_tensor", "ge_tensor", "le_tensor",
    "eq_tensor", "ne_tensor", "isnan", "isinf", "logical_and", "logical_or", "logical_not", "any", "all", "isclose",
    "norm", "norm_p_dim", "sum_dims", "cumprod", "median", "median_dim", "count_nonzero", "count_nonzero_dim", "argmin", "nonzero",
    "unique", "searchsorted", "tan", "asin", "acos", "atan", "erf", "erfc", "trunc", "frac", "fmod_scalar", "fmod_tensor",
    "remainder_scalar", "remainder_tensor", "lerp", "lerp_tensor", "addmm", "addcmul", "addcdiv", "where", "scatter", "scatter_add",
    "index_add", "select_scatter", "narrow_scatter", "argsort", "diagonal", "movedim", "tile", "flip", "roll", "split", "unbind", "cat2",
    "pad_mode", "interpolate", "cdist", "one_hot", "bernoulli", "multinomial", "zeros_like", "ones_like", "full_like", "rand_like",
    "randn_like",
)


def install_variable_methods(cls) -> None:
    """Give `cls` (the `Variable` class) every op of `VARIABLE_METHODS` it does not define itself."""
    g = globals()

    def unwrap(x):
        if isinstance(x, cls):
            return x.t
        if isinstance(x, (list, tuple)) and x and isinstance(x[0], cls):
            return type(x)(v.t for v in x)
        return x

    def wrap(r):
        if isinstance(r, torch.Tensor):
            return cls.wrap(r)
        if isinstance(r, (list, tuple)):
            return type(r)(wrap(v) for v in r)
        return r

    def make(fn: Callable):
        def method(self, *args, **kw):
            return wrap(fn(self.t, *[unwrap(a) for a in args], **{k: unwrap(v) for k, v in kw.items()}))
        method.__name__ = fn.__name__
        method.__doc__ = f"`tensor_ops.{fn.__name__}` on this variable's tensor (flodl-sys/shim.h `flodl_{fn.__name__}`)."
        return method

    for name in VARIABLE_METHODS:
        if name not in cls.__dict__:
            setattr(cls, name, make(g[name]))


def surface() -> Dict[str, Callable]:
    """Every public op by name: this module's and `tensor_nn_ops`' (used by the API reference and the tests)."""
    from . import tensor_nn_ops as nn_ops
    out = {k: v for k, v in vars(nn_ops).items() if callable(v) and not k.startswith("_") and getattr(v, "__module__", None) == nn_ops.__name__
           and not isinstance(v, type)}
    out.update({k: v for k, v in globals().items() if callable(v) and not k.startswith("_") and getattr(v, "__module__", None) == __name__
                and k not in ("install_variable_methods", "surface")})
    return out
