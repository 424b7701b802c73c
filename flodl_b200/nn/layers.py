"""Layers (flodl/src/nn/*.rs): Linear, convolutions, pooling, normalisation, dropout, embeddings,
recurrent cells and stacks, attention, bilinear, padding, resampling.

Parameter names ("weight", "bias", "running_mean", ...) and module `name()`s follow the
reference exactly because checkpoint keys are derived from them
(`"{node_id-or-tag}/{param_name}"`, flodl/src/graph/graph.rs:768-814).
"""
from __future__ import annotations

import math
from typing import List, Optional, Sequence, Tuple

import torch
import torch.nn.functional as F

from .. import ops as _ops
from ..autograd import Variable
from ..autograd import ops as A
from ..tensor import Device, TensorError
from . import init
from .module import Buffer, Module, Parameter

W = Variable.wrap


def _tuple(v, n):
    return tuple(v) if isinstance(v, (tuple, list)) else (v,) * n


# ----------------------------------------------------------------------------------------- Linear
class Linear(Module):
    """y = x W^T + b, weight `[out, in]`, kaiming-uniform(a=sqrt 5) + uniform bias
    (flodl/src/nn/linear.rs:27-105)."""

    def __init__(self, in_features: int, out_features: int, bias: bool = True, device=None):
        self.weight = Parameter(init.kaiming_uniform([out_features, in_features], in_features, math.sqrt(5.0), device), "weight")
        self.bias = Parameter(init.uniform_bias(in_features, [out_features], device), "bias") if bias else None

    @classmethod
    def new(cls, in_features, out_features):
        return cls(in_features, out_features)

    @classmethod
    def on_device(cls, in_features, out_features, device):
        return cls(in_features, out_features, True, device)

    @classmethod
    def no_bias(cls, in_features, out_features, device=None):
        return cls(in_features, out_features, False, device)

    no_bias_on_device = no_bias

    @classmethod
    def from_shared_weight(cls, weight: Parameter, bias: Optional[Parameter] = None):
        self = cls.__new__(cls)
        self.weight, self.bias = weight, bias
        return self

    def name(self):
        return "linear"

    def forward(self, x):
        return W(_ops.linear(x.t, self.weight.t, None if self.bias is None else self.bias.t))

    def own_parameters(self):
        return [self.weight] + ([self.bias] if self.bias is not None else [])


# ------------------------------------------------------------------------------------------- conv
class _ConvBuilder:
    """`Conv2d.configure(in, out, k).with_stride(2).with_padding(1).without_bias().on_device(d).done()`
    (flodl/src/nn/conv2d.rs:40-110; the 1-D and 3-D builders are the same shape)."""

    def __init__(self, cls, in_c, out_c, k):
        self.cls, self.a = cls, dict(in_channels=in_c, out_channels=out_c, kernel_size=k)

    def with_stride(self, s): self.a["stride"] = s; return self
    def with_padding(self, p): self.a["padding"] = p; return self
    def with_dilation(self, d): self.a["dilation"] = d; return self
    def with_groups(self, g): self.a["groups"] = g; return self
    def with_output_padding(self, p): self.a["output_padding"] = p; return self
    def without_bias(self): self.a["bias"] = False; return self
    def on_device(self, device): self.a["device"] = device; return self
    def done(self): return self.cls(**self.a)


Conv1dBuilder = Conv2dBuilder = Conv3dBuilder = _ConvBuilder
ConvTranspose1dBuilder = ConvTranspose2dBuilder = ConvTranspose3dBuilder = _ConvBuilder


class _ConvNd(Module):
    ND = 2
    NAME = "conv2d"
    TRANSPOSED = False

    def __init__(self, in_channels, out_channels, kernel_size, stride=1, padding=0, dilation=1, groups=1, bias=True,
                 output_padding=0, device=None):
        n = self.ND
        self.kernel_size, self.stride, self.padding = _tuple(kernel_size, n), _tuple(stride, n), _tuple(padding, n)
        self.dilation, self.groups, self.output_padding = _tuple(dilation, n), groups, _tuple(output_padding, n)
        self.in_channels, self.out_channels = in_channels, out_channels
        ksz = math.prod(self.kernel_size)
        if self.TRANSPOSED:
            shape = [in_channels, out_channels // groups, *self.kernel_size]
            fan_in = (out_channels // groups) * ksz
        else:
            shape = [out_channels, in_channels // groups, *self.kernel_size]
            fan_in = (in_channels // groups) * ksz
        self.weight = Parameter(init.kaiming_uniform(shape, fan_in, math.sqrt(5.0), device), "weight")
        self.bias = Parameter(init.uniform_bias(fan_in, [out_channels], device), "bias") if bias else None
        if n == 2 and not self.TRANSPOSED:
            # a flat-buffer engine stores this filter K-R-S-C (see parallel/flat.py)
            self.weight.t._fb_channels_last = True
        # set by a model whose next layer is a BatchNorm over this output (see autograd.ops.conv2d)
        self.bn_stats = False

    @classmethod
    def new(cls, in_channels, out_channels, kernel_size):
        return cls(in_channels, out_channels, kernel_size)

    @classmethod
    def no_bias(cls, in_channels, out_channels, kernel_size):
        return cls(in_channels, out_channels, kernel_size, bias=False)

    @classmethod
    def configure(cls, in_channels, out_channels, kernel_size):
        return _ConvBuilder(cls, in_channels, out_channels, kernel_size)

    @classmethod
    def build(cls, in_channels, out_channels, kernel_size, with_bias=True, stride=1, padding=0, dilation=1, groups=1, device=None):
        return cls(in_channels, out_channels, kernel_size, stride, padding, dilation, groups, with_bias, 0, device)

    def name(self):
        return self.NAME

    def own_parameters(self):
        return [self.weight] + ([self.bias] if self.bias is not None else [])

    def forward(self, x):
        b = None if self.bias is None else self.bias.variable
        fn = {(1, False): A.conv1d, (2, False): A.conv2d, (3, False): A.conv3d,
              (1, True): A.conv_transpose1d, (2, True): A.conv_transpose2d, (3, True): A.conv_transpose3d}[(self.ND, self.TRANSPOSED)]
        if self.TRANSPOSED:
            return fn(x, self.weight.variable, b, self.stride, self.padding, self.output_padding, self.groups, self.dilation)
        if self.ND == 2 and self.bn_stats and self.bias is None:
            return fn(x, self.weight.variable, b, self.stride, self.padding, self.dilation, self.groups, bn_stats=True)
        return fn(x, self.weight.variable, b, self.stride, self.padding, self.dilation, self.groups)


class Conv1d(_ConvNd): ND, NAME = 1, "conv1d"
class Conv2d(_ConvNd): ND, NAME = 2, "conv2d"
class Conv3d(_ConvNd): ND, NAME = 3, "conv3d"
class ConvTranspose1d(_ConvNd): ND, NAME, TRANSPOSED = 1, "conv_t1d", True
class ConvTranspose2d(_ConvNd): ND, NAME, TRANSPOSED = 2, "conv_t2d", True
class ConvTranspose3d(_ConvNd): ND, NAME, TRANSPOSED = 3, "conv_transpose3d", True


# ---------------------------------------------------------------------------------------- pooling
class _PoolKnobs:
    """Builder-style setters shared by the pooling layers: `MaxPool2d.new(3).padding(1).ceil_mode(True)`,
    `AvgPool2d.with_stride(3, 2)` (flodl/src/nn/pooling.rs:45-90, 138-180)."""

    @classmethod
    def with_stride(cls, kernel_size, stride): return cls(kernel_size, stride)
    def padding(self, p): self.p = p; return self
    def dilation(self, d): self.d = d; return self
    def ceil_mode(self, on: bool): self.c = bool(on); return self
    def count_include_pad(self, on: bool): self.i = bool(on); return self


class MaxPool2d(_PoolKnobs, Module):
    def __init__(self, kernel_size, stride=None, padding=0, dilation=1, ceil_mode=False):
        self.k, self.s, self.p, self.d, self.c = kernel_size, stride or kernel_size, padding, dilation, ceil_mode
    def name(self): return "maxpool2d"
    def forward(self, x): return A.max_pool2d(x, self.k, self.s, self.p, self.d, self.c)


class AvgPool2d(_PoolKnobs, Module):
    def __init__(self, kernel_size, stride=None, padding=0, ceil_mode=False, count_include_pad=True):
        self.k, self.s, self.p, self.c, self.i = kernel_size, stride or kernel_size, padding, ceil_mode, count_include_pad
    def name(self): return "avgpool2d"
    def forward(self, x): return A.avg_pool2d(x, self.k, self.s, self.p, self.c, self.i)


class MaxPool1d(_PoolKnobs, Module):
    def __init__(self, kernel_size, stride=None, padding=0, dilation=1, ceil_mode=False):
        self.k, self.s, self.p, self.d, self.c = kernel_size, stride or kernel_size, padding, dilation, ceil_mode
    def name(self): return "maxpool1d"
    def forward(self, x): return A.max_pool1d(x, self.k, self.s, self.p, self.d, self.c)


class AvgPool1d(_PoolKnobs, Module):
    def __init__(self, kernel_size, stride=None, padding=0, ceil_mode=False, count_include_pad=True):
        self.k, self.s, self.p, self.c, self.i = kernel_size, stride or kernel_size, padding, ceil_mode, count_include_pad
    def name(self): return "avgpool1d"
    def forward(self, x): return A.avg_pool1d(x, self.k, self.s, self.p, self.c, self.i)


class AdaptiveMaxPool2d(Module):
    def __init__(self, output_size): self.o = output_size
    def name(self): return "adaptive_maxpool2d"
    def forward(self, x): return A.adaptive_max_pool2d(x, self.o)


class AdaptiveAvgPool2d(Module):
    def __init__(self, output_size): self.o = output_size
    def name(self): return "adaptive_avgpool2d"
    def forward(self, x): return A.adaptive_avg_pool2d(x, self.o)


class PixelShuffle(Module):
    def __init__(self, upscale_factor): self.f = upscale_factor
    def name(self): return "pixel_shuffle"
    def forward(self, x): return A.pixel_shuffle(x, self.f)


class PixelUnshuffle(Module):
    def __init__(self, downscale_factor): self.f = downscale_factor
    def name(self): return "pixel_unshuffle"
    def forward(self, x): return A.pixel_unshuffle(x, self.f)


class Upsample(Module):
    """Resize the spatial dimensions. `Upsample(scale_factor=2)` / `Upsample(size=(H, W), mode="bilinear")` in
    the PyTorch spelling, or the reference's `Upsample.new([H, W], mode)` with mode 0 = nearest, 1 = bilinear,
    2 = bicubic, 3 = trilinear, then `.align_corners(True)` (flodl/src/nn/pooling.rs:549-580)."""
    MODES = ("nearest", "bilinear", "bicubic", "trilinear")

    def __init__(self, scale_factor=None, size=None, mode="nearest", align_corners=None):
        self.sf, self.size, self.ac = scale_factor, size, align_corners
        self.mode = self.MODES[mode] if isinstance(mode, int) else mode

    @classmethod
    def new(cls, output_size, mode=0):
        return cls(size=tuple(output_size), mode=mode)

    def align_corners(self, on: bool):
        self.ac = bool(on)
        return self

    def name(self): return "upsample"

    def forward(self, x):
        ac = self.ac if self.mode != "nearest" else None
        return W(F.interpolate(x.t, size=self.size, scale_factor=self.sf, mode=self.mode, align_corners=ac))


class _FoldKnobs:
    def dilation(self, d): self._set(dilation=d); return self
    def padding(self, p): self._set(padding=p); return self
    def stride(self, s): self._set(stride=s); return self


class Unfold(_FoldKnobs, Module):
    """im2col: `Unfold(k, dilation, padding, stride)`, or `Unfold.new(3).padding([1, 1]).stride([2, 2])`,
    `Unfold.with_kernel([3, 5])` (flodl/src/nn/pooling.rs:634-660)."""

    def __init__(self, kernel_size, dilation=1, padding=0, stride=1): self.a = (kernel_size, dilation, padding, stride)
    @classmethod
    def with_kernel(cls, kernel_size): return cls(tuple(kernel_size))
    def _set(self, **kw):
        k, d, p, s = self.a
        self.a = (k, kw.get("dilation", d), kw.get("padding", p), kw.get("stride", s))
    def name(self): return "unfold"
    def forward(self, x): return A.im2col(x, *self.a)


class Fold(_FoldKnobs, Module):
    """col2im, the inverse of `Unfold` (flodl/src/nn/pooling.rs:712-740)."""

    def __init__(self, output_size, kernel_size, dilation=1, padding=0, stride=1): self.a = (output_size, kernel_size, dilation, padding, stride)
    @classmethod
    def with_kernel(cls, output_size, kernel_size): return cls(tuple(output_size), tuple(kernel_size))
    def _set(self, **kw):
        o, k, d, p, s = self.a
        self.a = (o, k, kw.get("dilation", d), kw.get("padding", p), kw.get("stride", s))
    def name(self): return "fold"
    def forward(self, x): return A.col2im(x, *self.a)


class ZeroPad2d(Module):
    """Zero padding of `[B, C, H, W]`: one amount for all sides, or `asymmetric(left, right, top, bottom)`."""
    def __init__(self, padding): self.p = _tuple(padding, 4)
    @classmethod
    def asymmetric(cls, left, right, top, bottom): return cls((left, right, top, bottom))
    def name(self): return "zero_pad2d"
    def forward(self, x): return W(F.pad(x.t, self.p))


class ReflectionPad2d(Module):
    def __init__(self, padding): self.p = _tuple(padding, 4)
    @classmethod
    def asymmetric(cls, left, right, top, bottom): return cls((left, right, top, bottom))
    def name(self): return "reflection_pad2d"
    def forward(self, x): return W(F.pad(x.t, self.p, mode="reflect"))


# ---------------------------------------------------------------------------------- normalisation
class LayerNorm(Module):
    """LayerNorm over the last dim, eps 1e-5 by default (flodl/src/nn/layernorm.rs:17-70)."""

    def __init__(self, size: int, eps: float = 1e-5, device=None):
        d = Device.of(device).torch if device is not None else None
        self.weight = Parameter(torch.ones(size, device=d), "weight")
        self.bias = Parameter(torch.zeros(size, device=d), "bias")
        self.eps, self.size = eps, size

    @classmethod
    def new(cls, size): return cls(size)
    @classmethod
    def with_eps(cls, size, eps): return cls(size, eps)
    @classmethod
    def on_device(cls, size, device): return cls(size, 1e-5, device)
    @classmethod
    def on_device_with_eps(cls, size, eps, device): return cls(size, eps, device)

    def name(self): return "layernorm"
    def own_parameters(self): return [self.weight, self.bias]
    def forward(self, x): return W(_ops.layer_norm(x.t, self.weight.t, self.bias.t, self.eps))


class RMSNorm(Module):
    def __init__(self, size: int, eps: float = 1e-6, device=None):
        d = Device.of(device).torch if device is not None else None
        self.weight = Parameter(torch.ones(size, device=d), "weight")
        self._eps = eps
    @classmethod
    def new(cls, size): return cls(size)
    @classmethod
    def on_device(cls, size, device): return cls(size, device=device)
    def eps(self, eps): self._eps = eps; return self
    def name(self): return "rmsnorm"
    def own_parameters(self): return [self.weight]
    def forward(self, x):
        t = x.t
        f = t if t.dtype == torch.float64 else t.float()      # statistics in fp32 at least (fp64 stays fp64)
        ms = f.pow(2).mean(-1, keepdim=True)
        return W((f * torch.rsqrt(ms + self._eps)).to(t.dtype) * self.weight.t.to(t.dtype))


class GroupNorm(Module):
    def __init__(self, num_groups: int, num_channels: int, eps: float = 1e-5, device=None):
        d = Device.of(device).torch if device is not None else None
        self.g, self.eps = num_groups, eps
        self.weight = Parameter(torch.ones(num_channels, device=d), "weight")
        self.bias = Parameter(torch.zeros(num_channels, device=d), "bias")
    @classmethod
    def new(cls, g, c): return cls(g, c)
    @classmethod
    def on_device(cls, g, c, device): return cls(g, c, device=device)
    def name(self): return "groupnorm"
    def own_parameters(self): return [self.weight, self.bias]
    def forward(self, x): return A.group_norm(x, self.g, self.weight.variable, self.bias.variable, self.eps)


class BatchNorm(Module):
    """BatchNorm over dim 1 for [B, C] / [B, C, L] / [B, C, H, W]; eps 1e-5, momentum 0.1; training
    needs batch >= 2 (flodl/src/nn/batchnorm.rs)."""

    def __init__(self, num_features: int, device=None, eps: float = 1e-5, momentum: float = 0.1):
        d = Device.of(device).torch if device is not None else None
        self.weight = Parameter(torch.ones(num_features, device=d), "weight")
        self.bias = Parameter(torch.zeros(num_features, device=d), "bias")
        self.running_mean = Buffer(torch.zeros(num_features, device=d), "running_mean")
        self.running_var = Buffer(torch.ones(num_features, device=d), "running_var")
        self.num_features, self.eps, self.momentum = num_features, eps, momentum
        self.fuse_relu = False

    @classmethod
    def new(cls, n): return cls(n)
    @classmethod
    def on_device(cls, n, device): return cls(n, device)

    def name(self): return "batchnorm"
    def own_parameters(self): return [self.weight, self.bias]
    def own_buffers(self): return [self.running_mean, self.running_var]

    def forward(self, x, residual: Optional[Variable] = None, relu: Optional[bool] = None):
        if self.training and x.t.shape[0] < 2:
            raise TensorError("BatchNorm requires batch_size >= 2 in training mode (Bessel's correction divides by batch_size-1)")
        return W(_ops.batch_norm(x.t, self.running_mean.t, self.running_var.t, self.weight.t, self.bias.t, self.training,
                                 self.momentum, self.eps, self.fuse_relu if relu is None else relu,
                                 None if residual is None else residual.t))


class BatchNorm2d(BatchNorm):
    def name(self): return "batchnorm2d"
    def forward(self, x, residual=None, relu=None):
        if x.t.dim() != 4:
            raise TensorError("BatchNorm2d: input must be 4D [B, C, H, W]")
        return super().forward(x, residual, relu)


class InstanceNorm(Module):
    def __init__(self, num_features: int, affine: bool = True, eps: float = 1e-5, device=None):
        d = Device.of(device).torch if device is not None else None
        self.eps = eps
        self.weight = Parameter(torch.ones(num_features, device=d), "weight") if affine else None
        self.bias = Parameter(torch.zeros(num_features, device=d), "bias") if affine else None
    def name(self): return "instance_norm"
    def own_parameters(self): return [p for p in (self.weight, self.bias) if p is not None]
    def forward(self, x):
        return A.instance_norm(x, None if self.weight is None else self.weight.variable,
                               None if self.bias is None else self.bias.variable, eps=self.eps)


# ---------------------------------------------------------------------------------------- dropout
class Dropout(Module):
    def __init__(self, p: float = 0.5): self.p = p
    @classmethod
    def new(cls, p): return cls(p)
    def name(self): return "dropout"
    def forward(self, x): return W(_ops.dropout(x.t, self.p, self.training))


class Dropout2d(Module):
    def __init__(self, p: float = 0.5): self.p = p
    def name(self): return "dropout2d"
    def forward(self, x): return W(F.dropout2d(x.t, self.p, self.training))


class AlphaDropout(Module):
    def __init__(self, p: float = 0.5): self.p = p
    def name(self): return "alpha_dropout"
    def forward(self, x): return W(F.alpha_dropout(x.t, self.p, self.training))


# -------------------------------------------------------------------------------------- embedding
class Embedding(Module):
    """Lookup table, N(0,1) init; `padding_idx` row is zero and gets no gradient
    (flodl/src/nn/embedding.rs)."""

    def __init__(self, num_embeddings: int, embedding_dim: int, padding_idx: Optional[int] = None, device=None):
        w = init.normal([num_embeddings, embedding_dim], 0.0, 1.0, device)
        if padding_idx is not None:
            w[padding_idx].zero_()
        self.weight = Parameter(w, "weight")
        self.padding_idx = padding_idx
        self.num_embeddings, self.embedding_dim = num_embeddings, embedding_dim

    @classmethod
    def new(cls, n, d): return cls(n, d)
    @classmethod
    def on_device(cls, n, d, device): return cls(n, d, None, device)
    @classmethod
    def with_padding_idx(cls, n, d, padding_idx): return cls(n, d, padding_idx)
    @classmethod
    def on_device_with_padding_idx(cls, n, d, padding_idx, device): return cls(n, d, padding_idx, device)

    def name(self): return "embedding"
    def own_parameters(self): return [self.weight]

    def forward(self, x):
        idx = x.t if not x.t.is_floating_point() else x.t.long()
        return W(_ops.embedding(idx, self.weight.t, self.padding_idx))


class EmbeddingBag(Module):
    MODES = {0: "sum", 1: "mean", 2: "max"}

    def __init__(self, num_embeddings: int, embedding_dim: int, mode=1, device=None):
        self.weight = Parameter(init.normal([num_embeddings, embedding_dim], 0.0, 1.0, device), "weight")
        self.mode = self.MODES.get(mode, mode)
    def name(self): return "embedding_bag"
    def own_parameters(self): return [self.weight]
    def forward_bag(self, indices, offsets): return W(F.embedding_bag(indices, self.weight.t, offsets, mode=self.mode))
    def forward(self, x):
        idx = x.t.long()
        return W(F.embedding_bag(idx, self.weight.t, mode=self.mode)) if idx.dim() == 2 else self.forward_bag(idx, torch.zeros(1, dtype=torch.long, device=idx.device))


# -------------------------------------------------------------------------------------- recurrent
class GRUCell(Module):
    def __init__(self, input_size: int, hidden_size: int, device=None):
        k = hidden_size
        self.w_ih = Parameter(init.uniform_bias(k, [3 * k, input_size], device), "w_ih")
        self.w_hh = Parameter(init.uniform_bias(k, [3 * k, k], device), "w_hh")
        self.b_ih = Parameter(init.uniform_bias(k, [3 * k], device), "b_ih")
        self.b_hh = Parameter(init.uniform_bias(k, [3 * k], device), "b_hh")
        self.hidden_size = k
        self._h: Optional[Variable] = None
    def name(self): return "grucell"
    def own_parameters(self): return [self.w_ih, self.w_hh, self.b_ih, self.b_hh]
    def forward_step(self, x, h=None):
        if h is None:
            h = W(torch.zeros(x.t.shape[0], self.hidden_size, dtype=x.t.dtype, device=x.t.device))
        return A.gru_cell(x, h, self.w_ih.variable, self.w_hh.variable, self.b_ih.variable, self.b_hh.variable)
    def forward(self, x):
        self._h = self.forward_step(x, self._h)
        return self._h
    def reset(self): self._h = None
    def detach_state(self):
        if self._h is not None:
            self._h = self._h.detach()


class LSTMCell(Module):
    def __init__(self, input_size: int, hidden_size: int, device=None):
        k = hidden_size
        self.w_ih = Parameter(init.uniform_bias(k, [4 * k, input_size], device), "w_ih")
        self.w_hh = Parameter(init.uniform_bias(k, [4 * k, k], device), "w_hh")
        self.b_ih = Parameter(init.uniform_bias(k, [4 * k], device), "b_ih")
        self.b_hh = Parameter(init.uniform_bias(k, [4 * k], device), "b_hh")
        self.hidden_size = k
        self._state = None
    def name(self): return "lstmcell"
    def own_parameters(self): return [self.w_ih, self.w_hh, self.b_ih, self.b_hh]
    def forward_step(self, x, state=None):
        if state is None:
            z = W(torch.zeros(x.t.shape[0], self.hidden_size, dtype=x.t.dtype, device=x.t.device))
            state = (z, z)
        return A.lstm_cell(x, state[0], state[1], self.w_ih.variable, self.w_hh.variable, self.b_ih.variable, self.b_hh.variable)
    def forward(self, x):
        self._state = self.forward_step(x, self._state)
        return self._state[0]
    def reset(self): self._state = None
    def detach_state(self):
        if self._state is not None:
            self._state = (self._state[0].detach(), self._state[1].detach())


class _RNNBase(Module):
    MODE, GATES, NAME = "GRU", 3, "gru"

    def __init__(self, input_size: int, hidden_size: int, num_layers: int = 1, device=None):
        self.input_size, self.hidden_size, self.num_layers = input_size, hidden_size, num_layers
        self._batch_first = False
        self.params: List[Parameter] = []
        for l in range(num_layers):
            isz = input_size if l == 0 else hidden_size
            for nm, shape in (("weight_ih", [self.GATES * hidden_size, isz]), ("weight_hh", [self.GATES * hidden_size, hidden_size]),
                              ("bias_ih", [self.GATES * hidden_size]), ("bias_hh", [self.GATES * hidden_size])):
                self.params.append(Parameter(init.uniform_bias(hidden_size, shape, device), f"{nm}_l{l}"))

    @classmethod
    def new(cls, input_size, hidden_size, num_layers): return cls(input_size, hidden_size, num_layers)
    @classmethod
    def on_device(cls, input_size, hidden_size, num_layers, device): return cls(input_size, hidden_size, num_layers, device)
    def batch_first(self, flag: bool): self._batch_first = flag; return self
    def name(self): return self.NAME
    def own_parameters(self): return list(self.params)

    def forward_seq(self, x: Variable, state=None):
        """Whole-sequence pass through the fused RNN (cuDNN on CUDA, as in ops_training.cpp:358-500).
        Returns (output, final state)."""
        t = x.t
        B = t.shape[0] if self._batch_first else t.shape[1]
        flat = [p.t.to(t.dtype) if p.t.dtype != t.dtype else p.t for p in self.params]
        if self.MODE == "GRU":
            h0 = state.t if state is not None else torch.zeros(self.num_layers, B, self.hidden_size, dtype=t.dtype, device=t.device)
            out, hn = torch.gru(t, h0, flat, True, self.num_layers, 0.0, self.training, False, self._batch_first)
            return W(out), W(hn)
        if state is not None:
            h0, c0 = state[0].t, state[1].t
        else:
            h0 = torch.zeros(self.num_layers, B, self.hidden_size, dtype=t.dtype, device=t.device)
            c0 = torch.zeros_like(h0)
        out, hn, cn = torch.lstm(t, (h0, c0), flat, True, self.num_layers, 0.0, self.training, False, self._batch_first)
        return W(out), (W(hn), W(cn))

    def forward(self, x):
        return self.forward_seq(x)[0]


class GRU(_RNNBase): MODE, GATES, NAME = "GRU", 3, "gru"
class LSTM(_RNNBase): MODE, GATES, NAME = "LSTM", 4, "lstm"


# -------------------------------------------------------------------------------------- attention
class MultiheadAttention(Module):
    """Four xavier-uniform projections with zero bias around scaled dot-product attention
    (flodl/src/nn/attention.rs:20-160). Parameter names: q_proj.weight, q_proj.bias, k_proj..., out_proj....
    `mask` marks positions to exclude (non-zero = masked); a strictly upper-triangular [S, S] mask is
    recognised as causal and, like an absent mask, runs on the fused attention kernel."""

    def __init__(self, embed_dim: int, num_heads: int, device=None):
        if embed_dim % num_heads:
            raise TensorError(f"embed_dim ({embed_dim}) must be divisible by num_heads ({num_heads})")
        self.embed_dim, self.num_heads, self.head_dim = embed_dim, num_heads, embed_dim // num_heads
        self.scale = 1.0 / math.sqrt(self.head_dim)
        d = Device.of(device).torch if device is not None else None
        self.proj = {}
        for nm in ("q_proj", "k_proj", "v_proj", "out_proj"):
            w = Parameter(init.xavier_uniform([embed_dim, embed_dim], embed_dim, embed_dim, device), f"{nm}.weight")
            b = Parameter(torch.zeros(embed_dim, device=d), f"{nm}.bias")
            self.proj[nm] = (w, b)
        self.causal = False

    @classmethod
    def new(cls, embed_dim, num_heads): return cls(embed_dim, num_heads)
    @classmethod
    def on_device(cls, embed_dim, num_heads, device): return cls(embed_dim, num_heads, device)

    def name(self): return "multihead_attention"
    def own_parameters(self): return [p for nm in ("q_proj", "k_proj", "v_proj", "out_proj") for p in self.proj[nm]]

    def _lin(self, nm, x):
        w, b = self.proj[nm]
        return _ops.linear(x, w.t, b.t)

    def forward_ext(self, query, key, value, mask: Optional[torch.Tensor] = None):
        q, k, v = query.t, key.t, value.t
        B, Sq, Sk = q.shape[0], q.shape[1], k.shape[1]
        H, D = self.num_heads, self.head_dim
        qp = self._lin("q_proj", q).reshape(B, Sq, H, D)
        kp = self._lin("k_proj", k).reshape(B, Sk, H, D)
        vp = self._lin("v_proj", v).reshape(B, Sk, H, D)
        causal = self.causal
        add_mask = None
        if mask is not None:
            mb = mask != 0
            if mb.dim() == 2 and Sq == Sk and mb.shape == (Sq, Sk) and bool(torch.equal(mb, torch.ones_like(mb).triu(1))):
                causal = True
            else:
                add_mask = torch.zeros(mb.shape, dtype=torch.float32, device=q.device).masked_fill(mb, float("-inf"))
        if Sq == Sk:
            o = _ops.attention(q=qp, k=kp, v=vp, mask=add_mask, causal=causal, scale=self.scale)
        else:
            qh, kh, vh = (t.transpose(1, 2) for t in (qp, kp, vp))
            s = (qh @ kh.transpose(-1, -2)) * self.scale
            if add_mask is not None:
                s = s + add_mask.to(s.dtype)
            o = (torch.softmax(s, -1) @ vh).transpose(1, 2)
        return W(self._lin("out_proj", o.reshape(B, Sq, H * D)))

    def forward(self, x):
        return self.forward_ext(x, x, x, None)


class Bilinear(Module):
    def __init__(self, in1: int, in2: int, out: int, bias: bool = True, device=None):
        bound = 1.0 / math.sqrt(in1)
        self.weight = Parameter(init.uniform([out, in1, in2], -bound, bound, device), "weight")
        self.bias = Parameter(init.uniform([out], -bound, bound, device), "bias") if bias else None
    def name(self): return "bilinear"
    def own_parameters(self): return [self.weight] + ([self.bias] if self.bias is not None else [])
    def forward_pair(self, a, b): return A.bilinear(a, b, self.weight.variable, None if self.bias is None else self.bias.variable)
    forward_bilinear = forward_pair                                   # the reference's name (bilinear.rs:77)
    def forward(self, x): return self.forward_pair(x, x)


def gaussian_blur_2d(x: Variable, sigma: float, kernel_size: Optional[int] = None) -> Variable:
    """Depthwise separable Gaussian blur (flodl/src/nn/functional.rs)."""
    k = kernel_size or (int(2 * math.ceil(3 * sigma)) + 1)
    ax = torch.arange(k, dtype=torch.float32, device=x.t.device) - (k - 1) / 2
    g = torch.exp(-(ax ** 2) / (2 * sigma * sigma))
    g = (g / g.sum()).to(x.t.dtype)
    C = x.t.shape[1]
    t = F.conv2d(F.pad(x.t, (k // 2, k // 2, 0, 0), mode="reflect"), g.view(1, 1, 1, k).expand(C, 1, 1, k), groups=C)
    t = F.conv2d(F.pad(t, (0, 0, k // 2, k // 2), mode="reflect"), g.view(1, 1, k, 1).expand(C, 1, k, 1), groups=C)
    return W(t)


class GaussianBlur(Module):
    def __init__(self, sigma: float, kernel_size: Optional[int] = None): self.sigma, self.k = sigma, kernel_size
    def name(self): return "gaussian_blur"
    def forward(self, x): return gaussian_blur_2d(x, self.sigma, self.k)
