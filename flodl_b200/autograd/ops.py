"""Free-function differentiable ops on `Variable`s (flodl/src/autograd/ops.rs:570-987).

The ones on the named hot paths (`linear`, `layer_norm`, `scaled_dot_product_attention`, and
`conv2d` on CUDA) dispatch to the native kernels through `flodl_b200.ops`; the rest are the
PyTorch ops with the reference's argument conventions.
"""
from __future__ import annotations

from typing import Optional, Sequence

import torch
import torch.nn.functional as F

from .. import ops as _ops
from .variable import Variable, _t

W = Variable.wrap


def linear(x, weight, bias=None) -> Variable:
    return W(_ops.linear(_t(x), _t(weight), None if bias is None else _t(bias)))


def layer_norm(x, weight=None, bias=None, eps: float = 1e-5) -> Variable:
    return W(_ops.layer_norm(_t(x), None if weight is None else _t(weight), None if bias is None else _t(bias), eps))


def group_norm(x, num_groups: int, weight=None, bias=None, eps: float = 1e-5) -> Variable:
    return W(F.group_norm(_t(x), num_groups, None if weight is None else _t(weight), None if bias is None else _t(bias), eps))


def instance_norm(x, weight=None, bias=None, running_mean=None, running_var=None, use_input_stats=True, momentum=0.1, eps=1e-5) -> Variable:
    return W(F.instance_norm(_t(x), running_mean, running_var, None if weight is None else _t(weight),
                             None if bias is None else _t(bias), use_input_stats, momentum, eps))


def gru_cell(x, h, w_ih, w_hh, b_ih=None, b_hh=None) -> Variable:
    return W(torch.gru_cell(_t(x), _t(h), _t(w_ih), _t(w_hh), None if b_ih is None else _t(b_ih), None if b_hh is None else _t(b_hh)))


def lstm_cell(x, h, c, w_ih, w_hh, b_ih=None, b_hh=None):
    h2, c2 = torch.lstm_cell(_t(x), (_t(h), _t(c)), _t(w_ih), _t(w_hh), None if b_ih is None else _t(b_ih), None if b_hh is None else _t(b_hh))
    return W(h2), W(c2)


def _pair(v, n):
    return tuple(v) if isinstance(v, (tuple, list)) else (v,) * n


def conv1d(x, weight, bias=None, stride=1, padding=0, dilation=1, groups=1) -> Variable:
    return W(F.conv1d(_t(x), _cast(_t(weight), x), _castb(bias, x), stride, padding, dilation, groups))


def conv2d(x, weight, bias=None, stride=1, padding=0, dilation=1, groups=1, bn_stats=False) -> Variable:
    """`bn_stats`: the caller feeds the result straight into a training-mode BatchNorm, so the native
    kernel may accumulate the per-channel sums in its epilogue and hand them over with the tensor."""
    from ..ops import conv as _conv
    return W(_conv.conv2d(_t(x), _t(weight), None if bias is None else _t(bias), _pair(stride, 2), _pair(padding, 2), _pair(dilation, 2), groups,
                          bn_stats=bn_stats))


def conv3d(x, weight, bias=None, stride=1, padding=0, dilation=1, groups=1) -> Variable:
    return W(F.conv3d(_t(x), _cast(_t(weight), x), _castb(bias, x), stride, padding, dilation, groups))


def conv_transpose1d(x, weight, bias=None, stride=1, padding=0, output_padding=0, groups=1, dilation=1) -> Variable:
    return W(F.conv_transpose1d(_t(x), _cast(_t(weight), x), _castb(bias, x), stride, padding, output_padding, groups, dilation))


def conv_transpose2d(x, weight, bias=None, stride=1, padding=0, output_padding=0, groups=1, dilation=1) -> Variable:
    return W(F.conv_transpose2d(_t(x), _cast(_t(weight), x), _castb(bias, x), stride, padding, output_padding, groups, dilation))


def conv_transpose3d(x, weight, bias=None, stride=1, padding=0, output_padding=0, groups=1, dilation=1) -> Variable:
    return W(F.conv_transpose3d(_t(x), _cast(_t(weight), x), _castb(bias, x), stride, padding, output_padding, groups, dilation))


def _cast(w, x):
    xt = _t(x)
    return w if w.dtype == xt.dtype else w.to(xt.dtype)


def _castb(b, x):
    return None if b is None else _cast(_t(b), x)


def max_pool2d(x, kernel_size, stride=None, padding=0, dilation=1, ceil_mode=False) -> Variable:
    return W(F.max_pool2d(_t(x), kernel_size, stride, padding, dilation, ceil_mode))


def avg_pool2d(x, kernel_size, stride=None, padding=0, ceil_mode=False, count_include_pad=True) -> Variable:
    return W(F.avg_pool2d(_t(x), kernel_size, stride, padding, ceil_mode, count_include_pad))


def max_pool1d(x, kernel_size, stride=None, padding=0, dilation=1, ceil_mode=False) -> Variable:
    return W(F.max_pool1d(_t(x), kernel_size, stride, padding, dilation, ceil_mode))


def avg_pool1d(x, kernel_size, stride=None, padding=0, ceil_mode=False, count_include_pad=True) -> Variable:
    return W(F.avg_pool1d(_t(x), kernel_size, stride, padding, ceil_mode, count_include_pad))


def adaptive_avg_pool2d(x, output_size) -> Variable:
    return W(F.adaptive_avg_pool2d(_t(x), output_size))


def adaptive_max_pool2d(x, output_size) -> Variable:
    return W(F.adaptive_max_pool2d(_t(x), output_size))


def im2col(x, kernel_size, dilation=1, padding=0, stride=1) -> Variable:
    return W(F.unfold(_t(x), kernel_size, dilation, padding, stride))


def col2im(x, output_size, kernel_size, dilation=1, padding=0, stride=1) -> Variable:
    return W(F.fold(_t(x), output_size, kernel_size, dilation, padding, stride))


def pixel_shuffle(x, upscale_factor: int) -> Variable:
    return W(F.pixel_shuffle(_t(x), upscale_factor))


def pixel_unshuffle(x, downscale_factor: int) -> Variable:
    return W(F.pixel_unshuffle(_t(x), downscale_factor))


def bilinear(x1, x2, weight, bias=None) -> Variable:
    return W(F.bilinear(_t(x1), _t(x2), _t(weight), None if bias is None else _t(bias)))


def grid_sample(x, grid, mode="bilinear", padding_mode="zeros", align_corners=False) -> Variable:
    return W(F.grid_sample(_t(x), _t(grid), mode=mode, padding_mode=padding_mode, align_corners=align_corners))


def scaled_dot_product_attention(q, k, v, attn_mask=None, dropout_p: float = 0.0, is_causal: bool = False,
                                 scale: Optional[float] = None, training: bool = True) -> Variable:
    """q, k, v: [B, H, S, D] (the reference's layout, flodl/src/autograd/ops.rs:947-963)."""
    qt, kt, vt = (_t(a).transpose(1, 2) for a in (q, k, v))
    o = _ops.attention(q=qt, k=kt, v=vt, mask=None if attn_mask is None else _t(attn_mask), causal=is_causal,
                       p_drop=dropout_p, training=training, scale=scale)
    return W(o.transpose(1, 2))


def embedding(weight, indices, padding_idx: Optional[int] = None) -> Variable:
    return W(F.embedding(_t(indices), _t(weight), padding_idx))


def embedding_bag(weight, indices, offsets, mode: str = "mean") -> Variable:
    return W(F.embedding_bag(_t(indices), _t(weight), _t(offsets), mode=mode))


def dropout(x, p: float, training: bool = True) -> Variable:
    return W(_ops.dropout(_t(x), p, training))


def batch_norm(x, running_mean, running_var, weight=None, bias=None, training=True, momentum=0.1, eps=1e-5) -> Variable:
    return W(_ops.batch_norm(_t(x), running_mean, running_var, None if weight is None else _t(weight),
                             None if bias is None else _t(bias), training, momentum, eps))
