"""BatchNorm (+ residual add, + ReLU) dispatch: native fused kernel on CUDA, PyTorch elsewhere."""
from __future__ import annotations

import torch
import torch.nn.functional as F

from .. import _ext
from . import core


class _BatchNormFn(torch.autograd.Function):
    """Training-mode BN over [N, C, *spatial] with optional fused residual add and ReLU.
    One statistics pass and one normalise pass forward; backward reduces dgamma/dbeta and writes
    dx (and the residual gradient) in two passes."""

    @staticmethod
    def forward(ctx, x, residual, weight, bias, running_mean, running_var, momentum, eps, relu, sums=None):
        C = _ext.require()
        # channels-last tensors stay channels-last (the NHWC kernels); everything else is made NCHW-contiguous
        cl = _is_channels_last(x)
        fmt = torch.channels_last if cl else torch.contiguous_format
        xc = x.contiguous(memory_format=fmt)
        rc = None if residual is None else residual.contiguous(memory_format=fmt)
        if sums is not None and not cl:
            sums = None
        y, mean, rstd = C.bn_fwd(xc, rc, core._f32(weight), core._f32(bias), running_mean, running_var, eps, momentum, relu, True, sums)
        core._launched(1 if sums is not None else 2)
        ctx.save_for_backward(xc, y, mean, rstd)
        ctx.weight, ctx.bias, ctx.relu, ctx.has_res, ctx.fmt = weight, bias, relu, rc is not None, fmt
        return y

    @staticmethod
    def backward(ctx, dy):
        C = _ext.require()
        x, y, mean, rstd = ctx.saved_tensors
        w, b = ctx.weight, ctx.bias
        gslot, bslot = core._grad_slot(w), core._grad_slot(b)
        use_slots = gslot is not None and bslot is not None
        dx, dres, dg, db = C.bn_bwd(dy.contiguous(memory_format=ctx.fmt), x, y, core._f32(w), mean, rstd, ctx.relu, ctx.has_res,
                                    gslot.view(-1) if use_slots else None, bslot.view(-1) if use_slots else None)
        core._launched(2)
        if use_slots:
            core._touched(w)
            core._touched(b)
            dg = db = None
        else:
            dg = None if w is None else dg.to(w.dtype)
            db = None if b is None else db.to(b.dtype)
        return dx, (dres if ctx.has_res else None), dg, db, None, None, None, None, None, None


def _is_channels_last(x: torch.Tensor) -> bool:
    return x.dim() == 4 and x.is_contiguous(memory_format=torch.channels_last) and not x.is_contiguous() \
        and x.shape[1] % (8 if x.dtype == torch.bfloat16 else 4) == 0 and x.shape[1] <= 256


def _eligible(x: torch.Tensor, weight, training: bool) -> bool:
    C = _ext.load()
    return (core._native_ok(x) and training and C is not None and hasattr(C, "bn_fwd") and x.dim() >= 3
            and x.dtype in (torch.bfloat16, torch.float32) and weight is not None and x.numel() > 0)


def batch_norm(x, running_mean, running_var, weight, bias, training, momentum=0.1, eps=1e-5, relu=False, residual=None):
    if _eligible(x, weight, training) and (residual is None or residual.dtype == x.dtype):
        # sums accumulated by the convolution that produced x (see ops.conv.conv2d), if any
        sums = getattr(x, "_fb_bn_sums", None)
        return _BatchNormFn.apply(x, residual, weight, bias, running_mean, running_var, float(momentum), float(eps), bool(relu), sums)
    y = F.batch_norm(x, running_mean, running_var, weight, bias, training, momentum, eps)
    if residual is not None:
        y = y + residual
    return F.relu(y) if relu else y
