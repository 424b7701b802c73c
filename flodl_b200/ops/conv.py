"""conv2d dispatch. The native tcgen05 kernels cover channels-last bf16 activations with the CIFAR
ResNet's filter shapes (3x3 / 1x1, stride 1 or 2, 16/32/64 channels, groups 1): forward, stride-1
data gradient and filter gradient. Everything else (the 3-channel stem, strided data gradients,
other layouts and dtypes) runs the PyTorch op."""
from __future__ import annotations

import os

import torch
import torch.nn.functional as F

from .. import _ext
from . import core


# Widest channel count sent to the native data-gradient / forward kernels. Measured in a ResNet-20 step on
# B200: the native data gradient wins up to 32 channels and loses at 64 (one 36-instruction tile per CTA
# plus a 73 KB filter load; 1.264 ms per step against 1.183 with cuDNN there), while the native forward
# pays for itself at every width because its epilogue saves the BatchNorm statistics pass (1.200 vs 1.237).
_MAX_CI = int(os.environ.get("FLODL_B200_CONV_MAX_CI", "32"))
_MAX_FPROP_CI = int(os.environ.get("FLODL_B200_CONV_MAX_FPROP_CI", "64"))
_MAX_WGRAD_CI = int(os.environ.get("FLODL_B200_CONV_MAX_WGRAD_CI", "64"))


def _pair(v):
    return (int(v), int(v)) if isinstance(v, int) else tuple(int(a) for a in v)


def _padded_ci(x: torch.Tensor, ci: int) -> int:
    """An input layer with fewer than 16 channels (RGB) runs on the native kernels with its channels
    zero-padded to 16: the extra filter channels only ever see zeros, so neither the output nor the
    gradient of the real channels changes. Only where no input gradient is wanted."""
    return 16 if ci < 16 and not x.requires_grad else ci


def _pad_channels(t: torch.Tensor, c: int) -> torch.Tensor:
    out = torch.zeros((t.shape[0], c, t.shape[2], t.shape[3]), dtype=t.dtype, device=t.device).contiguous(memory_format=torch.channels_last)
    out[:, :t.shape[1]] = t
    return out


class _Conv2dShadowFn(torch.autograd.Function):
    """Convolution on channels-last bf16 activations whose filter lives in a flat parameter buffer:
    forward reads the bf16 shadow of the filter (already K-R-S-C, refreshed by the optimizer kernel),
    backward adds the filter gradient straight into the fp32 gradient slot. Compared with
    `weight.to(bf16)` under autograd this drops one cast per forward and the cast + layout change +
    accumulate chain per backward."""

    @staticmethod
    def forward(ctx, x, weight, stride, padding, dilation, groups, sums=None):
        w16 = weight._fb_bf16
        ctx.save_for_backward(x, w16)
        ctx.weight, ctx.conf = weight, (stride, padding, dilation, groups)
        core._launched()
        C = _ext.require()
        N, Ci, H, W = x.shape
        Co, _, k, kw = w16.shape
        ctx.simple = (dilation == (1, 1) and groups == 1 and k == kw and stride[0] == stride[1] and padding[0] == padding[1])
        ctx.pad_ci = 0
        cp = _padded_ci(x, Ci)
        if ctx.simple and cp != Ci and C.conv_fprop_supported(N, H, W, cp, Co, k, stride[0], padding[0]) \
                and C.conv_wgrad_supported(N, H, W, cp, Co, k, stride[0], padding[0]):
            xp = _pad_channels(x, cp)
            ctx.save_for_backward(xp, w16)
            ctx.pad_ci = Ci
            core._launched(4)
            return C.conv_fprop(xp, _pad_channels(w16, cp), stride[0], padding[0], sums)
        if ctx.simple and (Ci <= _MAX_FPROP_CI or sums is not None) and C.conv_fprop_supported(N, H, W, Ci, Co, k, stride[0], padding[0]):
            return C.conv_fprop(x, w16, stride[0], padding[0], sums)
        if sums is not None:
            raise RuntimeError("BatchNorm sums requested from a convolution the native kernel does not cover")
        return F.conv2d(x, w16, None, stride, padding, dilation, groups)

    @staticmethod
    def backward(ctx, dy):
        x, w16 = ctx.saved_tensors
        stride, padding, dilation, groups = ctx.conf
        dy = dy.contiguous(memory_format=torch.channels_last)
        C = _ext.require()
        N, Ci, H, W = x.shape
        Co, _, k, _ = w16.shape
        if ctx.pad_ci:
            # x is the zero-padded input saved by forward; only the real channels' filter gradient is kept
            dwp = torch.zeros((Co, Ci, k, k), dtype=torch.float32, device=x.device).contiguous(memory_format=torch.channels_last)
            C.conv_wgrad(x, dy, dwp, stride[0], padding[0])
            ctx.weight._fb_grad.add_(dwp[:, :ctx.pad_ci])
            core._launched(3)
            core._touched(ctx.weight)
            return None, None, None, None, None, None, None
        shape = (N, H, W, Ci, Co, k, stride[0], padding[0])
        native_w = ctx.simple and Ci <= _MAX_WGRAD_CI and C.conv_wgrad_supported(*shape)
        native_x = ctx.needs_input_grad[0] and ctx.simple and max(Ci, Co) <= _MAX_CI and C.conv_dgrad_supported(*shape)
        dx = dw = None
        if (ctx.needs_input_grad[0] and not native_x) or not native_w:
            dx, dw, _ = torch.ops.aten.convolution_backward(dy, x, w16, None, list(stride), list(padding), list(dilation), False, [0, 0], groups,
                                                            [ctx.needs_input_grad[0] and not native_x, not native_w, False])
            core._launched()
        if native_x:
            dx = C.conv_dgrad(dy, w16, stride[0], padding[0])
            core._launched()
        if native_w:
            # filter gradient on the tensor cores, accumulated into the fp32 slot in place
            C.conv_wgrad(x, dy, ctx.weight._fb_grad, stride[0], padding[0])
            core._launched()
        else:
            ctx.weight._fb_grad.add_(dw)
        core._touched(ctx.weight)
        return dx, None, None, None, None, None, None


def conv2d(x, weight, bias=None, stride=(1, 1), padding=(0, 0), dilation=(1, 1), groups=1, bn_stats=False):
    """`bn_stats`: a training-mode BatchNorm consumes the result directly; when the native forward
    kernel runs, it accumulates the per-channel sum and sum of squares in its epilogue and the result
    carries them as `_fb_bn_sums` (fp32 [2, Co]), which `ops.bn.batch_norm` picks up instead of making
    its own statistics pass."""
    if (x.dim() == 4 and x.is_cuda and core.FLAGS.native and x.dtype == torch.bfloat16 and getattr(weight, "_fb_bf16", None) is not None
            and getattr(weight, "_fb_channels_last", False) and x.is_contiguous(memory_format=torch.channels_last)):
        stride, padding, dilation = _pair(stride), _pair(padding), _pair(dilation)
        sums = None
        if bn_stats and bias is None and torch.is_grad_enabled() and x.shape[1] <= _MAX_FPROP_CI:
            N, Ci, H, W = x.shape
            Co, _, k, kw = weight.shape
            cp = _padded_ci(x, Ci)
            Cx = _ext.require()
            if (dilation == (1, 1) and groups == 1 and k == kw and stride[0] == stride[1] and padding[0] == padding[1]
                    and Cx.conv_fprop_supported(N, H, W, cp, Co, k, stride[0], padding[0])
                    and (cp == Ci or Cx.conv_wgrad_supported(N, H, W, cp, Co, k, stride[0], padding[0]))):
                sums = core.zero_scratch(2 * Co, x.device)
        y = _Conv2dShadowFn.apply(x, weight, stride, padding, dilation, int(groups), sums)
        if sums is not None:
            y._fb_bn_sums = sums.view(2, -1)
        return y if bias is None else y + bias.to(y.dtype).view(1, -1, 1, 1)
    if x.dim() == 4 and x.is_cuda and x.is_contiguous(memory_format=torch.channels_last) and not x.is_contiguous():
        # channels-last activations: hand the filter over in the matching (KRSC) layout in the same
        # cast, so the library convolution runs its NHWC tensor-core kernels without transposes
        w = weight.to(dtype=x.dtype, memory_format=torch.channels_last)
    else:
        w = weight if weight.dtype == x.dtype else weight.to(x.dtype)
    b = None if bias is None else (bias if bias.dtype == x.dtype else bias.to(x.dtype))
    return F.conv2d(x, w, b, stride, padding, dilation, groups)
