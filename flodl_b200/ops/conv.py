"""conv2d dispatch. The native implicit-GEMM kernel covers the NCHW bf16 shapes of the CIFAR
ResNet (3x3 / 1x1, stride 1 or 2, groups 1); everything else runs the PyTorch op."""
from __future__ import annotations

import torch
import torch.nn.functional as F

from .. import _ext
from . import core


def _pair(v):
    return (int(v), int(v)) if isinstance(v, int) else tuple(int(a) for a in v)


class _Conv2dShadowFn(torch.autograd.Function):
    """Convolution on channels-last bf16 activations whose filter lives in a flat parameter buffer:
    forward reads the bf16 shadow of the filter (already K-R-S-C, refreshed by the optimizer kernel),
    backward adds the filter gradient straight into the fp32 gradient slot. Compared with
    `weight.to(bf16)` under autograd this drops one cast per forward and the cast + layout change +
    accumulate chain per backward."""

    @staticmethod
    def forward(ctx, x, weight, stride, padding, dilation, groups):
        w16 = weight._fb_bf16
        ctx.save_for_backward(x, w16)
        ctx.weight, ctx.conf = weight, (stride, padding, dilation, groups)
        core._launched()
        return F.conv2d(x, w16, None, stride, padding, dilation, groups)

    @staticmethod
    def backward(ctx, dy):
        x, w16 = ctx.saved_tensors
        stride, padding, dilation, groups = ctx.conf
        dy = dy.contiguous(memory_format=torch.channels_last)
        C = _ext.require()
        N, Ci, H, W = x.shape
        Co, _, k, _ = w16.shape
        native = (dilation == (1, 1) and groups == 1 and stride[0] == stride[1] and padding[0] == padding[1]
                  and C.conv_wgrad_supported(N, H, W, Ci, Co, k, stride[0], padding[0]))
        dx, dw, _ = torch.ops.aten.convolution_backward(dy, x, w16, None, list(stride), list(padding), list(dilation), False, [0, 0], groups,
                                                        [ctx.needs_input_grad[0], not native, False])
        core._launched(2)
        if native:
            # filter gradient on the tensor cores, accumulated into the fp32 slot in place
            C.conv_wgrad(x, dy, ctx.weight._fb_grad, stride[0], padding[0])
        else:
            ctx.weight._fb_grad.add_(dw)
        core._touched(ctx.weight)
        return dx, None, None, None, None, None


def conv2d(x, weight, bias=None, stride=(1, 1), padding=(0, 0), dilation=(1, 1), groups=1):
    if (x.dim() == 4 and x.is_cuda and core.FLAGS.native and x.dtype == torch.bfloat16 and getattr(weight, "_fb_bf16", None) is not None
            and getattr(weight, "_fb_channels_last", False) and x.is_contiguous(memory_format=torch.channels_last)):
        y = _Conv2dShadowFn.apply(x, weight, _pair(stride), _pair(padding), _pair(dilation), int(groups))
        return y if bias is None else y + bias.to(y.dtype).view(1, -1, 1, 1)
    C = _ext.load() if x.is_cuda else None
    if C is not None and core.FLAGS.native and hasattr(C, "conv2d_fwd"):
        from . import conv_native
        if conv_native.eligible(x, weight, stride, padding, dilation, groups):
            return conv_native.conv2d(x, weight, bias, stride, padding)
    if x.dim() == 4 and x.is_cuda and x.is_contiguous(memory_format=torch.channels_last) and not x.is_contiguous():
        # channels-last activations: hand the filter over in the matching (KRSC) layout in the same
        # cast, so the library convolution runs its NHWC tensor-core kernels without transposes
        w = weight.to(dtype=x.dtype, memory_format=torch.channels_last)
    else:
        w = weight if weight.dtype == x.dtype else weight.to(x.dtype)
    b = None if bias is None else (bias if bias.dtype == x.dtype else bias.to(x.dtype))
    return F.conv2d(x, w, b, stride, padding, dilation, groups)
