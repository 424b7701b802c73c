"""conv2d dispatch. The native implicit-GEMM kernel covers the NCHW bf16 shapes of the CIFAR
ResNet (3x3 / 1x1, stride 1 or 2, groups 1); everything else runs the PyTorch op."""
from __future__ import annotations

import torch
import torch.nn.functional as F

from .. import _ext
from . import core


def conv2d(x, weight, bias=None, stride=(1, 1), padding=(0, 0), dilation=(1, 1), groups=1):
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
