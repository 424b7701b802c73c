"""CIFAR-style ResNet-20 (ddp-bench/src/models/resnet.rs:209-301): 3x3 stem (3->16) + BN + ReLU,
three stages of three BasicBlocks (16/32/64 channels, stride 2 + 1x1 projection shortcut at the
start of stages 2 and 3), global average pool, 10-way Linear. Convolutions have no bias.

On CUDA each BN runs this library's fused kernel: BN+ReLU after the first conv of a block and
BN + shortcut add + ReLU after the second, so a block is conv, bn_relu, conv, bn_add_relu."""
from __future__ import annotations

from typing import List

import torch

from ..autograd import Variable
from ..nn.layers import AdaptiveAvgPool2d, BatchNorm2d, Conv2d, Linear
from ..nn.module import Module


class BasicBlock(Module):
    def __init__(self, in_c: int, out_c: int, stride: int, device=None):
        self.conv1 = Conv2d(in_c, out_c, 3, stride, 1, bias=False, device=device)
        self.bn1 = BatchNorm2d(out_c, device)
        self.conv2 = Conv2d(out_c, out_c, 3, 1, 1, bias=False, device=device)
        self.bn2 = BatchNorm2d(out_c, device)
        self.down_conv = self.down_bn = None
        if stride != 1 or in_c != out_c:
            self.down_conv = Conv2d(in_c, out_c, 1, stride, 0, bias=False, device=device)
            self.down_bn = BatchNorm2d(out_c, device)
        # every convolution here feeds a BatchNorm directly: let its epilogue accumulate the statistics
        for conv in (self.conv1, self.conv2, self.down_conv):
            if conv is not None:
                conv.bn_stats = True

    def name(self): return "basic_block"

    def sub_modules(self) -> List[Module]:
        mods = [self.conv1, self.bn1, self.conv2, self.bn2]
        if self.down_conv is not None:
            mods += [self.down_conv, self.down_bn]
        return mods

    def forward(self, x: Variable) -> Variable:
        sc = x if self.down_conv is None else self.down_bn.forward(self.down_conv.forward(x), relu=False)
        h = self.bn1.forward(self.conv1.forward(x), relu=True)
        return self.bn2.forward(self.conv2.forward(h), residual=sc, relu=True)


class ResNet20(Module):
    def __init__(self, num_classes: int = 10, device=None):
        self.stem = Conv2d(3, 16, 3, 1, 1, bias=False, device=device)
        self.stem_bn = BatchNorm2d(16, device)
        self.stem.bn_stats = True
        self.blocks: List[BasicBlock] = []
        in_c = 16
        for out_c, stride in ((16, 1), (32, 2), (64, 2)):
            for i in range(3):
                self.blocks.append(BasicBlock(in_c, out_c, stride if i == 0 else 1, device))
                in_c = out_c
        self.pool = AdaptiveAvgPool2d(1)
        self.fc = Linear(64, num_classes, True, device)

    def name(self): return "resnet20"
    def sub_modules(self): return [self.stem, self.stem_bn, *self.blocks, self.pool, self.fc]

    def forward(self, x: Variable) -> Variable:
        if x.t.is_cuda and x.t.dim() == 4:
            # channels-last from the stem on: convolutions and the fused BatchNorm kernels both work on
            # N-H-W-C, so no layer pays for a layout transpose
            x = Variable.wrap(x.t.contiguous(memory_format=torch.channels_last))
        h = self.stem_bn.forward(self.stem.forward(x), relu=True)
        for b in self.blocks:
            h = b.forward(h)
        return self.fc.forward(self.pool.forward(h).flatten(1))


def resnet20(num_classes: int = 10, device=None) -> ResNet20:
    return ResNet20(num_classes, device)
