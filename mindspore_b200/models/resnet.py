"""ResNet-50 v1.5 (stride 2 on the 3x3 convolution of the down-sampling bottlenecks) for ImageNet-shaped input.

Every Conv2d -> BatchNorm2d -> (+ shortcut) -> ReLU group is one ``ConvBnAct`` cell.  On CUDA in bf16 it runs the
fused kernel unit (implicit-GEMM convolution with the BatchNorm statistics in its epilogue, one elementwise pass for
normalise + add + ReLU); elsewhere it composes nn.Conv2d and nn.BatchNorm2d.  Same architecture and initialisation
as the reference's test network (tests/st/networks/models/resnet50/src/resnet.py)."""
from __future__ import annotations

import math

import torch

from .. import nn
from ..common.initializer import HeNormal, initializer
from ..common.parameter import Parameter
from ..ops import conv_kernel
from ..ops.primitive import _wrap_out


class ConvBnAct(nn.Cell):
    def __init__(self, cin, cout, kernel, stride=1, relu=True, zero_gamma=False, dtype=torch.float32):
        super().__init__()
        self.stride, self.pad, self.relu = stride, kernel // 2, relu
        self.conv = nn.Conv2d(cin, cout, kernel, stride, pad_mode="pad", padding=kernel // 2,
                              weight_init=HeNormal(mode="fan_out", nonlinearity="relu"), dtype=dtype)
        self.bn = nn.BatchNorm2d(cout, eps=1e-5, momentum=0.9, gamma_init="zeros" if zero_gamma else "ones")
        if dtype != torch.float32:
            # trainable affine parameters share the weights' dtype (one flat optimizer arena with fp32 masters);
            # the moving statistics stay fp32
            for p in (self.bn.gamma, self.bn.beta):
                p.set_data(p.detach().to(dtype))

    def construct(self, x, residual=None):
        w = self.conv.weight
        if self.training and x.is_cuda and x.dtype == torch.bfloat16 and conv_kernel.available() \
                and w.shape[0] % 64 == 0:
            bn = self.bn
            y = conv_kernel.conv_bn_act(x.as_subclass(torch.Tensor), w, bn.gamma, bn.beta,
                                        bn.moving_mean.detach().as_subclass(torch.Tensor),
                                        bn.moving_variance.detach().as_subclass(torch.Tensor), self.stride, self.pad,
                                        self.relu, residual, bn.eps, bn.momentum)
            return _wrap_out(y)
        y = self.bn(self.conv(x))
        if residual is not None:
            y = y + residual
        return _wrap_out(torch.relu(y) if self.relu else y)


class Bottleneck(nn.Cell):
    expansion = 4

    def __init__(self, cin, width, stride, dtype):
        super().__init__()
        cout = width * self.expansion
        self.conv1 = ConvBnAct(cin, width, 1, 1, dtype=dtype)
        self.conv2 = ConvBnAct(width, width, 3, stride, dtype=dtype)
        self.conv3 = ConvBnAct(width, cout, 1, 1, relu=True, zero_gamma=True, dtype=dtype)   # ReLU after the add
        self.down = ConvBnAct(cin, cout, 1, stride, relu=False, dtype=dtype) if stride != 1 or cin != cout else None

    def construct(self, x):
        shortcut = self.down(x) if self.down is not None else x
        return self.conv3(self.conv2(self.conv1(x)), shortcut)


class ResNet(nn.Cell):
    def __init__(self, layers=(3, 4, 6, 3), num_classes=1000, dtype=torch.float32):
        super().__init__()
        self.stem = ConvBnAct(3, 64, 7, 2, dtype=dtype)
        blocks, cin = [], 64
        for i, (n, width) in enumerate(zip(layers, (64, 128, 256, 512))):
            for j in range(n):
                blocks.append(Bottleneck(cin, width, (1 if i == 0 else 2) if j == 0 else 1, dtype))
                cin = width * Bottleneck.expansion
        self.blocks = nn.CellList(blocks)
        self.fc = nn.Dense(cin, num_classes, dtype=dtype)
        self.num_classes = num_classes

    def construct(self, x):
        x = self.stem(x)
        if x.is_cuda and x.dtype == torch.bfloat16 and conv_kernel.available():
            x = conv_kernel.maxpool3x3s2(x.as_subclass(torch.Tensor))
        else:
            x = torch.nn.functional.max_pool2d(x, 3, 2, 1)
        for b in self.blocks:
            x = b(x)
        if x.is_cuda and x.dtype == torch.bfloat16 and conv_kernel.available():
            x = conv_kernel.global_avgpool(x.as_subclass(torch.Tensor))
        else:
            x = x.mean((2, 3))
        return self.fc(_wrap_out(x))


def resnet50(num_classes=1000, dtype=torch.float32):
    return ResNet((3, 4, 6, 3), num_classes, dtype)


class ResNetWithLoss(nn.Cell):
    """images [N, 3, H, W], labels [N] -> label-smoothed cross entropy."""

    def __init__(self, net, smoothing=0.1):
        super().__init__()
        self.net, self.smoothing = net, smoothing

    def construct(self, images, labels):
        logits = self.net(images).float()
        return _wrap_out(torch.nn.functional.cross_entropy(logits, labels.long(), label_smoothing=self.smoothing))


def flops_per_image(num_classes=1000):
    """Forward multiply-add FLOPs x2 of ResNet-50 at 224 x 224 (convolutions + classifier)."""
    total, size, cin = 2 * 112 * 112 * 64 * 147, 56, 64
    for i, (n, width) in enumerate(zip((3, 4, 6, 3), (64, 128, 256, 512))):
        for j in range(n):
            stride = (1 if i == 0 else 2) if j == 0 else 1
            out = size // stride
            total += 2 * size * size * cin * width + 2 * out * out * width * width * 9 + 2 * out * out * width * width * 4
            if stride != 1 or cin != width * 4:
                total += 2 * out * out * cin * width * 4
            size, cin = out, width * 4
    return total + 2 * cin * num_classes
