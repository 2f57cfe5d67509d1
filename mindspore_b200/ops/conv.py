"""Convolution / batch-norm entry points (NCHW API like the reference's Conv2D / BatchNorm primitives).

CUDA bf16 inputs go through the implicit-GEMM path in ``ops.conv_kernel`` (channels-last im2col tiles feeding
the tcgen05 GEMM, BatchNorm statistics and apply fused around it); other inputs use PyTorch.
Parity: plugin/device/gpu/kernel/nn/convolution/conv2d_cudnn_gpu_kernel.h:667-739 and
plugin/device/gpu/kernel/nn/batch_norm_gpu_kernel.cc:62-69 (cuDNN in the reference).
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F


def _pads(pad_mode, pad, x_hw, k_hw, stride, dil):
    mode = pad_mode.lower()
    if mode == "valid":
        return (0, 0, 0, 0)
    if mode == "pad":
        if isinstance(pad, int):
            return (pad, pad, pad, pad)
        pad = tuple(pad)
        return pad if len(pad) == 4 else (pad[0], pad[0], pad[1], pad[1])
    out = []
    for i in range(2):
        eff = (k_hw[i] - 1) * dil[i] + 1
        total = max((math.ceil(x_hw[i] / stride[i]) - 1) * stride[i] + eff - x_hw[i], 0)
        out += [total // 2, total - total // 2]
    return tuple(out)  # top, bottom, left, right


def conv2d(x, w, stride=(1, 1), pad_mode="valid", pad=0, dilation=(1, 1), group=1, bias=None):
    top, bottom, left, right = _pads(pad_mode, pad, x.shape[-2:], w.shape[-2:], stride, dilation)
    try:
        from . import conv_kernel
        if conv_kernel.supports(x, w, group, dilation):
            return conv_kernel.conv2d(x, w, tuple(stride), (top, bottom, left, right), dilation, bias)
    except ImportError:
        pass
    if top == bottom and left == right:
        return F.conv2d(x, w, bias, stride, (top, left), dilation, group)
    x = F.pad(x, (left, right, top, bottom))
    return F.conv2d(x, w, bias, stride, 0, dilation, group)


def batch_norm(x, scale, bias, mean, variance, training, momentum, eps):
    """Functional BN; in training mode updates ``mean``/``variance`` in place
    (moving = moving*(1-momentum) + batch*momentum, the reference's BatchNorm primitive convention)."""
    if training and x.is_cuda and x.dtype == torch.bfloat16 and x.dim() == 4 and x.shape[1] % 8 == 0 \
            and x.shape[1] <= 2048 and mean.dtype == torch.float32:
        from . import conv_kernel
        if conv_kernel.available():
            return conv_kernel.batch_norm_train(x, scale, bias, mean, variance, 1.0 - momentum, eps)
    if training:
        return F.batch_norm(x, mean, variance, scale, bias, True, momentum, eps)
    return F.batch_norm(x, mean, variance, scale, bias, False, 0.0, eps)
