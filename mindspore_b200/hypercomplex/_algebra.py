"""Layers over two-component number systems.

A tensor of such numbers is stored with the two components stacked in front: shape ``[2, N, ...]`` (``x[0]`` the real
part, ``x[1]`` the second component).  The three algebras differ only in the square of the second unit ``u``:
complex ``u^2 = -1``, dual ``u^2 = 0``, double (hyperbolic) ``u^2 = +1``.  A linear map with weight ``W = Wx + u Wy``
applied to ``x + u y`` is therefore ``(x Wx + s y Wy) + u (x Wy + y Wx)`` with ``s = u^2`` - four real products, here
evaluated as two (the two weights are concatenated along the output dimension).

Parity: python/mindspore/hypercomplex/hypercomplex/hc_dense.py, hc_conv.py, hc_bn.py, hc_pool.py and the
complex / dual / double sub-packages that instantiate them."""
from __future__ import annotations

import torch
import torch.nn.functional as F

from ..common.initializer import initializer
from ..common.parameter import Parameter
from ..common.tensor import as_tensor
from ..nn.cell import Cell


def _plain(t):
    return t.as_subclass(torch.Tensor) if isinstance(t, torch.Tensor) else torch.as_tensor(t)


def _check2(x, who):
    if x.dim() < 2 or x.shape[0] != 2:
        raise ValueError("For '%s', the first dimension of the input must hold the 2 components, but got shape %s"
                         % (who, tuple(x.shape)))


class _Linear(Cell):
    """Shared by Dense and ConvNd: ``op(x, w, b)`` is the real linear operator."""
    square = -1.0

    def _mix(self, x, op):
        xr, xi = x[0], x[1]
        wx, wy = _plain(self.weight_x), _plain(self.weight_y)
        both = torch.cat([wx, wy], 0)                       # one product per input component
        n = wx.shape[0]
        pr, pi = op(xr, both), op(xi, both)
        a, b = pr.split(n, dim=self._channel_dim)           # xr Wx, xr Wy
        c, d = pi.split(n, dim=self._channel_dim)           # xi Wx, xi Wy
        real = a + self.square * d if self.square else a
        imag = b + c
        if self.bias_x is not None:
            shape = [1] * real.dim()
            shape[self._channel_dim] = -1
            real = real + _plain(self.bias_x).reshape(shape)
            imag = imag + _plain(self.bias_y).reshape(shape)
        return as_tensor(torch.stack([real, imag]))


class Dense(_Linear):
    _channel_dim = -1

    def __init__(self, in_channels, out_channels, weight_init="normal", bias_init="zeros", has_bias=True):
        super().__init__()
        if in_channels <= 0 or out_channels <= 0:
            raise ValueError("For 'Dense', in_channels and out_channels must be positive")
        self.in_channels, self.out_channels, self.has_bias = in_channels, out_channels, has_bias
        self.weight_x = Parameter(initializer(weight_init, (out_channels, in_channels), torch.float32), name="weight_x")
        self.weight_y = Parameter(initializer(weight_init, (out_channels, in_channels), torch.float32), name="weight_y")
        self.bias_x = Parameter(initializer(bias_init, (out_channels,), torch.float32), name="bias_x") \
            if has_bias else None
        self.bias_y = Parameter(initializer(bias_init, (out_channels,), torch.float32), name="bias_y") \
            if has_bias else None

    def construct(self, u):
        x = _plain(u)
        _check2(x, "Dense")
        return self._mix(x, lambda t, w: F.linear(t, w))


class _ConvNd(_Linear):
    _channel_dim = 1
    _nd = 2

    def __init__(self, in_channels, out_channels, kernel_size, stride=1, pad_mode="same", padding=0, dilation=1,
                 group=1, has_bias=False, weight_init="normal", bias_init="zeros"):
        super().__init__()
        tup = lambda v: tuple(v) if isinstance(v, (tuple, list)) else (v,) * self._nd
        self.kernel_size, self.stride, self.dilation = tup(kernel_size), tup(stride), tup(dilation)
        if pad_mode not in ("same", "valid", "pad"):
            raise ValueError("pad_mode must be 'same', 'valid' or 'pad', but got %r" % (pad_mode,))
        self.pad_mode, self.padding, self.group = pad_mode, tup(padding), group
        shape = (out_channels, in_channels // group) + self.kernel_size
        self.weight_x = Parameter(initializer(weight_init, shape, torch.float32), name="weight_x")
        self.weight_y = Parameter(initializer(weight_init, shape, torch.float32), name="weight_y")
        self.bias_x = Parameter(initializer(bias_init, (out_channels,), torch.float32), name="bias_x") \
            if has_bias else None
        self.bias_y = Parameter(initializer(bias_init, (out_channels,), torch.float32), name="bias_y") \
            if has_bias else None

    def _op(self, t, w):
        fn = (F.conv1d, F.conv2d, F.conv3d)[self._nd - 1]
        if self.pad_mode == "same":
            if any(s != 1 for s in self.stride):
                pads = []
                for size, k, s, d in zip(t.shape[2:][::-1], self.kernel_size[::-1], self.stride[::-1],
                                         self.dilation[::-1]):
                    total = max((-(-size // s) - 1) * s + (k - 1) * d + 1 - size, 0)
                    pads += [total // 2, total - total // 2]
                return fn(F.pad(t, pads), w, None, self.stride, 0, self.dilation, self.group)
            return fn(t, w, None, 1, "same", self.dilation, self.group)
        pad = 0 if self.pad_mode == "valid" else self.padding
        return fn(t, w, None, self.stride, pad, self.dilation, self.group)

    def construct(self, u):
        x = _plain(u)
        _check2(x, type(self).__name__)
        return self._mix(x, self._op)


class Conv1d(_ConvNd):
    _nd = 1


class Conv2d(_ConvNd):
    _nd = 2


class Conv3d(_ConvNd):
    _nd = 3


class _BatchNorm(Cell):
    """Each component is normalised with its own statistics and affine parameters (the component-wise variant of the
    reference's layers)."""
    _nd = 2

    def __init__(self, num_features, eps=1e-5, momentum=0.9, affine=True, gamma_init="ones", beta_init="zeros",
                 moving_mean_init="zeros", moving_var_init="ones", use_batch_statistics=None, data_format="NCHW"):
        super().__init__()
        self.eps, self.momentum, self.use_batch_statistics = eps, momentum, use_batch_statistics
        mk = lambda init, name, grad=True: Parameter(initializer(init, (2, num_features), torch.float32), name=name,
                                                     requires_grad=grad)
        self.gamma, self.beta = mk(gamma_init, "gamma", affine), mk(beta_init, "beta", affine)
        self.moving_mean = mk(moving_mean_init, "moving_mean", False)
        self.moving_variance = mk(moving_var_init, "moving_variance", False)

    def construct(self, u):
        x = _plain(u)
        _check2(x, type(self).__name__)
        train = self.training if self.use_batch_statistics is None else bool(self.use_batch_statistics)
        outs = []
        for c in range(2):
            outs.append(F.batch_norm(x[c], _plain(self.moving_mean)[c], _plain(self.moving_variance)[c],
                                     _plain(self.gamma)[c], _plain(self.beta)[c], train, 1.0 - self.momentum,
                                     self.eps))
        return as_tensor(torch.stack(outs))


class BatchNorm1d(_BatchNorm):
    _nd = 1


class BatchNorm2d(_BatchNorm):
    _nd = 2


class BatchNorm3d(_BatchNorm):
    _nd = 3


class ReLU(Cell):
    """max(0, .) on both components."""

    def construct(self, u):
        return as_tensor(torch.relu(_plain(u)))


def _pool(name, fn):
    class _Pool(Cell):
        def __init__(self, *args, **kwargs):
            super().__init__()
            self.args, self.kwargs = args, kwargs

        def construct(self, u):
            x = _plain(u)
            _check2(x, name)
            return as_tensor(torch.stack([fn(x[0], *self.args, **self.kwargs), fn(x[1], *self.args, **self.kwargs)]))
    _Pool.__name__ = _Pool.__qualname__ = name
    return _Pool


MaxPool1d = _pool("MaxPool1d", lambda t, kernel_size=1, stride=1, **k: F.max_pool1d(t, kernel_size, stride))
MaxPool2d = _pool("MaxPool2d", lambda t, kernel_size=1, stride=1, **k: F.max_pool2d(t, kernel_size, stride))
AvgPool1d = _pool("AvgPool1d", lambda t, kernel_size=1, stride=1, **k: F.avg_pool1d(t, kernel_size, stride))
AvgPool2d = _pool("AvgPool2d", lambda t, kernel_size=1, stride=1, **k: F.avg_pool2d(t, kernel_size, stride))
AdaptiveAvgPool1d = _pool("AdaptiveAvgPool1d", lambda t, output_size: F.adaptive_avg_pool1d(t, output_size))
AdaptiveAvgPool2d = _pool("AdaptiveAvgPool2d", lambda t, output_size: F.adaptive_avg_pool2d(t, output_size))
AdaptiveAvgPool3d = _pool("AdaptiveAvgPool3d", lambda t, output_size: F.adaptive_avg_pool3d(t, output_size))
AdaptiveMaxPool1d = _pool("AdaptiveMaxPool1d", lambda t, output_size: F.adaptive_max_pool1d(t, output_size))
AdaptiveMaxPool2d = _pool("AdaptiveMaxPool2d", lambda t, output_size: F.adaptive_max_pool2d(t, output_size))

_NAMES = ["Dense", "Conv1d", "Conv2d", "Conv3d", "BatchNorm1d", "BatchNorm2d", "BatchNorm3d", "ReLU", "MaxPool1d",
          "MaxPool2d", "AvgPool1d", "AvgPool2d", "AdaptiveAvgPool1d", "AdaptiveAvgPool2d", "AdaptiveAvgPool3d",
          "AdaptiveMaxPool1d", "AdaptiveMaxPool2d"]


def make_namespace(square):
    """The layer classes of one algebra (``square`` = the second unit squared)."""
    ns = {}
    for n in _NAMES:
        base = globals()[n]
        ns[n] = type(n, (base,), {"square": float(square), "__doc__": base.__doc__}) if issubclass(base, _Linear) \
            else base
    return ns
