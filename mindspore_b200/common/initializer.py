"""Weight initializers.

Parity: mindspore/python/mindspore/common/initializer.py (Initializer base, Zero, One, Constant,
Uniform, Normal, TruncatedNormal, HeUniform/HeNormal, XavierUniform/XavierNormal, Orthogonal,
Identity, Dirac, Sparse, VarianceScaling and the string aliases accepted by ``initializer()``).
"""
from __future__ import annotations

import math
import numbers

import numpy as np
import torch

from . import dtype as mstype


def _fans(shape):
    if len(shape) == 0:
        return 1, 1
    if len(shape) == 1:
        return shape[0], shape[0]
    if len(shape) == 2:
        return shape[1], shape[0]
    rf = 1
    for s in shape[2:]:
        rf *= s
    return shape[1] * rf, shape[0] * rf


def _gain(nonlinearity, negative_slope=None):
    if nonlinearity in ("linear", "conv1d", "conv2d", "conv3d", "sigmoid"):
        return 1.0
    if nonlinearity == "tanh":
        return 5.0 / 3
    if nonlinearity == "relu":
        return math.sqrt(2.0)
    if nonlinearity == "leaky_relu":
        ns = 0.01 if negative_slope is None else negative_slope
        return math.sqrt(2.0 / (1 + ns ** 2))
    raise ValueError("Unsupported nonlinearity %r" % nonlinearity)


class Initializer:
    def __init__(self, **kwargs):
        self._kwargs = kwargs
        self._seed = None

    def _initialize(self, t):  # fills torch tensor t in place
        raise NotImplementedError

    def __call__(self, t):
        with torch.no_grad():
            self._initialize(t)
        return t


class Zero(Initializer):
    def _initialize(self, t):
        t.zero_()


class One(Initializer):
    def _initialize(self, t):
        t.fill_(1)


class Constant(Initializer):
    def __init__(self, value):
        super().__init__(value=value)
        self.value = value

    def _initialize(self, t):
        if isinstance(self.value, (np.ndarray, torch.Tensor)):
            t.copy_(torch.as_tensor(np.asarray(self.value) if isinstance(self.value, np.ndarray) else self.value)
                    .to(t.dtype).reshape(t.shape))
        else:
            t.fill_(self.value)


class Uniform(Initializer):
    def __init__(self, scale=0.07):
        super().__init__(scale=scale)
        self.scale = scale

    def _initialize(self, t):
        t.uniform_(-self.scale, self.scale)


class Normal(Initializer):
    def __init__(self, sigma=0.01, mean=0.0):
        super().__init__(sigma=sigma, mean=mean)
        self.sigma, self.mean = sigma, mean

    def _initialize(self, t):
        t.normal_(self.mean, self.sigma)


class TruncatedNormal(Initializer):
    def __init__(self, sigma=0.01, mean=0.0, a=-2.0, b=2.0):
        super().__init__(sigma=sigma)
        self.sigma, self.mean, self.a, self.b = sigma, mean, a, b

    def _initialize(self, t):
        torch.nn.init.trunc_normal_(t, self.mean, self.sigma, self.mean + self.a * self.sigma,
                                    self.mean + self.b * self.sigma)


class HeUniform(Initializer):
    def __init__(self, negative_slope=0, mode="fan_in", nonlinearity="leaky_relu"):
        super().__init__()
        self.negative_slope, self.mode, self.nonlinearity = negative_slope, mode, nonlinearity

    def _initialize(self, t):
        fan_in, fan_out = _fans(tuple(t.shape))
        fan = fan_in if self.mode == "fan_in" else fan_out
        bound = math.sqrt(3.0) * _gain(self.nonlinearity, self.negative_slope) / math.sqrt(fan)
        t.uniform_(-bound, bound)


class HeNormal(HeUniform):
    def _initialize(self, t):
        fan_in, fan_out = _fans(tuple(t.shape))
        fan = fan_in if self.mode == "fan_in" else fan_out
        t.normal_(0, _gain(self.nonlinearity, self.negative_slope) / math.sqrt(fan))


class XavierUniform(Initializer):
    def __init__(self, gain=1):
        super().__init__(gain=gain)
        self.gain = gain

    def _initialize(self, t):
        fan_in, fan_out = _fans(tuple(t.shape))
        bound = self.gain * math.sqrt(6.0 / (fan_in + fan_out))
        t.uniform_(-bound, bound)


class XavierNormal(XavierUniform):
    def _initialize(self, t):
        fan_in, fan_out = _fans(tuple(t.shape))
        t.normal_(0, self.gain * math.sqrt(2.0 / (fan_in + fan_out)))


class Orthogonal(Initializer):
    def __init__(self, gain=1.0):
        super().__init__(gain=gain)
        self.gain = gain

    def _initialize(self, t):
        tmp = torch.empty(t.shape, dtype=torch.float32)
        torch.nn.init.orthogonal_(tmp, self.gain)
        t.copy_(tmp.to(t.dtype))


class Identity(Initializer):
    def _initialize(self, t):
        if t.dim() != 2:
            raise ValueError("For Identity initializer, the dimension of the initialized tensor should be 2")
        t.copy_(torch.eye(t.shape[0], t.shape[1], dtype=t.dtype))


class Dirac(Initializer):
    def __init__(self, groups=1):
        super().__init__(groups=groups)
        self.groups = groups

    def _initialize(self, t):
        tmp = torch.empty(t.shape, dtype=torch.float32)
        torch.nn.init.dirac_(tmp, self.groups)
        t.copy_(tmp.to(t.dtype))


class Sparse(Initializer):
    def __init__(self, sparsity, sigma=0.01):
        super().__init__()
        self.sparsity, self.sigma = sparsity, sigma

    def _initialize(self, t):
        tmp = torch.empty(t.shape, dtype=torch.float32)
        torch.nn.init.sparse_(tmp, self.sparsity, self.sigma)
        t.copy_(tmp.to(t.dtype))


class VarianceScaling(Initializer):
    def __init__(self, scale=1.0, mode="fan_in", distribution="truncated_normal"):
        super().__init__()
        self.scale, self.mode, self.distribution = scale, mode, distribution

    def _initialize(self, t):
        fan_in, fan_out = _fans(tuple(t.shape))
        n = {"fan_in": fan_in, "fan_out": fan_out, "fan_avg": (fan_in + fan_out) / 2}[self.mode]
        s = self.scale / max(1.0, n)
        if self.distribution == "truncated_normal":
            std = math.sqrt(s) / 0.87962566103423978
            torch.nn.init.trunc_normal_(t, 0, std, -2 * std, 2 * std)
        elif self.distribution == "normal":
            t.normal_(0, math.sqrt(s))
        else:
            lim = math.sqrt(3 * s)
            t.uniform_(-lim, lim)


_ALIASES = {
    "zeros": Zero, "zero": Zero, "ones": One, "one": One, "uniform": Uniform, "normal": Normal,
    "truncatednormal": TruncatedNormal, "truncated_normal": TruncatedNormal, "he_uniform": HeUniform,
    "heuniform": HeUniform, "he_normal": HeNormal, "henormal": HeNormal, "xavier_uniform": XavierUniform,
    "xavieruniform": XavierUniform, "xavier_normal": XavierNormal, "xaviernormal": XavierNormal,
    "orthogonal": Orthogonal, "identity": Identity, "dirac": Dirac,
}


def _resolve(init):
    if isinstance(init, Initializer):
        return init
    if isinstance(init, str):
        cls = _ALIASES.get(init.lower())
        if cls is None:
            raise ValueError("The initializer name %r is not supported" % init)
        return cls()
    if isinstance(init, numbers.Number):
        return Constant(init)
    if isinstance(init, (np.ndarray, torch.Tensor)):
        return Constant(init)
    raise TypeError("Unsupported init type %s" % type(init))


def initializer(init, shape=None, dtype=mstype.float32):
    """Creates an initialised ``Tensor`` of ``shape``/``dtype`` (eagerly - no lazy init object)."""
    from .tensor import Tensor
    if isinstance(init, torch.Tensor) and shape is None:
        return Tensor(init, dtype=dtype)
    if shape is None:
        shape = ()
    if isinstance(shape, int):
        shape = (shape,)
    ini = _resolve(init)
    work_dtype = dtype if dtype in (torch.float32, torch.float64) or not dtype.is_floating_point else torch.float32
    from .. import context
    dev = context.device()
    n = 1
    for d in shape:
        n *= d
    if dev.type == "cuda" and n >= (1 << 20) and isinstance(ini, (Normal, Uniform, Zero, One, HeUniform, HeNormal,
                                                                   XavierUniform, XavierNormal, TruncatedNormal)):
        # large tensors are filled on the device, in the target dtype when that is exact enough (avoids a
        # multi-GB host detour for billion-parameter models)
        t = torch.empty(tuple(shape), dtype=dtype if dtype.is_floating_point else work_dtype, device=dev)
        ini(t)
        return Tensor(t.to(dtype))
    t = torch.empty(tuple(shape), dtype=work_dtype)
    ini(t)
    return Tensor(t.to(dtype))
