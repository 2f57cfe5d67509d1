"""Bijectors: ``forward``, ``inverse``, ``forward_log_jacobian``, ``inverse_log_jacobian``."""
from __future__ import annotations

import torch
import torch.distributions as D

from ...ops.primitive import _wrap_out
from ..cell import Cell

__all__ = ["Bijector", "Exp", "Softplus", "ScalarAffine", "PowerTransform", "GumbelCDF", "Invert"]


def _t(x):
    return x.float() if isinstance(x, torch.Tensor) else torch.as_tensor(x, dtype=torch.float32)


class Bijector(Cell):
    is_linear = False

    def __init__(self, is_constant_jacobian=False, is_injective=True, name=None, dtype=None, param=None):
        super().__init__()
        self.name = name or type(self).__name__
        self.is_constant_jacobian, self.is_injective = is_constant_jacobian, is_injective

    def _transform(self):
        raise NotImplementedError

    def forward(self, x):
        return _wrap_out(self._transform()(_t(x)))

    def inverse(self, y):
        return _wrap_out(self._transform().inv(_t(y)))

    def forward_log_jacobian(self, x):
        t = self._transform()
        x = _t(x)
        return _wrap_out(t.log_abs_det_jacobian(x, t(x)))

    def inverse_log_jacobian(self, y):
        t = self._transform()
        y = _t(y)
        return _wrap_out(-t.log_abs_det_jacobian(t.inv(y), y))

    def construct(self, name, *args, **kwargs):
        return getattr(self, name)(*args, **kwargs)


class Exp(Bijector):
    def _transform(self):
        return D.ExpTransform()


class Softplus(Bijector):
    def __init__(self, sharpness=1.0, name="Softplus"):
        super().__init__(name=name)
        self.sharpness = float(sharpness)

    def _transform(self):
        k = self.sharpness
        return D.ComposeTransform([D.AffineTransform(0.0, k), D.SoftplusTransform(), D.AffineTransform(0.0, 1.0 / k)])


class ScalarAffine(Bijector):
    is_linear = True

    def __init__(self, scale=1.0, shift=0.0, name="ScalarAffine"):
        super().__init__(is_constant_jacobian=True, name=name)
        self.scale, self.shift = scale, shift

    def _transform(self):
        return D.AffineTransform(_t(self.shift), _t(self.scale))


class PowerTransform(Bijector):
    """y = (1 + x * power) ** (1 / power); ``power = 0`` is ``exp``."""

    def __init__(self, power=0.0, name="PowerTransform"):
        super().__init__(name=name)
        if power < 0:
            raise ValueError("power must be non-negative, got %r" % (power,))
        self.power = float(power)

    def _transform(self):
        if self.power == 0:
            return D.ExpTransform()
        return D.ComposeTransform([D.AffineTransform(1.0, self.power), D.PowerTransform(1.0 / self.power)])


class GumbelCDF(Bijector):
    def __init__(self, loc=0.0, scale=1.0, name="GumbelCDF"):
        super().__init__(name=name)
        self.loc, self.scale = loc, scale

    def forward(self, x):
        return _wrap_out(torch.exp(-torch.exp(-(_t(x) - _t(self.loc)) / _t(self.scale))))

    def inverse(self, y):
        return _wrap_out(_t(self.loc) - _t(self.scale) * torch.log(-torch.log(_t(y))))

    def forward_log_jacobian(self, x):
        z = (_t(x) - _t(self.loc)) / _t(self.scale)
        return _wrap_out(-z - torch.exp(-z) - torch.log(_t(self.scale)))

    def inverse_log_jacobian(self, y):
        return _wrap_out(-self.forward_log_jacobian(self.inverse(y)))


class Invert(Bijector):
    def __init__(self, bijector, name=""):
        super().__init__(name=name or "Invert" + bijector.name)
        self.bijector = bijector

    def _transform(self):
        return self.bijector._transform().inv

    def forward(self, x):
        return self.bijector.inverse(x)

    def inverse(self, y):
        return self.bijector.forward(y)

    def forward_log_jacobian(self, x):
        return self.bijector.inverse_log_jacobian(x)

    def inverse_log_jacobian(self, y):
        return self.bijector.forward_log_jacobian(y)
