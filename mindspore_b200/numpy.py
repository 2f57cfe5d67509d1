"""``mindspore_b200.numpy``: NumPy-style array functions on framework tensors
(python/mindspore/numpy/{array_creations,array_ops,math_ops,logic_ops}.py)."""
from __future__ import annotations

import builtins

import numpy as _np
import torch

from .common.tensor import as_tensor as _T

float32, float16, float64, int32, int64, int8, uint8, bool_ = (torch.float32, torch.float16, torch.float64,
                                                                torch.int32, torch.int64, torch.int8, torch.uint8,
                                                                torch.bool)
pi, e, inf, nan = _np.pi, _np.e, _np.inf, _np.nan


def _t(x, dtype=None):
    if isinstance(x, torch.Tensor):
        return x if dtype is None else x.to(dtype)
    return torch.as_tensor(_np.asarray(x), dtype=dtype) if not isinstance(x, (int, float, bool)) else \
        torch.tensor(x, dtype=dtype)


def array(obj, dtype=None, copy=True, ndmin=0):
    t = _t(obj, dtype)
    if copy and isinstance(obj, torch.Tensor):
        t = t.clone()
    while t.dim() < ndmin:
        t = t.unsqueeze(0)
    return _T(t)


asarray = asfarray = array


def zeros(shape, dtype=torch.float32):
    return _T(torch.zeros(shape, dtype=dtype))


def ones(shape, dtype=torch.float32):
    return _T(torch.ones(shape, dtype=dtype))


def full(shape, fill_value, dtype=None):
    return _T(torch.full(shape if isinstance(shape, (tuple, list)) else (shape,), fill_value, dtype=dtype))


def empty(shape, dtype=torch.float32):
    return _T(torch.empty(shape, dtype=dtype))


def eye(N, M=None, k=0, dtype=torch.float32):
    m = torch.eye(N, M if M is not None else N, dtype=dtype)
    return _T(torch.roll(m, k, 1) * (torch.ones_like(m).triu(k) if k >= 0 else torch.ones_like(m).tril(k))) if k \
        else _T(m)


def arange(start, stop=None, step=1, dtype=None):
    return _T(torch.arange(start, stop, step, dtype=dtype) if stop is not None else torch.arange(start, dtype=dtype))


def linspace(start, stop, num=50, endpoint=True, dtype=None):
    return _T(torch.from_numpy(_np.linspace(start, stop, num, endpoint=endpoint)).to(dtype or torch.float32))


def _unary(name):
    fn = getattr(torch, name)
    return lambda x, dtype=None: _T(fn(_t(x)) if dtype is None else fn(_t(x)).to(dtype))


for _n in ("abs exp log sqrt sin cos tan tanh sinh cosh floor ceil sign square negative reciprocal log2 log10 log1p "
           "expm1 arcsin arccos arctan isnan isinf isfinite trunc").split():
    globals()[_n] = _unary(_n)
absolute = abs  # noqa: A001


def _binary(name):
    fn = getattr(torch, name)
    return lambda a, b, dtype=None: _T(fn(_t(a), _t(b)))


for _n, _tn in (("add", "add"), ("subtract", "sub"), ("multiply", "mul"), ("divide", "div"), ("power", "pow"),
                ("maximum", "maximum"), ("minimum", "minimum"), ("matmul", "matmul"), ("dot", "matmul"),
                ("equal", "eq"), ("not_equal", "ne"), ("greater", "gt"), ("greater_equal", "ge"), ("less", "lt"),
                ("less_equal", "le"), ("logical_and", "logical_and"), ("logical_or", "logical_or"),
                ("floor_divide", "floor_divide"), ("remainder", "remainder"), ("arctan2", "atan2")):
    globals()[_n] = _binary(_tn)
true_divide = divide  # noqa: F821


def _reduce(name):
    fn = getattr(torch, name)

    def f(a, axis=None, dtype=None, keepdims=False):
        t = _t(a)
        if axis is None:
            out = fn(t)
            return _T(out.reshape([1] * t.dim()) if keepdims else out)
        out = fn(t, dim=axis, keepdim=keepdims)
        return _T(out.values if hasattr(out, "values") else out)
    return f


sum = _reduce("sum")  # noqa: A001
mean = _reduce("mean")
prod = _reduce("prod")
amax = max = _reduce("amax")  # noqa: A001
amin = min = _reduce("amin")  # noqa: A001
std = _reduce("std")
var = _reduce("var")


def argmax(a, axis=None):
    return _T(torch.argmax(_t(a), dim=axis))


def argmin(a, axis=None):
    return _T(torch.argmin(_t(a), dim=axis))


def reshape(x, new_shape):
    return _T(_t(x).reshape(new_shape))


def transpose(a, axes=None):
    t = _t(a)
    return _T(t.permute(*axes) if axes is not None else t.permute(*reversed(builtins.range(t.dim()))))


def concatenate(arrays, axis=0):
    return _T(torch.cat([_t(a) for a in arrays], dim=axis))


def stack(arrays, axis=0):
    return _T(torch.stack([_t(a) for a in arrays], dim=axis))


def split(x, indices_or_sections, axis=0):
    t = _t(x)
    if isinstance(indices_or_sections, int):
        return tuple(_T(p) for p in torch.chunk(t, indices_or_sections, dim=axis))
    return tuple(_T(p) for p in torch.tensor_split(t, list(indices_or_sections), dim=axis))


def expand_dims(a, axis):
    return _T(_t(a).unsqueeze(axis))


def squeeze(a, axis=None):
    return _T(_t(a).squeeze() if axis is None else _t(a).squeeze(axis))


def where(condition, x=None, y=None):
    if x is None:
        return tuple(_T(i) for i in torch.where(_t(condition)))
    return _T(torch.where(_t(condition), _t(x), _t(y)))


def clip(x, xmin, xmax):
    return _T(torch.clamp(_t(x), xmin, xmax))


def tile(a, reps):
    return _T(_t(a).repeat(*((reps,) if isinstance(reps, int) else reps)))


def cumsum(a, axis=None, dtype=None):
    t = _t(a)
    return _T(torch.cumsum(t.reshape(-1) if axis is None else t, 0 if axis is None else axis, dtype=dtype))


def tril(m, k=0):
    return _T(torch.tril(_t(m), k))


def triu(m, k=0):
    return _T(torch.triu(_t(m), k))


def zeros_like(a, dtype=None):
    return _T(torch.zeros_like(_t(a), dtype=dtype))


def ones_like(a, dtype=None):
    return _T(torch.ones_like(_t(a), dtype=dtype))


def isclose(a, b, rtol=1e-05, atol=1e-08, equal_nan=False):
    return _T(torch.isclose(_t(a), _t(b), rtol, atol, equal_nan))


def allclose(a, b, rtol=1e-05, atol=1e-08):
    return bool(torch.allclose(_t(a), _t(b), rtol, atol))
