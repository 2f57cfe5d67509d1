"""Column transforms usable in ``Dataset.map`` (python/mindspore/dataset/transforms/transforms.py)."""
import numpy as np


class Compose:
    def __init__(self, transforms):
        self.transforms = list(transforms)

    def __call__(self, *x):
        for t in self.transforms:
            x = t(*x)
            if not isinstance(x, tuple):
                x = (x,)
        return x if len(x) > 1 else x[0]


class TypeCast:
    def __init__(self, data_type):
        import torch
        self.dtype = {torch.float32: np.float32, torch.int32: np.int32, torch.int64: np.int64,
                      torch.float16: np.float16, torch.uint8: np.uint8}.get(data_type, data_type)

    def __call__(self, x):
        return np.asarray(x).astype(self.dtype)


class OneHot:
    def __init__(self, num_classes, smoothing_rate=0.0):
        self.n, self.s = num_classes, smoothing_rate

    def __call__(self, x):
        out = np.full((self.n,), self.s / self.n, dtype=np.float32)
        out[int(x)] += 1.0 - self.s
        return out


# ------------------------------------------------------------------------------------------------ further transforms
import enum as _enum

import numpy as _np


class Relational(_enum.Enum):
    EQ = "eq"
    NE = "ne"
    GT = "gt"
    GE = "ge"
    LT = "lt"
    LE = "le"


class Fill:
    def __init__(self, fill_value):
        self.v = fill_value

    def __call__(self, x):
        return _np.full_like(_np.asarray(x), self.v)


class Mask:
    def __init__(self, operator, constant, dtype=_np.bool_):
        self.op, self.c, self.dtype = Relational(operator), constant, dtype

    def __call__(self, x):
        x = _np.asarray(x)
        fn = {"eq": _np.equal, "ne": _np.not_equal, "gt": _np.greater, "ge": _np.greater_equal, "lt": _np.less,
              "le": _np.less_equal}[self.op.value]
        return fn(x, self.c).astype(self.dtype)


class PadEnd:
    def __init__(self, pad_shape, pad_value=None):
        self.shape, self.value = list(pad_shape), pad_value

    def __call__(self, x):
        x = _np.asarray(x)
        fill = self.value if self.value is not None else ("" if x.dtype.kind in "OUS" else 0)
        out = _np.full(self.shape, fill, dtype=x.dtype)
        sl = tuple(slice(0, min(a, b)) for a, b in zip(x.shape, self.shape))
        out[sl] = x[sl]
        return out


class Concatenate:
    def __init__(self, axis=0, prepend=None, append=None):
        self.axis, self.pre, self.app = axis, prepend, append

    def __call__(self, *xs):
        parts = ([_np.asarray(self.pre)] if self.pre is not None else []) + [_np.asarray(x) for x in xs] + \
            ([_np.asarray(self.app)] if self.app is not None else [])
        return _np.concatenate(parts, self.axis)


class Duplicate:
    def __call__(self, x):
        return x, _np.array(x, copy=True)


class Unique:
    def __call__(self, x):
        x = _np.asarray(x).reshape(-1)
        uniq, first, inv, cnt = _np.unique(x, return_index=True, return_inverse=True, return_counts=True)
        order = _np.argsort(first)                           # first-occurrence order
        rank = _np.empty_like(order)
        rank[order] = _np.arange(len(order))
        return uniq[order], rank[inv].astype(_np.int32), cnt[order].astype(_np.int32)


class Slice:
    def __init__(self, *slices):
        def conv(s):
            if isinstance(s, int):
                return slice(s)
            if isinstance(s, (list, tuple)) and not isinstance(s, slice):
                return list(s)
            return s if s is not None else slice(None)
        self.s = tuple(conv(s) for s in slices)

    def __call__(self, x):
        return _np.asarray(x)[self.s]


class RandomApply:
    def __init__(self, transforms, prob=0.5):
        self.t, self.p = list(transforms), prob

    def __call__(self, *xs):
        if _np.random.random() >= self.p:
            return xs[0] if len(xs) == 1 else xs
        out = xs
        for t in self.t:
            out = t(*out) if isinstance(out, tuple) else t(out)
            out = out if isinstance(out, tuple) else (out,)
        return out[0] if len(out) == 1 else out


class RandomChoice:
    def __init__(self, transforms):
        self.t = list(transforms)

    def __call__(self, *xs):
        return self.t[_np.random.randint(len(self.t))](*xs)


class RandomOrder:
    def __init__(self, transforms):
        self.t = list(transforms)

    def __call__(self, x):
        for k in _np.random.permutation(len(self.t)):
            x = self.t[k](x)
        return x



class TensorOperation:
    """Base of transforms: a callable applied to the columns of a row."""

    def __call__(self, *inputs):
        return self.execute(*inputs) if hasattr(self, "execute") else self._run(*inputs)


class PyTensorOperation(TensorOperation):
    """Base of transforms written in Python."""


class CompoundOperation(TensorOperation):
    """Base of transforms that hold other transforms (``Compose``, ``RandomApply`` ...)."""

    def __init__(self, transforms=None):
        self.transforms = list(transforms or [])


class Plugin(TensorOperation):
    """Runs ``plugin_func(args)`` from a shared library through ctypes: the symbol takes (input pointer, element
    count, output pointer) over float32 data and returns the number of output elements."""

    def __init__(self, lib_path, func_name, user_args=None):
        import ctypes
        self.lib = ctypes.CDLL(lib_path)
        self.fn = getattr(self.lib, func_name)
        self.fn.restype = ctypes.c_longlong
        self.user_args = user_args

    def __call__(self, x):
        import ctypes

        import numpy as np
        a = np.ascontiguousarray(x, dtype=np.float32)
        out = np.empty_like(a)
        n = self.fn(a.ctypes.data_as(ctypes.c_void_p), ctypes.c_longlong(a.size), out.ctypes.data_as(ctypes.c_void_p))
        return out.reshape(-1)[:n].reshape(a.shape) if n == a.size else out.reshape(-1)[:n]


def not_random(func):
    """Marks a transform as deterministic."""
    func.random = False
    return func


def clean_unused_executors():
    """Releases executor objects kept for eager transform calls (none are cached here)."""
    return None
