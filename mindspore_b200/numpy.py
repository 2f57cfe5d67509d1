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


# ------------------------------------------------------------------------------------------------ wider coverage
# Functions that torch offers under the same name and meaning are forwarded to torch (they stay on the device and
# differentiable); the rest run through NumPy on the host and come back as tensors on the input's device.
import numpy as _onp


def _fwd(fn):
    def f(*args, **kwargs):
        kwargs = {("dim" if k == "axis" else "keepdim" if k == "keepdims" else k): v for k, v in kwargs.items()}
        out = fn(*args, **kwargs)
        return _w(out)
    f.__name__ = getattr(fn, "__name__", "fn")
    return f


def _w(out):
    from .ops.primitive import _wrap_out
    if isinstance(out, (tuple, list)) and not isinstance(out, torch.Size):
        return type(out)(_w(o) for o in out) if not hasattr(out, "_fields") else tuple(_w(o) for o in out)
    return _wrap_out(out)


for _n in """logspace diag diagflat trace meshgrid ravel swapaxes moveaxis vstack hstack dstack column_stack hsplit
vsplit dsplit fliplr flipud rot90 sort argsort searchsorted nansum cumprod nanmean median quantile
nanquantile bincount cov corrcoef vdot inner outer tensordot einsum kron cross fmod float_power exp2 logaddexp
logaddexp2 arcsinh arccosh arctanh hypot deg2rad rad2deg fix fmax fmin isneginf isposinf signbit copysign nan_to_num
diff gradient trapz gcd lcm heaviside bitwise_and bitwise_or bitwise_xor logical_not logical_xor count_nonzero
nonzero argwhere tril_indices triu_indices broadcast_to atleast_1d atleast_2d atleast_3d vander sinc rand randn
randint full_like empty_like take unique""".split():
    if _n not in globals() and hasattr(torch, _n):
        globals()[_n] = _fwd(getattr(torch, _n))

_ALIASES = {"take_along_axis": torch.take_along_dim, "broadcast_arrays": torch.broadcast_tensors, "mod": torch.remainder,
            "fabs": torch.abs, "invert": torch.bitwise_not, "around": torch.round, "round": torch.round,
            "rint": torch.round, "degrees": torch.rad2deg, "radians": torch.deg2rad, "norm": torch.linalg.norm,
            "nanmax": lambda x, dim=None, keepdim=False: torch.amax(torch.nan_to_num(x, nan=float("-inf")),
                                                                    dim if dim is not None else tuple(range(x.dim())), keepdim),
            "nanmin": lambda x, dim=None, keepdim=False: torch.amin(torch.nan_to_num(x, nan=float("inf")),
                                                                    dim if dim is not None else tuple(range(x.dim())), keepdim),
            "cbrt": lambda x: torch.sign(x) * torch.abs(x) ** (1.0 / 3), "identity": lambda n, dtype=None: torch.eye(n, dtype=dtype),
            "flatnonzero": lambda x: torch.nonzero(x.reshape(-1)).reshape(-1),
            "array_equal": lambda a, b: bool(a.shape == b.shape and torch.equal(torch.as_tensor(a), torch.as_tensor(b))),
            "ptp": lambda x, dim=None, keepdim=False: (torch.amax(x, dim, keepdim) - torch.amin(x, dim, keepdim))
            if dim is not None else x.max() - x.min(),
            "repeat": lambda a, repeats, dim=None: torch.repeat_interleave(a, repeats, dim=dim),
            "average": lambda a, dim=None, weights=None: (a.mean() if dim is None else a.mean(dim)) if weights is None
            else ((a * weights).sum(dim if dim is not None else tuple(range(a.dim())))
                  / weights.sum(dim if dim is not None else tuple(range(weights.dim())))),
            "divmod": lambda a, b: (torch.floor_divide(a, b), torch.remainder(a, b))}
_ALIASES["flip"] = lambda m, dim=None: torch.flip(m, tuple(range(m.dim())) if dim is None else
                                                  ((dim,) if isinstance(dim, int) else tuple(dim)))
_ALIASES["roll"] = lambda a, shift, dim=None: torch.roll(a, shift) if dim is None else torch.roll(a, shift, dim)
for _n, _f in _ALIASES.items():
    if _n not in globals():
        globals()[_n] = _fwd(_f)


def _host(name):
    fn = getattr(_onp, name)

    def f(*args, **kwargs):
        dev = next((a.device for a in args if isinstance(a, torch.Tensor)), None)

        def down(x):
            if isinstance(x, torch.Tensor):
                x = x.detach().cpu()
                return x.float().numpy() if x.dtype == torch.bfloat16 else x.numpy()
            if isinstance(x, (list, tuple)):
                return type(x)(down(y) for y in x)
            return x

        def up(x):
            if isinstance(x, _onp.ndarray):
                if x.dtype == object or x.dtype.kind in "US":
                    return x
                t = torch.from_numpy(_onp.ascontiguousarray(x))
                return _w(t.to(dev) if dev is not None else t)
            if isinstance(x, (list, tuple)):
                return type(x)(up(y) for y in x)
            if isinstance(x, _onp.generic):
                return x.item()
            return x
        return up(fn(*down(args), **{k: down(v) for k, v in kwargs.items()}))
    f.__name__ = name
    f.__doc__ = "numpy.%s evaluated on the host; tensors come back on the input's device." % name
    return f


for _n in """geomspace rollaxis array_split choose select piecewise nanargmax nanargmin nancumsum nanstd nanvar
percentile histogram histogram2d histogramdd digitize correlate convolve interp ediff1d array_equiv tri diag_indices
ix_ indices unravel_index ravel_multi_index pad apply_along_axis apply_over_axes polyadd polysub polymul polyval
polyder polyint bartlett blackman hamming hanning kaiser""".split():
    if _n not in globals() and hasattr(_onp, _n):
        globals()[_n] = _host(_n)
mgrid, ogrid = _onp.mgrid, _onp.ogrid


# ---------------------------------------------------------------------------------------------------- numpy.fft
def _fft_namespace():
    import types as _types

    import torch as _torch

    from .ops import function_ext as _fx
    mod = _types.ModuleType(__name__ + ".fft")
    for _n in ("fft", "ifft", "fft2", "ifft2", "fftn", "ifftn", "fftshift", "ifftshift", "rfft", "irfft"):
        setattr(mod, _n, getattr(_fx, _n))
    mod.__all__ = ["fft", "ifft", "fft2", "ifft2", "fftn", "ifftn", "fftshift", "ifftshift", "rfft", "irfft"]
    import sys as _sys
    _sys.modules[mod.__name__] = mod
    return mod


fft = _fft_namespace()
fft2, ifft2, fftn, ifftn, fftshift, ifftshift, ifft = (fft.fft2, fft.ifft2, fft.fftn, fft.ifftn, fft.fftshift,
                                                       fft.ifftshift, fft.ifft)


# ---------------------------------------------------------------------------------------------------- remaining names
def _p(x):
    t = _t(x)
    return t.as_subclass(torch.Tensor) if isinstance(t, torch.Tensor) else t


def append(arr, values, axis=None):
    a, v = _p(arr), _p(values)
    if axis is None:
        return _w(torch.cat([a.reshape(-1), v.reshape(-1).to(a.dtype)]))
    return _w(torch.cat([a, v.to(a.dtype)], axis))


def array_str(a):
    return str(_p(a).cpu().numpy())


def size(a, axis=None):
    t = _p(a)
    return t.numel() if axis is None else t.shape[axis]


def diagonal(a, offset=0, axis1=0, axis2=1):
    return _w(torch.diagonal(_p(a), offset, axis1, axis2))


def copy_(a):
    return _w(_p(a).clone())


def intersect1d(ar1, ar2, assume_unique=False, return_indices=False):
    a, b = _p(ar1).reshape(-1), _p(ar2).reshape(-1)
    ua = a if assume_unique else torch.unique(a)
    ub = b if assume_unique else torch.unique(b)
    common = torch.sort(ua[torch.isin(ua, ub)]).values
    if not return_indices:
        return _w(common)
    first = lambda src: torch.stack([torch.nonzero(src == c)[0, 0] for c in common]) if common.numel() else \
        torch.zeros(0, dtype=torch.int64)
    return _w(common), _w(first(a)), _w(first(b))


def isin(element, test_elements, invert=False):
    return _w(torch.isin(_p(element), _p(test_elements), invert=invert))


def in1d(ar1, ar2, invert=False):
    return _w(torch.isin(_p(ar1).reshape(-1), _p(ar2), invert=invert))


def setdiff1d(ar1, ar2, assume_unique=False):
    a = _p(ar1).reshape(-1)
    a = a if assume_unique else torch.unique(a)
    return _w(a[~torch.isin(a, _p(ar2))])


def isscalar(element):
    return isinstance(element, (int, float, complex, bool, str, bytes, _np.generic)) or (
        isinstance(element, torch.Tensor) and element.dim() == 0 and False)


def sometrue(a, axis=None, keepdims=False):
    t = _p(a).bool()
    return _w(t.any() if axis is None else t.any(axis, keepdims))


def matrix_power(a, n):
    return _w(torch.linalg.matrix_power(_p(a), n))


def multi_dot(arrays):
    return _w(torch.linalg.multi_dot([_p(a) if _p(a).dim() else _p(a).reshape(1) for a in arrays]))


def positive(a, dtype=None):
    return _w(_p(a).to(dtype) if dtype is not None else _p(a).clone())


def promote_types(type1, type2):
    from .common import dtype as _mstype
    t1 = _mstype.to_torch(type1) if not isinstance(type1, torch.dtype) else type1
    t2 = _mstype.to_torch(type2) if not isinstance(type2, torch.dtype) else type2
    return torch.promote_types(t1, t2)


def result_type(*arrays_and_dtypes):
    out = None
    for a in arrays_and_dtypes:
        dt = a if isinstance(a, torch.dtype) else _p(a).dtype if isinstance(a, (torch.Tensor, list, tuple, _np.ndarray)) \
            else torch.as_tensor(a).dtype
        out = dt if out is None else torch.promote_types(out, dt)
    return out


def divmod_(x1, x2, dtype=None):
    a, b = _p(x1), _p(x2)
    q, r = torch.floor_divide(a, b), torch.remainder(a, b)
    return (_w(q.to(dtype)), _w(r.to(dtype))) if dtype is not None else (_w(q), _w(r))


def sum_(a, axis=None, dtype=None, keepdims=False, initial=None):
    t = _p(a)
    out = t.sum(dtype=dtype) if axis is None and not keepdims else t.sum(
        axis if axis is not None else tuple(range(t.dim())), keepdims, dtype=dtype)
    return _w(out + initial if initial is not None else out)


def unwrap(p, discont=3.141592653589793, axis=-1):
    t = _p(p)
    d = torch.diff(t, dim=axis)
    dm = torch.remainder(d + _np.pi, 2 * _np.pi) - _np.pi
    dm = torch.where((dm == -_np.pi) & (d > 0), torch.full_like(dm, _np.pi), dm)
    corr = torch.where(d.abs() < discont, torch.zeros_like(d), dm - d)
    first = t.narrow(axis, 0, 1)
    return _w(torch.cat([first, t.narrow(axis, 1, t.shape[axis] - 1) + torch.cumsum(corr, axis)], axis))


def histogram_bin_edges(a, bins=10, range=None, weights=None):  # noqa: A002
    return _w(torch.as_tensor(_np.histogram_bin_edges(_p(a).cpu().numpy(), bins, range)))


def tri_indices(n, k=0, m=None, upper=True):
    m = n if m is None else m
    fn = torch.triu_indices if upper else torch.tril_indices
    idx = fn(n, m, k)
    return _w(idx[0]), _w(idx[1])


def tril_indices_from(arr, k=0):
    t = _p(arr)
    idx = torch.tril_indices(t.shape[-2], t.shape[-1], k)
    return _w(idx[0]), _w(idx[1])


def triu_indices_from(arr, k=0):
    t = _p(arr)
    idx = torch.triu_indices(t.shape[-2], t.shape[-1], k)
    return _w(idx[0]), _w(idx[1])


def roll_along_axis(a, shift, axis):
    return _w(torch.roll(_p(a), shift, axis))


def convert_neg_indices(indices, ndim):
    t = _p(indices)
    return _w(torch.where(t < 0, t + ndim, t))


class NdGrid:
    """``mgrid`` / ``ogrid``: ``grid[0:3, 0:2]`` -> dense (``sparse=False``) or open coordinate arrays; a complex
    step ``5j`` means that many points including the end."""

    def __init__(self, sparse=False):
        self.sparse = sparse

    def __getitem__(self, keys):
        keys = keys if isinstance(keys, tuple) else (keys,)
        axes = []
        for k in keys:
            start = 0 if k.start is None else k.start
            step = 1 if k.step is None else k.step
            if isinstance(step, complex):
                axes.append(torch.linspace(float(start), float(k.stop), int(abs(step))))
            else:
                axes.append(torch.arange(start, k.stop, step))
        if len(axes) == 1:
            return _w(axes[0])
        if self.sparse:
            return tuple(_w(a.reshape([-1 if i == j else 1 for j in builtins.range(len(axes))]))
                         for i, a in enumerate(axes))
        return _w(torch.stack(torch.meshgrid(*axes, indexing="ij")))


class MGridClass(NdGrid):
    def __init__(self):
        super().__init__(False)


class OGridClass(NdGrid):
    def __init__(self):
        super().__init__(True)


mgrid, ogrid = MGridClass(), OGridClass()
asarray_const = asfarray_const = lambda a, dtype=None: _w(_t(a, dtype))  # noqa: E731
empty_compile = lambda dtype, shape: _w(torch.empty(tuple(shape), dtype=dtype))  # noqa: E731


class UniqueNet:
    """Callable form of ``unique`` (a Cell in the reference, kept for import compatibility)."""

    def __call__(self, x):
        out, inv = torch.unique(_p(x), return_inverse=True)
        return _w(out), _w(inv)


def comput_avg(a, axis=None, weights=None):
    return average(a, axis, weights) if "average" in globals() else _w(_p(a).float().mean())


def compute_weights_for_mean(x, x_avg, axis):
    t = _p(x)
    n = t.numel() if axis is None else t.shape[axis]
    return _w(torch.full_like(_p(x_avg), 1.0 / n))


def check_gradient_arguments(f, axis, edge_order):
    if edge_order != 1:
        raise NotImplementedError("edge_order != 1 not implemented")
    return axis if axis is not None else tuple(builtins.range(_p(f).dim()))
