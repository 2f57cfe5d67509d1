"""Functional API (``mindspore.ops.<fn>``): thin functions over the primitive classes.

Parity: mindspore/python/mindspore/ops/function/{math_func,array_func,nn_func,random_func}.py and
ops/functional.py - the widely used subset; every function routes through a Primitive so that graph
tracing and auto-parallel see the same node names as with the class API.
"""
from __future__ import annotations

import builtins
import numbers

import numpy as np
import torch
import torch.nn.functional as F

from ..common import dtype as mstype
from ..common.tensor import Tensor, as_tensor
from . import composite as C
from . import operations as P
from .primitive import _wrap_out

_cache = {}


def _prim(cls, *args, **kwargs):
    key = (cls, args, tuple(sorted(kwargs.items())))
    try:
        p = _cache.get(key)
    except TypeError:
        return cls(*args, **kwargs)
    if p is None:
        p = cls(*args, **kwargs)
        _cache[key] = p
    return p


def _gen_unary(name, cls):
    def fn(x):
        return _prim(cls)(x)
    fn.__name__ = name
    return fn


def _gen_binary(name, cls):
    def fn(x, y):
        return _prim(cls)(x, y)
    fn.__name__ = name
    return fn


_UN = {
    "abs": "Abs", "absolute": "Abs", "neg": "Neg", "negative": "Neg", "exp": "Exp", "expm1": "Expm1", "log": "Log",
    "log1p": "Log1p", "sqrt": "Sqrt", "rsqrt": "Rsqrt", "square": "Square", "sign": "Sign", "sin": "Sin",
    "cos": "Cos", "tan": "Tan", "asin": "Asin", "acos": "ACos", "atan": "Atan", "sinh": "Sinh", "cosh": "Cosh",
    "tanh": "Tanh", "asinh": "Asinh", "acosh": "Acosh", "atanh": "Atanh", "erf": "Erf", "erfc": "Erfc",
    "erfinv": "Erfinv", "floor": "Floor", "ceil": "Ceil", "trunc": "Trunc", "reciprocal": "Reciprocal",
    "logical_not": "LogicalNot", "isnan": "IsNan", "isinf": "IsInf", "isfinite": "IsFinite", "sigmoid": "Sigmoid",
    "relu": "ReLU", "relu6": "ReLU6", "silu": "SiLU", "mish": "Mish", "softsign": "Softsign",
    "hardsigmoid": "HSigmoid", "hardswish": "HSwish", "selu": "SeLU", "lgamma": "Lgamma", "digamma": "Digamma",
    "ones_like": "OnesLike", "zeros_like": "ZerosLike", "identity": "Identity", "invert": "Invert",
    "fast_gelu": "FastGeLU", "sinc": "Sinc", "bitwise_not": "Invert",
}
_BIN = {
    "add": "Add", "sub": "Sub", "subtract": "Sub", "mul": "Mul", "multiply": "Mul", "div": "Div", "divide": "Div",
    "true_divide": "RealDiv", "floor_div": "FloorDiv", "floor_divide": "FloorDiv", "floor_mod": "FloorMod",
    "remainder": "FloorMod", "fmod": "Mod", "pow": "Pow", "maximum": "Maximum", "minimum": "Minimum",
    "equal": "Equal", "eq": "Equal", "not_equal": "NotEqual", "ne": "NotEqual", "greater": "Greater", "gt": "Greater",
    "greater_equal": "GreaterEqual", "ge": "GreaterEqual", "less": "Less", "lt": "Less", "less_equal": "LessEqual",
    "le": "LessEqual", "logical_and": "LogicalAnd", "logical_or": "LogicalOr", "logical_xor": "LogicalXor",
    "bitwise_and": "BitwiseAnd", "bitwise_or": "BitwiseOr", "bitwise_xor": "BitwiseXor", "atan2": "Atan2",
    "xlogy": "Xlogy", "xdivy": "Xdivy", "hypot": "Hypot", "gcd": "Gcd", "lcm": "Lcm", "squared_difference":
    "SquaredDifference", "tensor_add": "Add", "tensor_sub": "Sub", "tensor_mul": "Mul", "tensor_div": "RealDiv",
    "tensor_pow": "Pow", "tensor_gt": "Greater", "tensor_lt": "Less", "tensor_ge": "GreaterEqual",
    "tensor_le": "LessEqual", "div_no_nan": "DivNoNan",
}
for _fn, _cls in _UN.items():
    globals()[_fn] = _gen_unary(_fn, getattr(P, _cls))
for _fn, _cls in _BIN.items():
    globals()[_fn] = _gen_binary(_fn, getattr(P, _cls))


def round(x, decimals=0):  # noqa: A001
    return _wrap_out(torch.round(x, decimals=decimals))


def cast(x, dtype):
    return _prim(P.Cast)(x, dtype)


def matmul(a, b):
    if isinstance(a, torch.Tensor) and isinstance(b, torch.Tensor) and a.dim() == 2 and b.dim() == 2:
        return _prim(P.MatMul)(a, b)
    if isinstance(a, torch.Tensor) and isinstance(b, torch.Tensor) and a.dim() == b.dim() and a.dim() >= 3:
        return _prim(P.BatchMatMul)(a, b)
    return _prim(P.MatMulExt)(a, b)


def bmm(a, b):
    return _prim(P.BatchMatMul)(a, b)


def batch_dot(a, b):
    return _prim(P.BatchMatMul)(a, b)


def dense(x, w, b=None):
    from . import fused
    return _wrap_out(fused.linear(x, w, b))


def addn(xs):
    return _prim(P.AddN)(xs)


def reduce_sum(x, axis=(), keep_dims=False):
    return _prim(P.ReduceSum, keep_dims)(x, axis)


def reduce_mean(x, axis=(), keep_dims=False):
    return _prim(P.ReduceMean, keep_dims)(x, axis)


def reduce_max(x, axis=(), keep_dims=False):
    return _prim(P.ReduceMax, keep_dims)(x, axis)


def reduce_min(x, axis=(), keep_dims=False):
    return _prim(P.ReduceMin, keep_dims)(x, axis)


def sum(x, dim=None, keepdim=False, *, dtype=None):  # noqa: A001
    out = _prim(P.ReduceSum, keepdim)(x, () if dim is None else dim)
    return out.to(dtype) if dtype is not None else out


def mean(x, axis=None, keep_dims=False):
    return _prim(P.ReduceMean, keep_dims)(x, () if axis is None else axis)


def amax(x, axis=None, keepdims=False):
    return _prim(P.ReduceMax, keepdims)(x, () if axis is None else axis)


def amin(x, axis=None, keepdims=False):
    return _prim(P.ReduceMin, keepdims)(x, () if axis is None else axis)


def prod(x, axis=None, keep_dims=False):
    return _prim(P.ReduceProd, keep_dims)(x, () if axis is None else axis)


def all(x, axis=None, keep_dims=False):  # noqa: A001
    return _prim(P.ReduceAll, keep_dims)(x, () if axis is None else axis)


def any(x, axis=None, keep_dims=False):  # noqa: A001
    return _prim(P.ReduceAny, keep_dims)(x, () if axis is None else axis)


def max(x, axis=None, keepdims=False):  # noqa: A001
    if axis is None:
        return _prim(P.ReduceMax)(x, ())
    idx, val = _prim(P.ArgMaxWithValue, axis, keepdims)(x)
    return val, idx


def min(x, axis=None, keepdims=False):  # noqa: A001
    if axis is None:
        return _prim(P.ReduceMin)(x, ())
    idx, val = _prim(P.ArgMinWithValue, axis, keepdims)(x)
    return val, idx


def argmax(x, dim=None, keepdim=False):
    if dim is None:
        return _wrap_out(torch.argmax(x))
    out = _prim(P.Argmax, dim, mstype.int64)(x)
    return out.unsqueeze(dim) if keepdim else out


def argmin(x, axis=None, keepdims=False):
    if axis is None:
        return _wrap_out(torch.argmin(x))
    out = _prim(P.Argmin, axis, mstype.int64)(x)
    return out.unsqueeze(axis) if keepdims else out


def cumsum(x, axis, dtype=None):
    out = _prim(P.CumSum)(x, axis)
    return out.to(dtype) if dtype is not None else out


def topk(x, k, dim=None, largest=True, sorted=True):  # noqa: A002
    if dim in (None, -1, x.dim() - 1) and largest:
        return _prim(P.TopK, sorted)(x, k)
    v, i = torch.topk(x, k, dim=-1 if dim is None else dim, largest=largest, sorted=sorted)
    return _wrap_out(v), _wrap_out(i)


def sort(x, axis=-1, descending=False):
    return _prim(P.Sort, axis, descending)(x)


def reshape(x, shape):
    return _prim(P.Reshape)(x, shape)


def shape(x):
    return tuple(x.shape)


def rank(x):
    return x.dim()


def size(x):
    return x.numel()


def dtype(x):
    return x.dtype


def transpose(x, perm):
    return _prim(P.Transpose)(x, perm)


def permute(x, axis):
    return _prim(P.Transpose)(x, axis)


def swapaxes(x, a, b):
    perm = list(builtins.range(x.dim()))
    perm[a], perm[b] = perm[b], perm[a]
    return _prim(P.Transpose)(x, tuple(perm))


def expand_dims(x, axis):
    return _prim(P.ExpandDims)(x, axis)


unsqueeze = expand_dims


def squeeze(x, axis=None):
    return _prim(P.Squeeze, () if axis is None else axis)(x)


def concat(xs, axis=0):
    return _prim(P.Concat, axis)(xs)


cat = concat


def stack(xs, axis=0):
    return _prim(P.Stack, axis)(xs)


def unstack(x, axis=0):
    return _prim(P.Unstack, axis)(x)


unbind = unstack


def split(x, split_size_or_sections, axis=0):
    return _wrap_out(tuple(torch.split(x, split_size_or_sections, dim=axis)))


def chunk(x, chunks, axis=0):
    return _wrap_out(tuple(torch.chunk(x, chunks, dim=axis)))


def tile(x, dims):
    return _prim(P.Tile)(x, dims)


def broadcast_to(x, shape):
    return _prim(P.BroadcastTo, tuple(shape))(x)


def gather(x, indices, axis, batch_dims=0):
    return _prim(P.Gather, batch_dims)(x, indices, axis)


def gather_elements(x, dim, index):
    return _prim(P.GatherD)(x, dim, index)


gather_d = gather_elements


def gather_nd(x, indices):
    return _prim(P.GatherNd)(x, indices)


def scatter_nd(indices, updates, shape):
    return _prim(P.ScatterNd)(indices, updates, shape)


def tensor_scatter_update(x, indices, updates):
    return _prim(P.TensorScatterUpdate)(x, indices, updates)


def tensor_scatter_add(x, indices, updates):
    return _prim(P.TensorScatterAdd)(x, indices, updates)


def unsorted_segment_sum(x, ids, n):
    return _prim(P.UnsortedSegmentSum)(x, ids, n)


def one_hot(indices, depth, on_value=1, off_value=0, axis=-1):
    return _prim(P.OneHot, axis)(indices, depth, on_value, off_value)


def cond(pred, true_fn, false_fn, *operands):
    """Traceable conditional: ``true_fn(*operands) if pred else false_fn(*operands)``.  In graph mode both branches
    become sub-graphs behind one Switch node and the branch is chosen at every run (``graph/control_flow.py``)."""
    from ..graph.control_flow import cond as _cond
    return _cond(pred, true_fn, false_fn, *operands)


def while_loop(cond_fn, body_fn, init_val, max_iterations=None):
    """Traceable loop: see ``graph/control_flow.py::while_loop``."""
    from ..graph.control_flow import while_loop as _w
    return _w(cond_fn, body_fn, init_val, max_iterations)


def fori_loop(lower, upper, body_fn, init_val, unroll=True):
    from ..graph.control_flow import fori_loop as _f
    return _f(lower, upper, body_fn, init_val, unroll)


def scan(f, init, xs, length=None):
    from ..graph.control_flow import scan as _s
    return _s(f, init, xs, length)


def select(cond, x, y):
    return _prim(P.Select)(cond, x, y)


def where(cond, x, y):
    return _prim(P.Select)(cond, x, y)


def masked_fill(x, mask, value):
    return _prim(P.MaskedFill)(x, mask, value)


def fill(type, shape, value):  # noqa: A002
    return _prim(P.Fill)(type, shape, value)


def full(size, fill_value, *, dtype=None):
    v = torch.as_tensor(fill_value)
    return _wrap_out(torch.full(tuple(size) if not isinstance(size, int) else (size,), v.item(),
                                dtype=dtype if dtype is not None else (mstype.float32 if v.is_floating_point() else v.dtype)))


def zeros(shape, dtype=mstype.float32):
    return _prim(P.Zeros)(shape, dtype if dtype is not None else mstype.float32)


def ones(shape, dtype=mstype.float32):
    return _prim(P.Ones)(shape, dtype if dtype is not None else mstype.float32)


def arange(start=0, end=None, step=1, *, dtype=None):
    if end is None:
        start, end = 0, start
    return _wrap_out(torch.arange(start, end, step, dtype=dtype))


def range(start, limit, delta):  # noqa: A001
    return _prim(P.Range)(start, limit, delta)


def linspace(start, end, steps):
    return _prim(P.LinSpace)(start, end, steps)


def eye(n, m=None, dtype=mstype.float32):
    return _prim(P.Eye)(n, m if m is not None else n, dtype)


def tril(x, diagonal=0):
    return _prim(P.Tril, diagonal)(x)


def triu(x, diagonal=0):
    return _prim(P.Triu, diagonal)(x)


def flip(x, dims):
    return _prim(P.ReverseV2, tuple(dims))(x)


def clamp(x, min=None, max=None):  # noqa: A002
    return C.clip_by_value(x, min, max)


clip = clamp
clip_by_value = C.clip_by_value
clip_by_global_norm = C.clip_by_global_norm


def flatten(x, order="C", *, start_dim=1, end_dim=-1):
    return _wrap_out(torch.flatten(x, start_dim, end_dim))


def slice(x, begin, size):  # noqa: A001
    return _prim(P.Slice)(x, begin, size)


def strided_slice(x, begin, end, strides, begin_mask=0, end_mask=0, ellipsis_mask=0, new_axis_mask=0,
                  shrink_axis_mask=0):
    return _prim(P.StridedSlice, begin_mask, end_mask, ellipsis_mask, new_axis_mask, shrink_axis_mask)(
        x, begin, end, strides)


def pad(x, padding, mode="constant", value=None):
    return _wrap_out(F.pad(x, list(padding), mode=mode, value=value))


def assign(var, value):
    return _prim(P.Assign)(var, value)


def assign_add(var, value):
    return _prim(P.AssignAdd)(var, value)


def assign_sub(var, value):
    return _prim(P.AssignSub)(var, value)


def depend(value, expr):
    return _prim(P.Depend)(value, expr)


def stop_gradient(x):
    return _prim(P.StopGradient)(x)


def einsum(equation, *operands):
    return _prim(P.Einsum, equation)(operands)


def norm(x, ord=None, dim=None, keepdim=False, *, dtype=None):  # noqa: A002
    return _wrap_out(torch.linalg.norm(x, ord=ord, dim=dim, keepdim=keepdim, dtype=dtype))


def lerp(s, e, w):
    return _prim(P.Lerp)(s, e, w)


def addcmul(x, a, b, value=1):
    return _prim(P.Addcmul)(x, a, b, value)


def addcdiv(x, a, b, value=1):
    return _prim(P.Addcdiv)(x, a, b, value)


def isclose(a, b, rtol=1e-5, atol=1e-8, equal_nan=False):
    return _wrap_out(torch.isclose(a, b, rtol=rtol, atol=atol, equal_nan=equal_nan))


def logsumexp(x, axis, keep_dims=False):
    return _wrap_out(torch.logsumexp(x, dim=axis, keepdim=keep_dims))


def std(x, axis=None, ddof=0, keepdims=False):
    return _wrap_out(torch.std(x, dim=axis, correction=ddof, keepdim=keepdims))


def var(x, axis=None, ddof=0, keepdims=False):
    return _wrap_out(torch.var(x, dim=axis, correction=ddof, keepdim=keepdims))


def scalar_to_tensor(x, dtype=None):
    return Tensor(x, dtype=dtype)


def tuple_to_array(t):
    return Tensor(np.array(t))


def scalar_cast(x, dtype):
    return mstype.dtype_to_pytype(dtype)(x)


def is_tensor(x):
    return isinstance(x, torch.Tensor)


def isconstant(x):
    return not isinstance(x, torch.Tensor)


# ------------------------------------------------------------------------------------ nn functional
def softmax(x, axis=-1, *, dtype=None):
    out = _prim(P.Softmax, axis)(x if dtype is None else x.to(dtype))
    return out


def log_softmax(x, axis=-1):
    return _prim(P.LogSoftmax, axis)(x)


def gelu(x, approximate="none"):
    if approximate == "tanh":
        return _prim(P.GeLU)(x)
    return _wrap_out(F.gelu(x))


def elu(x, alpha=1.0):
    return _prim(P.Elu, alpha)(x)


def leaky_relu(x, alpha=0.2):
    return _prim(P.LeakyReLU, alpha)(x)


def softplus(x, beta=1, threshold=20):
    return _wrap_out(F.softplus(x, beta, threshold))


def dropout(x, p=0.5, training=True, seed=None):
    if not training or p == 0:
        return x
    return _prim(P.Dropout, 1.0 - p)(x)[0]


def layer_norm(x, normalized_shape, weight=None, bias=None, eps=1e-5):
    from . import fused
    if len(normalized_shape) == 1 and weight is not None:
        return _wrap_out(fused.layer_norm(x, weight, bias, eps))
    return _wrap_out(F.layer_norm(x, tuple(normalized_shape), weight, bias, eps))


def rms_norm(x, gamma, epsilon=1e-6):
    return _prim(P.RmsNorm, epsilon)(x, gamma)


def cross_entropy(x, target, weight=None, ignore_index=-100, reduction="mean", label_smoothing=0.0):
    if weight is None and reduction == "mean" and label_smoothing == 0.0 and not target.is_floating_point() \
            and x.is_cuda and x.dim() == 2:
        from . import fused
        return _wrap_out(fused.softmax_cross_entropy(x, target, ignore_index))
    tgt = target if target.is_floating_point() else target.long()
    return _wrap_out(F.cross_entropy(x, tgt, weight, ignore_index=ignore_index, reduction=reduction,
                                     label_smoothing=label_smoothing))


def nll_loss(x, target, weight=None, ignore_index=-100, reduction="mean", label_smoothing=0.0):
    return _wrap_out(F.nll_loss(x, target.long(), weight, ignore_index=ignore_index, reduction=reduction))


def mse_loss(x, y, reduction="mean"):
    return _wrap_out(F.mse_loss(x, y, reduction=reduction))


def l1_loss(x, y, reduction="mean"):
    return _wrap_out(F.l1_loss(x, y, reduction=reduction))


def smooth_l1_loss(x, y, beta=1.0, reduction="none"):
    return _prim(P.SmoothL1Loss, beta, reduction)(x, y)


def binary_cross_entropy(x, y, weight=None, reduction="mean"):
    return _prim(P.BinaryCrossEntropy, reduction)(x, y, weight)


def binary_cross_entropy_with_logits(x, y, weight=None, pos_weight=None, reduction="mean"):
    return _wrap_out(F.binary_cross_entropy_with_logits(x, y, weight, pos_weight=pos_weight, reduction=reduction))


def kl_div(x, y, reduction="mean"):
    return _prim(P.KLDivLoss, reduction)(x, y)


def conv2d(x, weight, bias=None, stride=1, pad_mode="valid", padding=0, dilation=1, groups=1):
    from . import conv as _conv
    return _wrap_out(_conv.conv2d(x, weight, P._pair(stride), pad_mode, padding, P._pair(dilation), groups, bias))


def max_pool2d(x, kernel_size, stride=None, padding=0, dilation=1, return_indices=False, ceil_mode=False):
    return _wrap_out(F.max_pool2d(x, kernel_size, stride, padding, dilation, ceil_mode, return_indices))


def avg_pool2d(x, kernel_size=1, stride=1, padding=0, ceil_mode=False, count_include_pad=True, divisor_override=0):
    return _wrap_out(F.avg_pool2d(x, kernel_size, stride, padding, ceil_mode, count_include_pad,
                                  divisor_override or None))


def adaptive_avg_pool2d(x, output_size):
    return _wrap_out(F.adaptive_avg_pool2d(x, output_size))


def interpolate(x, size=None, scale_factor=None, mode="nearest", align_corners=None, recompute_scale_factor=None):
    return _wrap_out(F.interpolate(x, size=size, scale_factor=scale_factor, mode=mode, align_corners=align_corners))


def embedding(ids, weight, padding_idx=None, max_norm=None, norm_type=2.0, scale_grad_by_freq=False):
    from . import fused
    return _wrap_out(fused.embedding(weight, ids))


def flash_attention_score(query, key, value, head_num, real_shift=None, drop_mask=None, padding_mask=None,
                          attn_mask=None, prefix=None, actual_seq_qlen=None, actual_seq_kvlen=None, keep_prob=1.0,
                          scalar_value=1.0, pre_tokens=2147483647, next_tokens=2147483647, inner_precise=0,
                          input_layout="BSH", sparse_mode=0):
    prim = _prim(P.FlashAttentionScore, head_num, keep_prob, scalar_value, pre_tokens, next_tokens, inner_precise,
                 input_layout, sparse_mode)
    return prim(query, key, value, real_shift, drop_mask, padding_mask, attn_mask, prefix)[3]


# ------------------------------------------------------------------------------------ random
def standard_normal(shape, seed=None):
    return _prim(P.StandardNormal)(shape)


def normal(shape, mean, stddev, seed=None):
    return _wrap_out(torch.randn(tuple(shape)) * stddev + mean)


def uniform(shape, minval, maxval, seed=None, dtype=mstype.float32):
    lo = float(minval) if not isinstance(minval, torch.Tensor) else minval
    hi = float(maxval) if not isinstance(maxval, torch.Tensor) else maxval
    if dtype in (mstype.int32, mstype.int64):
        return _wrap_out(torch.randint(int(lo), int(hi), tuple(shape), dtype=dtype))
    return _wrap_out(torch.rand(tuple(shape)) * (hi - lo) + lo)


def rand(*size, dtype=None, seed=None):
    if len(size) == 1 and isinstance(size[0], (tuple, list)):
        size = tuple(size[0])
    return _wrap_out(torch.rand(size, dtype=dtype or mstype.float32))


def randn(*size, dtype=None, seed=None):
    if len(size) == 1 and isinstance(size[0], (tuple, list)):
        size = tuple(size[0])
    return _wrap_out(torch.randn(size, dtype=dtype or mstype.float32))


def randint(low, high, size, seed=None, *, dtype=None):
    return _wrap_out(torch.randint(low, high, tuple(size), dtype=dtype or mstype.int64))


def multinomial(x, num_samples, replacement=True, seed=None):
    return _wrap_out(torch.multinomial(x, num_samples, replacement))


# autodiff re-exports
grad = C.grad
value_and_grad = C.value_and_grad
vjp = C.vjp
jvp = C.jvp
jacfwd = C.jacfwd
jacrev = C.jacrev
partial = C.partial


# ------------------------------------------------------------------------------------------------ further functions
def _torch_fn(fn):
    def f(*args, **kwargs):
        return _wrap_out(fn(*args, **kwargs))
    f.__name__ = getattr(fn, "__name__", "fn")
    f.__doc__ = "Same arguments as torch.%s; returns framework tensors." % f.__name__
    return f


for _name in """argsort nonzero repeat_interleave scatter scatter_add cdist baddbmm outer inner kron roll rot90 meshgrid
cumprod diff searchsorted bucketize histc bincount tensor_split hsplit vsplit dsplit narrow index_select masked_select
take index_add index_fill bernoulli randperm rand_like randn_like randint_like polygamma mvlgamma allclose isreal
is_complex is_floating_point numel addbmm addmm addmv addr trace det logdet slogdet inverse pinverse matrix_power
cross dot mv mm vander tril_indices triu_indices combinations cartesian_prod block_diag atleast_1d atleast_2d
atleast_3d column_stack row_stack hstack vstack dstack swapaxes moveaxis movedim flipud fliplr nan_to_num nansum
nanmean nanmedian nanquantile quantile msort kthvalue mode median var_mean std_mean aminmax amax amin count_nonzero
heaviside copysign nextafter ldexp frexp logaddexp logaddexp2 float_power fmax fmin hypot igamma igammac i0 sinc
xlogy sgn signbit trapz trapezoid cumulative_trapezoid renorm gcd lcm deg2rad rad2deg bitwise_left_shift
bitwise_right_shift logical_xor isneginf isposinf view_as_real view_as_complex real imag conj angle polar""".split():
    if _name not in globals() and hasattr(torch, _name):
        globals()[_name] = _torch_fn(getattr(torch, _name))


def unique(input, sorted=True, return_inverse=False, return_counts=False, dim=None):    # noqa: A002
    return _wrap_out(torch.unique(input, sorted=sorted, return_inverse=return_inverse, return_counts=return_counts,
                                  dim=dim))


def cummax(input, axis):          # noqa: A002
    v, i = torch.cummax(input, axis)
    return _wrap_out(v), _wrap_out(i)


def cummin(input, axis):          # noqa: A002
    v, i = torch.cummin(input, axis)
    return _wrap_out(v), _wrap_out(i)


def shuffle(x, seed=None):
    g = torch.Generator()
    g.manual_seed(int(seed)) if seed is not None else g.seed()
    return _wrap_out(x[torch.randperm(x.shape[0], generator=g).to(x.device)])


def inplace_update(x, v, indices):
    out = x.clone()
    out[torch.as_tensor(indices, device=x.device)] = v.to(x.dtype)
    return _wrap_out(out)


def swish(x):
    return _wrap_out(torch.nn.functional.silu(x))


def prelu(x, weight):
    return _wrap_out(torch.nn.functional.prelu(x, weight))


def batch_norm(input_x, running_mean, running_var, weight, bias, training=False, momentum=0.1, eps=1e-5):
    return _wrap_out(torch.nn.functional.batch_norm(input_x, running_mean, running_var, weight, bias, training,
                                                    momentum, eps))


def grid_sample(input, grid, mode="bilinear", padding_mode="zeros", align_corners=False):      # noqa: A002
    return _wrap_out(torch.nn.functional.grid_sample(input, grid, mode, padding_mode, align_corners))


def unfold(input, kernel_size, dilation=1, padding=0, stride=1):      # noqa: A002
    return _wrap_out(torch.nn.functional.unfold(input, kernel_size, dilation, padding, stride))


def fold(input, output_size, kernel_size, dilation=1, padding=0, stride=1):      # noqa: A002
    size = tuple(int(v) for v in (output_size.tolist() if isinstance(output_size, torch.Tensor) else output_size))
    return _wrap_out(torch.nn.functional.fold(input, size, kernel_size, dilation, padding, stride))
