"""``Tensor``: a ``torch.Tensor`` subclass with MindSpore's constructor and method names.

Because it *is* a torch tensor, every kernel, collective and autograd path works on it with no
conversion; the subclass only adds the MindSpore surface (``asnumpy``, ``astype``, ``axis=`` /
``keep_dims=`` keyword spellings, ``size`` as an element count, ``Tensor(np_array, dtype)``).

Parity: mindspore/python/mindspore/common/tensor.py (constructor :190-310, asnumpy, astype,
init_data for ``init=`` tensors, the ~400 method surface) - the commonly used subset is covered.
"""
from __future__ import annotations

import numbers

import numpy as np
import torch

from . import dtype as mstype


def _sharded_mode():
    from ..context import _AutoParallelContext
    return _AutoParallelContext()._v["parallel_mode"] in ("semi_auto_parallel", "auto_parallel")


class _SizeInt(int):
    """``Tensor.size`` in MindSpore is the element count; torch code calls ``size()``.  Both work."""

    def __new__(cls, tensor):
        obj = int.__new__(cls, tensor.numel())
        obj._t = tensor
        return obj

    def __call__(self, dim=None):
        if dim is None:
            return torch.Tensor.size(self._t)
        return torch.Tensor.size(self._t, dim)


def _to_torch(data, dtype=None, device=None):
    if isinstance(data, torch.Tensor):
        t = data.detach() if not isinstance(data, Tensor) else data
        t = t.as_subclass(torch.Tensor)
    elif isinstance(data, np.ndarray):
        if data.dtype == np.float64 and dtype is None:
            dtype = mstype.float64
        t = torch.from_numpy(np.ascontiguousarray(data))
    elif isinstance(data, (bool, np.bool_)):
        t = torch.tensor(bool(data), dtype=torch.bool)
    elif isinstance(data, numbers.Integral):
        t = torch.tensor(int(data), dtype=torch.int64)
    elif isinstance(data, numbers.Real):
        t = torch.tensor(float(data), dtype=torch.float32)
    elif isinstance(data, numbers.Complex):
        t = torch.tensor(complex(data), dtype=torch.complex64)
    elif isinstance(data, (list, tuple)):
        arr = np.array(data)
        if arr.dtype == np.float64:
            arr = arr.astype(np.float32)
        t = torch.from_numpy(arr)
    elif isinstance(data, np.generic):
        t = torch.from_numpy(np.asarray(data))
    else:
        raise TypeError("For Tensor, the input_data must be Tensor, numpy.ndarray, list, tuple, int, float or bool, "
                        "but got %s" % type(data))
    if dtype is not None and t.dtype != dtype:
        t = t.to(dtype)
    if device is not None and t.device != device:
        t = t.to(device)
    return t


class Tensor(torch.Tensor):
    """Tensor(input_data=None, dtype=None, shape=None, init=None, const_arg=False)."""

    @staticmethod
    def __new__(cls, input_data=None, dtype=None, shape=None, init=None, const_arg=False, device=None):
        if input_data is None and init is None and dtype is not None and (
                shape is None or any(d is None or not isinstance(d, int) for d in shape)):
            # a placeholder of an input signature: dimensions that are None or a Symbol are known at run time only
            # (shape=None: the rank too).  It holds no storage; unknown dimensions show as their smallest value.
            dims = [2, 2] if shape is None else [d if isinstance(d, int) else getattr(d, "min", 1) for d in shape]
            obj = torch.Tensor._make_subclass(cls, torch.empty(dims, dtype=dtype, device="meta"), False)
            obj.const_arg = const_arg
            obj.symbolic_shape = None if shape is None else tuple(shape)
            obj.dynamic_rank = shape is None
            return obj
        if input_data is None:
            if init is None or shape is None:
                if shape is not None and dtype is not None and init is None:
                    t = torch.empty(tuple(shape), dtype=dtype)
                else:
                    raise ValueError("Tensor needs input_data, or init together with shape and dtype")
            else:
                from .initializer import initializer as _mk
                src = _mk(init, tuple(shape), dtype or mstype.float32)
                t = src.as_subclass(torch.Tensor)
        else:
            t = _to_torch(input_data, dtype, device)
            if shape is not None and tuple(shape) != tuple(t.shape):
                t = t.reshape(tuple(shape))
        if device is None:
            from .. import context
            dev = context.device()
            if t.device != dev and dev.type == "cuda":
                t = t.to(dev)
        obj = torch.Tensor._make_subclass(cls, t, t.requires_grad if t.is_floating_point() else False)
        obj.const_arg = const_arg
        return obj

    def __init__(self, *args, **kwargs):
        pass

    @classmethod
    def __torch_function__(cls, func, types, args=(), kwargs=None):
        out = super().__torch_function__(func, types, args, kwargs or {})
        if _sharded_mode():
            from ..parallel import spmd
            spmd.propagate_elementwise(func, args, out)
        return out

    # ------------------------------------------------------------------ conversion
    def asnumpy(self):
        t = self.detach().as_subclass(torch.Tensor)
        if t.dtype == torch.bfloat16:
            t = t.float()
        return t.cpu().numpy()

    def numpy(self, *a, **k):
        return self.asnumpy()

    def astype(self, dtype, copy=True):
        if isinstance(dtype, str):
            dtype = getattr(mstype, dtype)
        return self.to(dtype)

    def item(self, index=None):
        if index is None:
            return torch.Tensor.item(self)
        return torch.Tensor.item(self[index])

    def tolist(self):
        return self.asnumpy().tolist()

    def __reduce_ex__(self, proto):
        return (_rebuild_tensor, (self.asnumpy(), self.dtype))

    def __deepcopy__(self, memo):
        out = Tensor(self.detach().as_subclass(torch.Tensor).clone())
        memo[id(self)] = out
        return out

    def __repr__(self):
        t = self.detach().as_subclass(torch.Tensor)
        return "Tensor(shape=%s, dtype=%s, value=\n%s)" % (list(t.shape), _dtype_name(t.dtype),
                                                          np.array2string(self.asnumpy(), separator=", "))

    __str__ = lambda self: str(self.asnumpy())  # noqa: E731

    def __hash__(self):
        return id(self)

    def __bool__(self):
        from ..graph import tracer
        session = tracer.current()
        if session is not None:
            session.note_host_branch(self)
        return bool(torch.Tensor.__bool__(self.as_subclass(torch.Tensor)))

    # ------------------------------------------------------------------ attributes
    @property
    def size(self):
        return _SizeInt(self)

    @property
    def itemsize(self):
        return self.element_size()

    @property
    def nbytes(self):
        return self.element_size() * self.numel()

    @property
    def strides(self):
        return tuple(s * self.element_size() for s in self.stride())

    @property
    def has_init(self):
        return False

    def init_data(self, slice_index=None, shape=None, opt_shard_group=None):
        return self

    def set_const_arg(self, const_arg=True):
        self.const_arg = const_arg

    # ------------------------------------------------------------------ MindSpore spellings
    def _axis_kw(self, fn, axis, keep_dims, **kw):
        if axis is None or axis == ():
            out = fn(self, **kw)
            if keep_dims:
                out = out.reshape((1,) * self.dim())
            return out
        return fn(self, dim=axis, keepdim=keep_dims, **kw)

    def sum(self, axis=None, dtype=None, keepdims=False, initial=None, *, dim=None, keepdim=None):
        axis = dim if dim is not None else axis
        keepdims = keepdim if keepdim is not None else keepdims
        if isinstance(dtype, bool):  # torch positional spelling sum(dim, keepdim)
            keepdims, dtype = dtype, None
        kw = {"dtype": dtype} if dtype is not None else {}
        out = self._axis_kw(torch.Tensor.sum, axis, keepdims, **kw)
        return out + initial if initial is not None else out

    def mean(self, axis=None, keep_dims=False, *, dim=None, keepdim=None, keepdims=None, dtype=None):
        axis = dim if dim is not None else axis
        keep = keepdim if keepdim is not None else (keepdims if keepdims is not None else keep_dims)
        kw = {"dtype": dtype} if dtype is not None else {}
        return self._axis_kw(torch.Tensor.mean, axis, keep, **kw)

    def max(self, axis=None, keepdims=False, *, dim=None, keepdim=None, initial=None, where=True,
            return_indices=False):
        axis = dim if dim is not None else axis
        keep = keepdim if keepdim is not None else keepdims
        if isinstance(axis, torch.Tensor):  # torch.max(a, b) spelling
            return torch.maximum(self, axis)
        if axis is None:
            return torch.Tensor.max(self)
        if dim is not None:
            return torch.Tensor.max(self, dim=axis, keepdim=keep)
        vals = torch.amax(self, dim=axis, keepdim=keep)
        if return_indices:
            return vals, torch.argmax(self, dim=axis, keepdim=keep)
        return vals

    def min(self, axis=None, keepdims=False, *, dim=None, keepdim=None, initial=None, where=True,
            return_indices=False):
        axis = dim if dim is not None else axis
        keep = keepdim if keepdim is not None else keepdims
        if isinstance(axis, torch.Tensor):
            return torch.minimum(self, axis)
        if axis is None:
            return torch.Tensor.min(self)
        if dim is not None:
            return torch.Tensor.min(self, dim=axis, keepdim=keep)
        vals = torch.amin(self, dim=axis, keepdim=keep)
        if return_indices:
            return vals, torch.argmin(self, dim=axis, keepdim=keep)
        return vals

    def argmax(self, axis=None, keepdims=False, *, dim=None, keepdim=None):
        axis = dim if dim is not None else axis
        keep = keepdim if keepdim is not None else keepdims
        return torch.Tensor.argmax(self, dim=axis, keepdim=keep)

    def argmin(self, axis=None, keepdims=False, *, dim=None, keepdim=None):
        axis = dim if dim is not None else axis
        keep = keepdim if keepdim is not None else keepdims
        return torch.Tensor.argmin(self, dim=axis, keepdim=keep)

    def prod(self, axis=None, keep_dims=False, dtype=None, *, dim=None, keepdim=None):
        axis = dim if dim is not None else axis
        keep = keepdim if keepdim is not None else keep_dims
        if axis is None:
            return torch.Tensor.prod(self)
        return torch.Tensor.prod(self, dim=axis, keepdim=keep)

    def all(self, axis=None, keep_dims=False, *, dim=None, keepdim=None):
        axis = dim if dim is not None else axis
        keep = keepdim if keepdim is not None else keep_dims
        return self._axis_kw(torch.Tensor.all, axis, keep)

    def any(self, axis=None, keep_dims=False, *, dim=None, keepdim=None):
        axis = dim if dim is not None else axis
        keep = keepdim if keepdim is not None else keep_dims
        return self._axis_kw(torch.Tensor.any, axis, keep)

    def std(self, axis=None, ddof=0, keepdims=False, *, dim=None, keepdim=None, correction=None, unbiased=None):
        axis = dim if dim is not None else axis
        keep = keepdim if keepdim is not None else keepdims
        corr = correction if correction is not None else (int(unbiased) if unbiased is not None else ddof)
        return torch.std(self, dim=axis, correction=corr, keepdim=keep)

    def var(self, axis=None, ddof=0, keepdims=False, *, dim=None, keepdim=None, correction=None, unbiased=None):
        axis = dim if dim is not None else axis
        keep = keepdim if keepdim is not None else keepdims
        corr = correction if correction is not None else (int(unbiased) if unbiased is not None else ddof)
        return torch.var(self, dim=axis, correction=corr, keepdim=keep)

    def cumsum(self, axis=None, dtype=None, *, dim=None):
        axis = dim if dim is not None else axis
        if axis is None:
            return torch.Tensor.cumsum(self.reshape(-1), 0, dtype=dtype)
        return torch.Tensor.cumsum(self, axis, dtype=dtype)

    def transpose(self, *axes):
        if len(axes) == 1 and isinstance(axes[0], (tuple, list)):
            axes = tuple(axes[0])
        if len(axes) == 0:
            return self.permute(*reversed(range(self.dim())))
        if len(axes) == 2 and self.dim() != 2:
            return torch.Tensor.transpose(self, axes[0], axes[1])
        return self.permute(*axes)

    def swapaxes(self, axis0, axis1):
        return torch.Tensor.transpose(self, axis0, axis1)

    def expand_dims(self, axis):
        return self.unsqueeze(axis)

    def squeeze(self, axis=None, *, dim=None):
        axis = dim if dim is not None else axis
        if axis is None:
            return torch.Tensor.squeeze(self)
        return torch.Tensor.squeeze(self, axis)

    def flatten(self, order="C", *, start_dim=0, end_dim=-1):
        if isinstance(order, int):  # torch positional spelling flatten(start, end)
            return torch.Tensor.flatten(self, order, start_dim if start_dim != 0 else -1)
        return torch.Tensor.flatten(self, start_dim, end_dim)

    def ravel(self):
        return self.reshape(-1)

    def copy(self):
        return self.clone()

    def fill(self, value):
        return torch.full_like(self, value)

    def clip(self, xmin=None, xmax=None, dtype=None, *, min=None, max=None):
        out = torch.clamp(self, min=min if min is not None else xmin, max=max if max is not None else xmax)
        return out.to(dtype) if dtype is not None else out

    def broadcast_to(self, shape):
        return torch.broadcast_to(self, tuple(shape))

    def tile(self, *reps):
        if len(reps) == 1 and isinstance(reps[0], (tuple, list)):
            reps = tuple(reps[0])
        return torch.Tensor.tile(self, reps)

    def repeat(self, repeats, axis=None):
        if isinstance(repeats, (tuple, list)) and axis is None and len(repeats) > 1:
            return torch.Tensor.repeat(self, *repeats)
        return torch.repeat_interleave(self, repeats, dim=axis)

    def masked_fill(self, mask, value):
        return torch.Tensor.masked_fill(self, mask.bool() if mask.dtype != torch.bool else mask, value)

    def gather_elements(self, dim, index):
        return torch.gather(self, dim, index)

    def take(self, indices, axis=None, mode="clip"):
        if axis is None:
            return torch.take(self, indices)
        return torch.index_select(self, axis, indices.reshape(-1)).reshape(
            self.shape[:axis] + tuple(indices.shape) + self.shape[axis + 1:])

    def top_k(self, k, dim=None, largest=True, sorted=True):
        return torch.topk(self, k, dim=-1 if dim is None else dim, largest=largest, sorted=sorted)

    def assign_value(self, value):
        with torch.no_grad():
            self.copy_(_to_torch(value, self.dtype, self.device))
        return self

    def set_dtype(self, dtype):
        return self.to(dtype)

    def isclose(self, x2, rtol=1e-5, atol=1e-8, equal_nan=False):
        return torch.isclose(self, x2, rtol=rtol, atol=atol, equal_nan=equal_nan)

    def asnumpy_or_none(self):
        return self.asnumpy()


def _dtype_name(t):
    try:
        return mstype.ckpt_type_name(t)
    except KeyError:
        return str(t)


def _rebuild_tensor(arr, dtype):
    return Tensor(arr, dtype=dtype)


def as_tensor(x, dtype=None):
    """Wraps without copying when ``x`` already is a torch tensor on the right device."""
    if isinstance(x, Tensor) and (dtype is None or x.dtype == dtype):
        return x
    if isinstance(x, torch.Tensor):
        t = x if dtype is None or x.dtype == dtype else x.to(dtype)
        return t.as_subclass(Tensor)
    return Tensor(x, dtype=dtype)
