"""MindSpore-only ``Tensor`` methods that ``torch.Tensor`` does not already provide under the same name
(python/mindspore/common/tensor.py: itemset :1110, ptp :2360, choose :2890, searchsorted :2960, gather_nd :3710,
tensor-scatter family, unsorted_segment_* , to_coo / to_csr, move_to / offload ...).  Attached to ``Tensor`` on import."""
from __future__ import annotations

import numpy as np
import torch

from .tensor import Tensor


def _w(t):
    return t if isinstance(t, Tensor) or not isinstance(t, torch.Tensor) else t.as_subclass(Tensor)


def _p(t):
    return t.detach().as_subclass(torch.Tensor) if isinstance(t, torch.Tensor) else torch.as_tensor(t)


def itemset(self, *args):
    """``itemset(value)`` for a 1-element tensor, ``itemset(index, value)`` otherwise; returns a new tensor."""
    out = _p(self).clone()
    if len(args) == 1:
        if out.numel() != 1:
            raise ValueError("itemset with one argument needs a tensor of exactly one element")
        out.reshape(-1)[0] = args[0]
    elif len(args) == 2:
        idx = args[0]
        if isinstance(idx, int):
            out.reshape(-1)[idx] = args[1]
        else:
            out[tuple(idx)] = args[1]
    else:
        raise ValueError("itemset takes 1 or 2 arguments, got %d" % len(args))
    return _w(out)


def fills(self, value):
    return _w(torch.full_like(_p(self), float(value) if not isinstance(value, torch.Tensor) else value.item()))


def ptp(self, axis=None, keepdims=False):
    x = _p(self)
    if axis is None:
        return _w(x.max() - x.min())
    return _w(x.amax(axis, keepdim=keepdims) - x.amin(axis, keepdim=keepdims))


def to_tensor(self, slice_index=None, shape=None, opt_shard_group=None):
    return self


def init_check(self):
    return self


def from_numpy(array):
    if not isinstance(array, np.ndarray):
        raise TypeError("For 'Tensor.from_numpy', the argument must be a numpy.ndarray, got %s" % type(array).__name__)
    if not array.flags.c_contiguous:
        raise ValueError("For 'Tensor.from_numpy', the array must be C-contiguous")
    return torch.from_numpy(array).as_subclass(Tensor)


def choose(self, choices, mode="clip"):
    idx = _p(self).long()
    ch = torch.stack([_p(c).expand(idx.shape) if _p(c).shape != idx.shape else _p(c) for c in choices]) \
        if isinstance(choices, (list, tuple)) else _p(choices)
    n = ch.shape[0]
    if mode == "clip":
        idx = idx.clamp(0, n - 1)
    elif mode == "wrap":
        idx = idx % n
    elif bool(((idx < 0) | (idx >= n)).any()):
        raise ValueError("invalid entry in choice array")
    return _w(torch.gather(ch, 0, idx.unsqueeze(0)).squeeze(0))


def searchsorted(self, v, side="left", sorter=None):
    a = _p(self)
    if sorter is not None:
        a = a[_p(sorter).long()]
    return _w(torch.searchsorted(a, _p(v), right=(side == "right")).to(torch.int32))


def gather_nd(self, indices):
    idx = _p(indices).long()
    return _w(_p(self)[tuple(idx[..., i] for i in range(idx.shape[-1]))])


def _tensor_scatter(name):
    def method(self, indices, updates):
        from ..ops import operations as P
        return getattr(P, name)()(self, indices, updates)
    method.__name__ = name
    return method


def inplace_update(self, v, indices):
    from ..ops import operations as P
    return P.InplaceUpdate(indices)(self, v)


def random_categorical(self, num_sample, seed=0, dtype=torch.int64):
    g = torch.Generator().manual_seed(int(seed)) if seed else None
    probs = torch.softmax(_p(self).float(), -1)
    return _w(torch.multinomial(probs.cpu(), int(num_sample), replacement=True, generator=g).to(dtype))


def one_hot(self, depth, on_value=1, off_value=0, axis=-1):
    oh = torch.nn.functional.one_hot(_p(self).long(), int(depth))
    out = torch.where(oh.bool(), torch.as_tensor(on_value), torch.as_tensor(off_value))
    if axis not in (-1, out.dim() - 1):
        out = out.movedim(-1, axis)
    return _w(out)


def unique_with_pad(self, pad_num):
    x = _p(self)
    uniq, inv = torch.unique(x, sorted=False, return_inverse=True)
    # first-occurrence order, as the reference produces
    first = torch.full((uniq.numel(),), x.numel(), dtype=torch.long).scatter_reduce(0, inv, torch.arange(x.numel()), "amin")
    order = torch.argsort(first)
    rank = torch.empty_like(order)
    rank[order] = torch.arange(order.numel())
    out = torch.full_like(x, pad_num)
    out[:uniq.numel()] = uniq[order]
    return _w(out), _w(rank[inv].to(x.dtype))


def _segment(name):
    def method(self, segment_ids, num_segments):
        from ..ops import operations as P
        return getattr(P, name)()(self, segment_ids, num_segments)
    method.__name__ = name
    return method


def col2im(self, output_size, kernel_size, dilation, padding_value, stride):
    x = _p(self)
    n, c, k, l = x.shape
    return _w(torch.nn.functional.fold(x.reshape(n, c * k, l), tuple(int(v) for v in _p(output_size).tolist())
                                       if isinstance(output_size, torch.Tensor) else output_size,
                                       kernel_size, dilation, padding_value, stride))


def soft_shrink(self, lambd=0.5):
    return _w(torch.nn.functional.softshrink(_p(self), lambd))


def pinv(self, atol=None, rtol=None, hermitian=False):
    return _w(torch.linalg.pinv(_p(self), atol=atol, rtol=rtol, hermitian=hermitian))


def matrix_determinant(self):
    return _w(torch.linalg.det(_p(self)))


def bucketize(self, boundaries, right=False):
    return _w(torch.bucketize(_p(self), torch.as_tensor(boundaries, dtype=_p(self).dtype), right=right).to(torch.int32))


def to_coo(self):
    from .api import COOTensor
    x = _p(self)
    idx = torch.nonzero(x)
    return COOTensor(idx, x[tuple(idx.t())], tuple(x.shape))


def to_csr(self):
    return to_coo(self).to_csr()


def move_to(self, to, blocking=True):
    if to not in ("CPU", "GPU", "Ascend"):
        raise ValueError("For 'Tensor.move_to', 'to' must be CPU, GPU or Ascend, got %r" % (to,))
    if to == "Ascend":
        raise RuntimeError("this build drives no Ascend device")
    return _w(_p(self).to("cuda" if to == "GPU" else "cpu", non_blocking=not blocking))


def offload(self, file_path):
    """Writes the tensor to ``file_path`` (numpy format) and remembers the path."""
    np.save(file_path, _p(self).float().cpu().numpy() if self.dtype == torch.bfloat16 else _p(self).cpu().numpy())
    self._offload_path = file_path if file_path.endswith(".npy") else file_path + ".npy"
    return True


def offload_file_path(self):
    return getattr(self, "_offload_path", "")


def stub_sync(self):
    if self.is_cuda:
        torch.cuda.current_stream().synchronize()
    return self


def flush_from_cache(self):
    return None


def get_bytes(self):
    t = _p(self).cpu().contiguous()
    return (t.view(torch.uint8) if t.dtype == torch.bfloat16 else t).numpy().tobytes()


def slice_shape(self):
    return tuple(self.shape)


def approximate_equal(self, other, tolerance=1e-5):
    return _w((_p(self) - _p(torch.as_tensor(other))).abs() < tolerance)


def argmax_with_value(self, axis=0, keep_dims=False):
    r = torch.max(_p(self), axis, keep_dims)
    return _w(r.indices.to(torch.int32)), _w(r.values)


def argmin_with_value(self, axis=0, keep_dims=False):
    r = torch.min(_p(self), axis, keep_dims)
    return _w(r.indices.to(torch.int32)), _w(r.values)


def cauchy(self, median=0.0, sigma=1.0):
    return _w(torch.empty_like(_p(self)).cauchy_(median, sigma))


def log_normal(self, mean=1.0, std=2.0):
    return _w(torch.empty_like(_p(self)).log_normal_(mean, std))


def uniform(self, from_=0.0, to=1.0, generator=None):
    return _w(torch.empty_like(_p(self)).uniform_(from_, to))


def eigvals(self):
    return _w(torch.linalg.eigvals(_p(self)))


def fill_diagonal(self, fill_value, wrap=False):
    return _w(_p(self).clone().fill_diagonal_(fill_value, wrap))


def fold(self, output_size, kernel_size, dilation=1, padding=0, stride=1):
    return _w(torch.nn.functional.fold(_p(self), tuple(int(v) for v in torch.as_tensor(output_size).tolist()),
                                       kernel_size, dilation, padding, stride))


def inv(self):
    return _w(torch.reciprocal(_p(self)))


def invert(self):
    return _w(torch.bitwise_not(_p(self)))


def log_matrix_determinant(self):
    sign, logabs = torch.linalg.slogdet(_p(self))
    return _w(sign), _w(logabs)


def reverse(self, axis):
    return _w(torch.flip(_p(self), tuple(axis) if isinstance(axis, (tuple, list)) else (axis,)))


def reverse_sequence(self, seq_lengths, seq_dim=0, batch_dim=0):
    from ..ops.function_ext import reverse_sequence as _rs
    return _rs(self, seq_lengths, seq_dim, batch_dim)


def xdivy(self, y):
    a = _p(self)
    b = _p(torch.as_tensor(y))
    return _w(torch.where(a == 0, torch.zeros_like(a / b), a / b))


def value(self):
    """The tensor held by a Parameter (a Tensor is its own value)."""
    return _w(_p(self).detach())


def is_persistent_data(self):
    return False


def slice_num_of_persistent_data(self):
    return 1


def slice_shape_of_persistent_data(self):
    return tuple(self.shape)


def asnumpy_of_slice_persistent_data(self, param_key, slice_index):
    return _p(self).detach().cpu().numpy()


def _install():
    methods = dict(approximate_equal=approximate_equal, argmax_with_value=argmax_with_value,
                   argmin_with_value=argmin_with_value, cauchy=cauchy, log_normal=log_normal, uniform=uniform,
                   eigvals=eigvals, fill_diagonal=fill_diagonal, fold=fold, inv=inv, invert=invert,
                   log_matrix_determinant=log_matrix_determinant, reverse=reverse, reverse_sequence=reverse_sequence,
                   xdivy=xdivy, value=value, is_persistent_data=is_persistent_data,
                   slice_num_of_persistent_data=slice_num_of_persistent_data,
                   slice_shape_of_persistent_data=slice_shape_of_persistent_data,
                   asnumpy_of_slice_persistent_data=asnumpy_of_slice_persistent_data,
                   itemset=itemset, fills=fills, ptp=ptp, to_tensor=to_tensor, init_check=init_check, choose=choose,
                   searchsorted=searchsorted, gather_nd=gather_nd, inplace_update=inplace_update,
                   random_categorical=random_categorical, one_hot=one_hot, unique_with_pad=unique_with_pad,
                   col2im=col2im, soft_shrink=soft_shrink, pinv=pinv, matrix_determinant=matrix_determinant,
                   bucketize=bucketize, to_coo=to_coo, to_csr=to_csr, move_to=move_to, offload=offload,
                   offload_file_path=offload_file_path, stub_sync=stub_sync, flush_from_cache=flush_from_cache,
                   get_bytes=get_bytes, slice_shape=slice_shape,
                   scatter_sub=_tensor_scatter("TensorScatterSub"), scatter_mul=_tensor_scatter("TensorScatterMul"),
                   scatter_div=_tensor_scatter("TensorScatterDiv"), scatter_max=_tensor_scatter("TensorScatterMax"),
                   scatter_min=_tensor_scatter("TensorScatterMin"),
                   unsorted_segment_sum=_segment("UnsortedSegmentSum"), unsorted_segment_min=_segment("UnsortedSegmentMin"),
                   unsorted_segment_max=_segment("UnsortedSegmentMax"), unsorted_segment_prod=_segment("UnsortedSegmentProd"))
    for name, fn in methods.items():
        if name not in Tensor.__dict__:
            setattr(Tensor, name, fn)
    if "from_numpy" not in Tensor.__dict__:
        Tensor.from_numpy = staticmethod(from_numpy)


_install()
