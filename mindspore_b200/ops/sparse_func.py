"""Functional API on the sparse containers (``COOTensor``, ``CSRTensor``, ``RowTensor``): constructors / accessors,
format conversions, element-wise functions of the stored values (``coo_abs`` ... ``csr_tanh``: zeros stay implicit,
so only functions are meaningful that the reference also applies to the values alone), and the CSR products.

Parity: python/mindspore/ops/function/sparse_func.py, sparse_unary_func.py."""
from __future__ import annotations

import torch
import torch.nn.functional as F

from ..common.api import COOTensor, CSRTensor, RowTensor
from .primitive import _wrap_out


def _t(x):
    return x.as_subclass(torch.Tensor) if isinstance(x, torch.Tensor) else torch.as_tensor(x)


def _need(x, kind, who):
    if not isinstance(x, kind):
        raise TypeError("For '%s', the input must be a %s, but got %s" % (who, kind.__name__, type(x).__name__))


# ---------------------------------------------------------------------------------------------------- make / get
def make_coo_tensor(indices, values, dense_shape):
    return COOTensor(indices, values, dense_shape)


make_sparse_tensor = make_coo_tensor


def make_csr_tensor(indptr, indices, values, dense_shape):
    return CSRTensor(indptr, indices, values, dense_shape)


def make_row_tensor(indices, values, dense_shape):
    return RowTensor(indices, values, dense_shape)


make_row_tensor_inner = make_row_tensor


def make_map_parameter(key_dtype=None, value_dtype=None, value_shape=None, key_tensor=None, value_tensor=None,
                       default_value="normal", **kwargs):
    from ..experimental.map_parameter import MapParameter
    kw = {}
    if key_dtype is not None:
        kw["key_dtype"] = key_dtype
    if value_dtype is not None:
        kw["value_dtype"] = value_dtype
    if value_shape is not None:
        kw["value_shape"] = value_shape
    mp = MapParameter(default_value=default_value, **kw)
    if key_tensor is not None and value_tensor is not None:
        mp.put(key_tensor, value_tensor)
    return mp


def coo_tensor_get_indices(x):
    _need(x, COOTensor, "coo_tensor_get_indices")
    return x.indices


def coo_tensor_get_values(x):
    _need(x, COOTensor, "coo_tensor_get_values")
    return x.values


def coo_tensor_get_dense_shape(x):
    _need(x, COOTensor, "coo_tensor_get_dense_shape")
    return x.shape


def csr_tensor_get_indptr(x):
    _need(x, CSRTensor, "csr_tensor_get_indptr")
    return x.indptr


def csr_tensor_get_indices(x):
    _need(x, CSRTensor, "csr_tensor_get_indices")
    return x.indices


def csr_tensor_get_values(x):
    _need(x, CSRTensor, "csr_tensor_get_values")
    return x.values


def csr_tensor_get_dense_shape(x):
    _need(x, CSRTensor, "csr_tensor_get_dense_shape")
    return x.shape


def row_tensor_get_indices(x):
    _need(x, RowTensor, "row_tensor_get_indices")
    return x.indices


def row_tensor_get_values(x):
    _need(x, RowTensor, "row_tensor_get_values")
    return x.values


def row_tensor_get_dense_shape(x):
    _need(x, RowTensor, "row_tensor_get_dense_shape")
    return x.dense_shape


def row_tensor_add(x, y):
    """Dense tensor ``y`` plus the rows of ``x``."""
    _need(x, RowTensor, "row_tensor_add")
    out = _t(y).clone()
    out.index_add_(0, _t(x.indices).long(), _t(x.values).to(out.dtype))
    return _wrap_out(out)


# ---------------------------------------------------------------------------------------------------- conversions
def dense_to_sparse_coo(tensor):
    t = _t(tensor)
    idx = torch.nonzero(t)
    return COOTensor(idx, t[tuple(idx.t())], tuple(t.shape))


def dense_to_sparse_csr(tensor):
    return dense_to_sparse_coo(tensor).to_csr()


def coo2csr(row_indices, height):
    """Row ids of sorted COO entries -> the CSR row pointer."""
    rows = _t(row_indices).long()
    ptr = torch.zeros(int(height) + 1, dtype=torch.int32)
    ptr[1:] = torch.cumsum(torch.bincount(rows, minlength=int(height)), 0).to(torch.int32)
    return _wrap_out(ptr)


def csr2coo(indptr, nnz):
    ptr = _t(indptr).long()
    rows = torch.repeat_interleave(torch.arange(ptr.numel() - 1), ptr[1:] - ptr[:-1])
    if rows.numel() != int(nnz):
        raise ValueError("For 'csr2coo', 'nnz' (%d) does not match the row pointer (%d entries)"
                         % (int(nnz), rows.numel()))
    return _wrap_out(rows.to(torch.int32))


def csr_to_coo(tensor):
    _need(tensor, CSRTensor, "csr_to_coo")
    return tensor.to_coo()


def csr_to_dense(csr_tensor):
    _need(csr_tensor, CSRTensor, "csr_to_dense")
    return csr_tensor.to_dense()


def coalesce(x_indices, x_values, x_shape):
    """``x_indices`` [ndim, nnz] (the primitive's layout): duplicates summed, entries sorted."""
    t = torch.sparse_coo_tensor(_t(x_indices).long(), _t(x_values), tuple(int(s) for s in _t(x_shape).tolist())
                                if isinstance(x_shape, torch.Tensor) else tuple(x_shape)).coalesce()
    return _wrap_out(t.indices()), _wrap_out(t.values()), _wrap_out(torch.tensor(t.shape, dtype=torch.int64))


# ---------------------------------------------------------------------------------------------------- arithmetic
def coo_add(x1, x2, thresh):
    _need(x1, COOTensor, "coo_add")
    _need(x2, COOTensor, "coo_add")
    return x1.add(x2, float(thresh) if not isinstance(thresh, torch.Tensor) else float(_t(thresh)))


def coo_concat(sp_input, concat_dim=0):
    sp_input = list(sp_input)
    for s in sp_input:
        _need(s, COOTensor, "coo_concat")
    nd = sp_input[0].ndim
    d = concat_dim % nd
    idx, vals, off = [], [], 0
    for s in sp_input:
        i = _t(s.indices).long().clone()
        i[:, d] += off
        off += s.shape[d]
        idx.append(i)
        vals.append(_t(s.values))
    shape = list(sp_input[0].shape)
    shape[d] = off
    return COOTensor(torch.cat(idx), torch.cat(vals), tuple(shape))


def csr_add(a, b, alpha, beta):
    """alpha * a + beta * b."""
    _need(a, CSRTensor, "csr_add")
    _need(b, CSRTensor, "csr_add")
    al = float(_t(alpha)) if isinstance(alpha, torch.Tensor) else float(alpha)
    be = float(_t(beta)) if isinstance(beta, torch.Tensor) else float(beta)
    ca, cb = a.to_coo(), b.to_coo()
    summed = COOTensor(ca.indices, _t(ca.values) * al, ca.shape).add(COOTensor(cb.indices, _t(cb.values) * be, cb.shape))
    return summed.to_csr()


def csr_mul(x, y):
    _need(x, CSRTensor, "csr_mul")
    return x * _t(y)


def csr_div(x, y):
    _need(x, CSRTensor, "csr_div")
    d = _t(y)
    if d.dim() == 0:
        return CSRTensor(x.indptr, x.indices, _t(x.values) / d, x.shape)
    picked = d.expand(x.shape)[x._rows(), _t(x.indices).long()]
    return CSRTensor(x.indptr, x.indices, _t(x.values) / picked, x.shape)


def csr_gather(indptr, indices, dense, sparse_shape):
    """The entries of ``dense`` at the positions a CSR pattern stores."""
    ptr = _t(indptr).long()
    rows = torch.repeat_interleave(torch.arange(ptr.numel() - 1), ptr[1:] - ptr[:-1])
    return _wrap_out(_t(dense)[rows, _t(indices).long()])


def csr_mv(csr_tensor, dense):
    _need(csr_tensor, CSRTensor, "csr_mv")
    return csr_tensor.mv(_t(dense))


def csr_mm(a, b, trans_a=False, trans_b=False, adjoint_a=False, adjoint_b=False):
    _need(a, CSRTensor, "csr_mm")
    d = _t(b)
    if trans_b or adjoint_b:
        d = d.mH if adjoint_b else d.t()
    if trans_a or adjoint_a:
        dense_a = _t(a.to_dense())
        return _wrap_out((dense_a.mH if adjoint_a else dense_a.t()) @ d)
    return a.mm(d)


def csr_reduce_sum(csr_tensor, axis):
    _need(csr_tensor, CSRTensor, "csr_reduce_sum")
    return csr_tensor.sum(axis)


def csr_softmax(logits, dtype=None):
    """Softmax over the stored entries of each row."""
    _need(logits, CSRTensor, "csr_softmax")
    v = _t(logits.values).float()
    rows = logits._rows()
    n = logits.shape[0]
    mx = torch.full((n,), float("-inf")).scatter_reduce(0, rows, v, "amax")
    e = torch.exp(v - mx[rows])
    den = torch.zeros(n).index_add_(0, rows, e)
    out = e / den[rows]
    if dtype is not None:
        from ..common import dtype as mstype
        out = out.to(mstype.to_torch(dtype) if not isinstance(dtype, torch.dtype) else dtype)
    else:
        out = out.to(_t(logits.values).dtype)
    return CSRTensor(logits.indptr, logits.indices, out, logits.shape)


# ---------------------------------------------------------------------------------------------------- unary
_UNARY = {
    "abs": torch.abs, "acos": torch.acos, "acosh": torch.acosh, "asin": torch.asin, "asinh": torch.asinh,
    "atan": torch.atan, "atanh": torch.atanh, "ceil": torch.ceil, "cos": torch.cos, "cosh": torch.cosh,
    "exp": torch.exp, "expm1": torch.expm1, "floor": torch.floor, "inv": torch.reciprocal,
    "isfinite": torch.isfinite, "isinf": torch.isinf, "isnan": torch.isnan, "log": torch.log, "log1p": torch.log1p,
    "neg": torch.neg, "relu": torch.relu, "relu6": F.relu6, "round": torch.round, "sigmoid": torch.sigmoid,
    "sin": torch.sin, "sinh": torch.sinh, "softsign": F.softsign, "sqrt": torch.sqrt, "square": torch.square,
    "tan": torch.tan, "tanh": torch.tanh,
}


def _make_unary(kind, name, fn):
    if kind == "coo":
        def op(x):
            _need(x, COOTensor, "coo_" + name)
            return COOTensor(x.indices, fn(_t(x.values)), x.shape)
    else:
        def op(x):
            _need(x, CSRTensor, "csr_" + name)
            return CSRTensor(x.indptr, x.indices, fn(_t(x.values)), x.shape)
    op.__name__ = "%s_%s" % (kind, name)
    op.__doc__ = "%s of the stored values of a %s." % (name, "COOTensor" if kind == "coo" else "CSRTensor")
    return op


for _kind in ("coo", "csr"):
    for _name, _fn in _UNARY.items():
        globals()["%s_%s" % (_kind, _name)] = _make_unary(_kind, _name, _fn)

__all__ = [n for n in dir() if not n.startswith("_") and n not in ("annotations", "torch", "F", "COOTensor",
                                                                    "CSRTensor", "RowTensor")]
