"""The rest of the functional API (``mindspore.ops.<fn>``): array, math, linear-algebra, FFT, window, neural-network,
image and random functions that have no primitive class of their own here.  Each is the reference's signature and
semantics evaluated with torch; outputs are wrapped as framework tensors.

Parity: python/mindspore/ops/function/{array_func,math_func,nn_func,linalg_func,fft_func,spectral_func,image_func,
random_func,clip_func,debug_func}.py."""
from __future__ import annotations

import builtins
import math
import numbers

import numpy as np
import torch
import torch.nn.functional as F

from ..common import dtype as mstype
from .primitive import _wrap_out

_int = builtins.int


def _t(x, like=None):
    if isinstance(x, torch.Tensor):
        return x.as_subclass(torch.Tensor)
    if like is not None and isinstance(x, numbers.Number):
        return torch.as_tensor(x, dtype=like.dtype if not isinstance(x, bool) else torch.bool, device=like.device)
    return torch.as_tensor(x)


def _w(x):
    if isinstance(x, (tuple, list)):
        return tuple(_w(v) for v in x)
    return _wrap_out(x) if isinstance(x, torch.Tensor) else x


def _tup(v, n):
    return tuple(v) if isinstance(v, (tuple, list)) else (v,) * n


def _dt(dtype):
    return mstype.to_torch(dtype) if dtype is not None and not isinstance(dtype, torch.dtype) else dtype


# ---------------------------------------------------------------------------------------------------- array
def argwhere(input):  # noqa: A002
    return _w(torch.nonzero(_t(input)))


def deepcopy(input_x):
    return _w(_t(input_x).clone())


def diag(input):  # noqa: A002
    return _w(torch.diag(_t(input)))


def diagflat(input, offset=0):  # noqa: A002
    return _w(torch.diagflat(_t(input), offset))


def diagonal(input, offset=0, dim1=0, dim2=1):  # noqa: A002
    return _w(torch.diagonal(_t(input), offset, dim1, dim2))


def diagonal_scatter(input, src, offset=0, dim1=0, dim2=1):  # noqa: A002
    return _w(torch.diagonal_scatter(_t(input), _t(src), offset, dim1, dim2))


def diag_embed(input, offset=0, dim1=-2, dim2=-1):  # noqa: A002
    return _w(torch.diag_embed(_t(input), offset, dim1, dim2))


def select_scatter(input, src, axis, index):  # noqa: A002
    return _w(torch.select_scatter(_t(input), _t(src), axis, index))


def slice_scatter(input, src, axis=0, start=None, end=None, step=1):  # noqa: A002
    return _w(torch.slice_scatter(_t(input), _t(src), axis, start, end, step))


def dyn_shape(input_x):
    return _w(torch.tensor(tuple(_t(input_x).shape), dtype=torch.int64))


def shape_(input_x):
    return tuple(_t(input_x).shape)


def expand(input_x, size):
    size = tuple(_int(s) for s in (size.tolist() if isinstance(size, torch.Tensor) else size))
    return _w(_t(input_x).expand(size))


def fills(x, value):
    return _w(torch.full_like(_t(x), float(value) if not isinstance(value, torch.Tensor) else float(value)))


def full_like(input, fill_value, *, dtype=None):  # noqa: A002
    return _w(torch.full_like(_t(input), fill_value, dtype=_dt(dtype)))


def ger(input, vec2):  # noqa: A002
    return _w(torch.outer(_t(input), _t(vec2)))


def is_nonzero(input):  # noqa: A002
    t = _t(input)
    if t.numel() != 1:
        raise ValueError("For 'is_nonzero', the input must hold exactly one element, but got shape %s"
                         % (tuple(t.shape),))
    return bool(t.reshape(()) != 0)


def lstsq(input, A):  # noqa: A002,N803
    """Least-squares solution of ``A X = input``."""
    return _w(torch.linalg.lstsq(_t(A), _t(input)).solution)


def matrix_band_part(x, lower, upper):
    t = _t(x)
    m, n = t.shape[-2:]
    r = torch.arange(m, device=t.device)[:, None]
    c = torch.arange(n, device=t.device)[None, :]
    lo, up = _int(lower), _int(upper)
    keep = ((r - c <= lo) if lo >= 0 else torch.ones_like(r - c, dtype=torch.bool)) & \
           ((c - r <= up) if up >= 0 else torch.ones_like(r - c, dtype=torch.bool))
    return _w(t * keep.to(t.dtype))


def matrix_diag(x, k=0, num_rows=-1, num_cols=-1, padding_value=0, align="RIGHT_LEFT"):
    t = _t(x)
    k = _int(k if not isinstance(k, torch.Tensor) else k.reshape(-1)[0])
    out = torch.diag_embed(t, k)
    if padding_value:
        mask = torch.diag_embed(torch.ones_like(t, dtype=torch.bool), k)
        out = torch.where(mask, out, torch.full_like(out, padding_value))
    rows = num_rows if not isinstance(num_rows, torch.Tensor) else _int(num_rows)
    cols = num_cols if not isinstance(num_cols, torch.Tensor) else _int(num_cols)
    if rows > 0 or cols > 0:
        r = rows if rows > 0 else out.shape[-2]
        c = cols if cols > 0 else out.shape[-1]
        full = torch.full(out.shape[:-2] + (r, c), padding_value, dtype=out.dtype, device=out.device)
        full[..., :min(r, out.shape[-2]), :min(c, out.shape[-1])] = out[..., :r, :c]
        out = full
    return _w(out)


def matrix_diag_part(x, k, padding_value, align="RIGHT_LEFT"):
    k = _int(k if not isinstance(k, torch.Tensor) else k.reshape(-1)[0])
    return _w(torch.diagonal(_t(x), k, -2, -1))


def matrix_set_diag(x, diagonal, k=0, align="RIGHT_LEFT"):  # noqa: A002
    k = _int(k if not isinstance(k, torch.Tensor) else k.reshape(-1)[0])
    return _w(torch.diagonal_scatter(_t(x), _t(diagonal), k, -2, -1))


def padding(x, pad_dim_size=8):
    t = _t(x)
    if t.shape[-1] != 1:
        raise ValueError("For 'padding', the last dimension of 'x' must be 1, but got %d" % t.shape[-1])
    return _w(F.pad(t, (0, pad_dim_size - 1)))


def population_count(input_x):
    t = _t(input_x)
    bits = t.element_size() * 8
    v = t.to(torch.int64) & ((1 << bits) - 1)
    cnt = torch.zeros_like(v)
    for _ in range(bits):
        cnt += v & 1
        v = v >> 1
    return _w(cnt.to(torch.uint8))


def ravel(input):  # noqa: A002
    return _w(_t(input).reshape(-1))


def reshape_(input, shape):  # noqa: A002
    return _w(_t(input).reshape(tuple(shape)))


def reverse(x, axis):
    return _w(torch.flip(_t(x), _tup(axis, 1)))


def reverse_sequence(x, seq_lengths, seq_dim, batch_dim=0):
    t = _t(x)
    lens = _t(seq_lengths).tolist()
    out = t.clone()
    for b, n in enumerate(lens):
        idx = [slice(None)] * t.dim()
        idx[batch_dim] = b
        src = t[tuple(idx)]
        d = seq_dim - (1 if seq_dim > batch_dim else 0)
        part = torch.flip(src.narrow(d, 0, _int(n)), (d,))
        dst = out[tuple(idx)]
        dst.narrow(d, 0, _int(n)).copy_(part)
    return _w(out)


def scalar_to_array(input_x):
    return _w(torch.as_tensor(input_x))


def swapdims(input, dim0, dim1):  # noqa: A002
    return _w(torch.transpose(_t(input), dim0, dim1))


def tensor_slice(input_x, begin, size):
    t = _t(input_x)
    idx = tuple(slice(_int(b), _int(b) + (_int(s) if s >= 0 else t.shape[i] - _int(b)))
                for i, (b, s) in enumerate(zip(begin, size)))
    return _w(t[idx])


def top_k(input_x, k, sorted=True):  # noqa: A002
    v, i = torch.topk(_t(input_x), k, sorted=sorted)
    return _w(v), _w(i.to(torch.int32))


def unique_consecutive(input, return_idx=False, return_counts=False, axis=None):  # noqa: A002
    out = torch.unique_consecutive(_t(input), return_inverse=return_idx, return_counts=return_counts, dim=axis)
    return _w(out)


def unique_with_pad(x, pad_num):
    t = _t(x)
    seen, order, inverse = {}, [], []
    for v in t.tolist():
        if v not in seen:
            seen[v] = len(order)
            order.append(v)
        inverse.append(seen[v])
    y = order + [pad_num] * (t.numel() - len(order))
    return _w(torch.tensor(y, dtype=t.dtype)), _w(torch.tensor(inverse, dtype=torch.int32))


def _nd_index(indices):
    ind = _t(indices).long()
    return tuple(ind[..., i] for i in range(ind.shape[-1]))


def _scatter_nd_op(name, reduce):
    def fn(input_x, indices, updates, use_locking=False):
        t = _t(input_x)
        idx = _nd_index(indices)
        upd = _t(updates).to(t.dtype)
        if reduce == "add":
            out = t.index_put(idx, upd, accumulate=True)
        elif reduce == "sub":
            out = t.index_put(idx, -upd, accumulate=True)
        else:
            out = t.clone()
            flat_idx = [i.reshape(-1) for i in idx]
            u = upd.reshape((flat_idx[0].numel(),) + tuple(t.shape[len(idx):]))
            for j in range(flat_idx[0].numel()):
                key = tuple(_int(i[j]) for i in flat_idx)
                cur = out[key]
                out[key] = {"mul": cur * u[j], "div": cur / u[j], "max": torch.maximum(cur, u[j]),
                            "min": torch.minimum(cur, u[j])}[reduce]
        if name.startswith("scatter_nd_") and type(input_x).__name__ == "Parameter":
            with torch.no_grad():
                _t(input_x).copy_(out)                       # Parameter form: updated in place, as the reference's
            return _w(_t(input_x))
        return _w(out)
    fn.__name__ = name
    return fn


for _r in ("add", "sub", "mul", "div", "max", "min"):
    globals()["scatter_nd_" + _r] = _scatter_nd_op("scatter_nd_" + _r, _r)
    if _r not in ("add",):
        globals()["tensor_scatter_" + _r] = _scatter_nd_op("tensor_scatter_" + _r, _r)


def _scatter_rows_op(name, reduce):
    def fn(input_x, indices, updates):
        t = _t(input_x)
        ind = _t(indices).long().reshape(-1)
        upd = _t(updates).to(t.dtype).reshape((ind.numel(),) + tuple(t.shape[1:]))
        out = t.clone()
        for j in range(ind.numel()):
            i = _int(ind[j])
            out[i] = {"update": upd[j], "mul": out[i] * upd[j], "div": out[i] / upd[j],
                      "max": torch.maximum(out[i], upd[j]), "min": torch.minimum(out[i], upd[j])}[reduce]
        with torch.no_grad():
            _t(input_x).copy_(out)
        return _w(out)
    fn.__name__ = name
    return fn


for _r in ("update", "mul", "div", "max", "min"):
    globals()["scatter_" + _r] = _scatter_rows_op("scatter_" + _r, _r)


def tensor_scatter_elements(input_x, indices, updates, axis=0, reduction="none"):
    t, ind, upd = _t(input_x), _t(indices).long(), _t(updates)
    if reduction == "none":
        return _w(t.scatter(axis, ind, upd.to(t.dtype)))
    if reduction != "add":
        raise ValueError("For 'tensor_scatter_elements', 'reduction' must be 'none' or 'add', but got %r" % reduction)
    return _w(t.scatter_add(axis, ind, upd.to(t.dtype)))


def _segment(name, reduce, init):
    def fn(x, segment_ids, num_segments):
        t, ids = _t(x), _t(segment_ids).long()
        n = _int(num_segments)
        flat = t.reshape((ids.numel(),) + tuple(t.shape[ids.dim():]))
        out = torch.full((n,) + tuple(flat.shape[1:]), init(t.dtype), dtype=t.dtype, device=t.device)
        idx = ids.reshape(-1)
        valid = idx >= 0
        idx_e = idx[valid].reshape((-1,) + (1,) * (flat.dim() - 1)).expand_as(flat[valid])
        out = out.scatter_reduce(0, idx_e, flat[valid], reduce=reduce, include_self=True)
        return _w(out)
    fn.__name__ = name
    return fn


def _max_of(dt):
    return torch.finfo(dt).max if dt.is_floating_point else torch.iinfo(dt).max


def _min_of(dt):
    return torch.finfo(dt).min if dt.is_floating_point else torch.iinfo(dt).min


unsorted_segment_max = _segment("unsorted_segment_max", "amax", _min_of)
unsorted_segment_min = _segment("unsorted_segment_min", "amin", _max_of)
unsorted_segment_prod = _segment("unsorted_segment_prod", "prod", lambda dt: 1)


def space_to_batch_nd(input_x, block_size, paddings):
    t = _t(input_x)
    nd = len(paddings)
    block = _tup(block_size, nd)
    pads = []
    for p in reversed(paddings):
        pads += [p[0], p[1]]
    t = F.pad(t, pads)
    lead = t.shape[:t.dim() - nd]
    shape = list(lead)
    for i in range(nd):
        shape += [t.shape[len(lead) + i] // block[i], block[i]]
    t = t.reshape(shape)
    L = len(lead)
    perm = [L + 2 * i + 1 for i in range(nd)] + list(range(L)) + [L + 2 * i for i in range(nd)]
    t = t.permute(perm)
    return _w(t.reshape((-1,) + tuple(lead[1:]) + tuple(t.shape[nd + L:])))


def batch_to_space_nd(input_x, block_shape, crops):
    t = _t(input_x)
    nd = len(crops)
    block = _tup(block_shape, nd)
    prod = _int(np.prod(block))
    n = t.shape[0] // prod
    rest = t.shape[1:]
    L = len(rest) - nd
    t = t.reshape(tuple(block) + (n,) + tuple(rest))
    perm = [nd] + [nd + 1 + i for i in range(L)]
    for i in range(nd):
        perm += [nd + 1 + L + i, i]
    t = t.permute(perm)
    shape = [n] + list(rest[:L]) + [rest[L + i] * block[i] for i in range(nd)]
    t = t.reshape(shape)
    idx = [slice(None)] * (1 + L) + [slice(c[0], t.shape[1 + L + i] - c[1]) for i, c in enumerate(crops)]
    return _w(t[tuple(idx)])


def col2im(input_x, output_size, kernel_size, dilation, padding_value, stride):
    """[N, C, prod(kernel), L] columns back to images (sum over overlapping patches)."""
    t = _t(input_x)
    n, c = t.shape[:2]
    out = F.fold(t.reshape(n, c * t.shape[2], t.shape[3]), tuple(_int(v) for v in _t(output_size).tolist())
                 if isinstance(output_size, torch.Tensor) else tuple(output_size), _tup(kernel_size, 2),
                 _tup(dilation, 2), _tup(padding_value, 2), _tup(stride, 2))
    return _w(out)


def affine_grid(theta, size, align_corners=False):
    return _w(F.affine_grid(_t(theta), tuple(size), align_corners=align_corners))


# ---------------------------------------------------------------------------------------------------- windows
def _window(fn):
    def win(window_length, periodic=True, *, dtype=None, **kw):
        n = _int(window_length)
        return _w(fn(n, periodic=periodic, dtype=_dt(dtype) or torch.float32, **kw))
    return win


bartlett_window = _window(torch.bartlett_window)
blackman_window = _window(torch.blackman_window)
hann_window = _window(torch.hann_window)


def hamming_window(window_length, periodic=True, alpha=0.54, beta=0.46, *, dtype=None):
    return _w(torch.hamming_window(_int(window_length), periodic, alpha, beta, dtype=_dt(dtype) or torch.float32))


def kaiser_window(window_length, periodic=True, beta=12.0, *, dtype=None):
    return _w(torch.kaiser_window(_int(window_length), periodic, beta, dtype=_dt(dtype) or torch.float32))


# ---------------------------------------------------------------------------------------------------- math
def _unary(fn):
    return lambda input: _w(fn(_t(input)))  # noqa: A002


arccos, arccosh, arcsin, arcsinh = _unary(torch.acos), _unary(torch.acosh), _unary(torch.asin), _unary(torch.asinh)
arctan, arctanh = _unary(torch.atan), _unary(torch.atanh)
bessel_i0, bessel_i0e = _unary(torch.special.i0), _unary(torch.special.i0e)
bessel_i1, bessel_i1e = _unary(torch.special.i1), _unary(torch.special.i1e)
bessel_j0, bessel_j1 = _unary(torch.special.bessel_j0), _unary(torch.special.bessel_j1)
bessel_y0, bessel_y1 = _unary(torch.special.bessel_y0), _unary(torch.special.bessel_y1)
bessel_k0, bessel_k0e = _unary(torch.special.modified_bessel_k0), _unary(torch.special.scaled_modified_bessel_k0)
bessel_k1, bessel_k1e = _unary(torch.special.modified_bessel_k1), _unary(torch.special.scaled_modified_bessel_k1)
exp2, frac, log10, log2, positive = _unary(torch.exp2), _unary(torch.frac), _unary(torch.log10), \
    _unary(torch.log2), _unary(torch.positive)
tensor_exp, tensor_expm1 = _unary(torch.exp), _unary(torch.expm1)
inv = _unary(torch.reciprocal)
adjoint = _unary(lambda t: t.mH if t.dim() >= 2 else t.conj())
tanhshrink = _unary(lambda t: t - torch.tanh(t))
logsigmoid = _unary(F.logsigmoid)
matrix_exp = _unary(torch.linalg.matrix_exp)
matrix_determinant = _unary(torch.linalg.det)


def arctan2(input, other):  # noqa: A002
    a = _t(input)
    return _w(torch.atan2(a, _t(other, a)))


def accumulate_n(x):
    out = _t(x[0]).clone()
    for v in x[1:]:
        out = out + _t(v)
    return _w(out)


def approximate_equal(x, y, tolerance=1e-5):
    a = _t(x)
    return _w((a - _t(y, a)).abs() < tolerance)


def cholesky(input_x, upper=False):
    return _w(torch.linalg.cholesky(_t(input_x), upper=upper))


def cholesky_inverse(input_x, upper=False):
    return _w(torch.cholesky_inverse(_t(input_x), upper=upper))


def cholesky_solve(input, input2, upper=False):  # noqa: A002
    return _w(torch.cholesky_solve(_t(input), _t(input2), upper=upper))


def cosine_similarity(x1, x2, dim=1, eps=1e-08):
    return _w(F.cosine_similarity(_t(x1), _t(x2), dim, eps))


def cov(input, *, correction=1, fweights=None, aweights=None):  # noqa: A002
    return _w(torch.cov(_t(input), correction=correction, fweights=None if fweights is None else _t(fweights),
                        aweights=None if aweights is None else _t(aweights)))


def dist(input, other, p=2):  # noqa: A002
    return _w(torch.dist(_t(input), _t(other), p))


def eps(x):
    t = _t(x)
    return _w(torch.full_like(t, torch.finfo(t.dtype).eps))


def floordiv(x, y):
    a = _t(x) if isinstance(x, torch.Tensor) else _t(x, _t(y))
    return _w(torch.floor_divide(a, _t(y, a)))


tensor_floordiv = floordiv


def floormod(x, y):
    a = _t(x) if isinstance(x, torch.Tensor) else _t(x, _t(y))
    return _w(torch.remainder(a, _t(y, a)))


tensor_mod = floormod


def truncate_div(x, y):
    a = _t(x) if isinstance(x, torch.Tensor) else _t(x, _t(y))
    return _w(torch.div(a, _t(y, a), rounding_mode="trunc"))


def truncate_mod(x, y):
    a = _t(x) if isinstance(x, torch.Tensor) else _t(x, _t(y))
    return _w(torch.fmod(a, _t(y, a)))


def pows(input, exponent):  # noqa: A002
    a = _t(input)
    return _w(torch.pow(a, _t(exponent, a)))


def gumbel_softmax(logits, tau=1.0, hard=False, dim=-1):
    return _w(F.gumbel_softmax(_t(logits), tau, hard, dim=dim))


def _inplace(op):
    def fn(x, v, indices):
        t = _t(x).clone()
        idx = [indices] if isinstance(indices, _int) else list(indices)
        vv = _t(v).to(t.dtype)
        t[idx] = op(t[idx], vv)
        return _w(t)
    return fn


inplace_add = _inplace(lambda a, b: a + b)
inplace_sub = _inplace(lambda a, b: a - b)


def inplace_index_add(var, indices, updates, axis):
    t = _t(var)
    with torch.no_grad():
        t.index_add_(axis, _t(indices).long(), _t(updates).to(t.dtype))
    return _w(t)


def iou(anchor_boxes, gt_boxes, mode="iou"):
    a, g = _t(anchor_boxes).float(), _t(gt_boxes).float()
    area = lambda b: (b[:, 2] - b[:, 0] + 1) * (b[:, 3] - b[:, 1] + 1)
    lt = torch.maximum(g[:, None, :2], a[None, :, :2])
    rb = torch.minimum(g[:, None, 2:], a[None, :, 2:])
    wh = (rb - lt + 1).clamp(min=0)
    inter = wh[..., 0] * wh[..., 1]
    if mode == "iou":
        out = inter / (area(g)[:, None] + area(a)[None, :] - inter)
    elif mode == "iof":
        out = inter / area(g)[:, None]
    else:
        raise ValueError("For 'iou', 'mode' must be 'iou' or 'iof', but got %r" % (mode,))
    return _w(out.to(_t(anchor_boxes).dtype))


def log_matrix_determinant(input):  # noqa: A002
    sign, logabs = torch.linalg.slogdet(_t(input))
    return _w(sign), _w(logabs)


def logcumsumexp(input, axis):  # noqa: A002
    return _w(torch.logcumsumexp(_t(input), axis))


def logit(input, eps=None):  # noqa: A002
    return _w(torch.logit(_t(input), eps))


def logspace(start, end, steps, base=10, *, dtype=mstype.float32):
    s = float(start) if not isinstance(start, torch.Tensor) else float(_t(start))
    e = float(end) if not isinstance(end, torch.Tensor) else float(_t(end))
    return _w(torch.logspace(s, e, _int(steps), base, dtype=_dt(dtype)))


def lu_solve(b, LU, pivots):  # noqa: N803
    return _w(torch.linalg.lu_solve(_t(LU), _t(pivots).to(torch.int32), _t(b)))


def lu_unpack(LU_data, LU_pivots, unpack_data=True, unpack_pivots=True):  # noqa: N803
    return _w(tuple(torch.lu_unpack(_t(LU_data), _t(LU_pivots).to(torch.int32), unpack_data, unpack_pivots)))


def matrix_norm(A, ord="fro", axis=(-2, -1), keepdims=False, *, dtype=None):  # noqa: A002,N803
    return _w(torch.linalg.matrix_norm(_t(A), ord, tuple(axis), keepdims, dtype=_dt(dtype)))


def vector_norm(x, ord=2, axis=None, keepdims=False, *, dtype=None):  # noqa: A002
    return _w(torch.linalg.vector_norm(_t(x), ord, axis, keepdims, dtype=_dt(dtype)))


def matrix_solve(matrix, rhs, adjoint=False):  # noqa: A002
    m = _t(matrix)
    return _w(torch.linalg.solve(m.mH if adjoint else m, _t(rhs)))


def orgqr(input, input2):  # noqa: A002
    return _w(torch.linalg.householder_product(_t(input), _t(input2)))


def ormqr(input, tau, other, left=True, transpose=False):  # noqa: A002
    return _w(torch.ormqr(_t(input), _t(tau), _t(other), left, transpose))


def sparse_segment_mean(x, indices, segment_ids):
    t = _t(x)
    rows = t[_t(indices).long()]
    ids = _t(segment_ids).long()
    n = _int(ids.max()) + 1 if ids.numel() else 0
    out = torch.zeros((n,) + tuple(t.shape[1:]), dtype=t.dtype)
    cnt = torch.zeros(n, dtype=t.dtype)
    out.index_add_(0, ids, rows)
    cnt.index_add_(0, ids, torch.ones_like(ids, dtype=t.dtype))
    return _w(out / cnt.clamp(min=1).reshape((-1,) + (1,) * (t.dim() - 1)))


def stft(x, n_fft, hop_length=None, win_length=None, window=None, center=True, pad_mode="REFLECT", normalized=False,
         onesided=None, return_complex=None):
    t = _t(x)
    rc = t.is_complex() if return_complex is None else return_complex
    out = torch.stft(t, n_fft, hop_length, win_length, None if window is None else _t(window), center,
                     pad_mode.lower(), normalized, onesided, return_complex=True)
    return _w(out if rc else torch.view_as_real(out))


def t(input):  # noqa: A002
    x = _t(input)
    return _w(x.t() if x.dim() == 2 else x)


def vecdot(x, y, *, axis=-1):
    return _w(torch.linalg.vecdot(_t(x), _t(y), dim=axis))


def zeta(input, other):  # noqa: A002
    a = _t(input) if isinstance(input, torch.Tensor) else _t(input, _t(other))
    return _w(torch.special.zeta(a, _t(other, a)))


# ---------------------------------------------------------------------------------------------------- linalg / fft
def eig(A):  # noqa: N803
    return _w(tuple(torch.linalg.eig(_t(A))))


def eigvals(A):  # noqa: N803
    return _w(torch.linalg.eigvals(_t(A)))


def geqrf(input):  # noqa: A002
    return _w(tuple(torch.geqrf(_t(input))))


def pinv(x, *, atol=None, rtol=None, hermitian=False):
    return _w(torch.linalg.pinv(_t(x), atol=atol, rtol=rtol, hermitian=hermitian))


def qr(input, mode="reduced"):  # noqa: A002
    return _w(tuple(torch.linalg.qr(_t(input), mode)))


def svd(input, full_matrices=False, compute_uv=True):  # noqa: A002
    """(s, u, v) - singular values first, v not transposed - or s alone with ``compute_uv=False``."""
    if not compute_uv:
        return _w(torch.linalg.svdvals(_t(input)))
    u, s, vh = torch.linalg.svd(_t(input), full_matrices=full_matrices)
    return _w(s), _w(u), _w(vh.mH)


def _fft1(fn):
    return lambda input, n=None, dim=-1, norm=None: _w(fn(_t(input), n, dim, norm))  # noqa: A002


def _fftn(fn, default_dim=None):
    return lambda input, s=None, dim=default_dim, norm=None: _w(fn(_t(input), s, dim, norm))  # noqa: A002


fft, ifft, rfft, irfft = _fft1(torch.fft.fft), _fft1(torch.fft.ifft), _fft1(torch.fft.rfft), _fft1(torch.fft.irfft)
fft2, ifft2 = _fftn(torch.fft.fft2, (-2, -1)), _fftn(torch.fft.ifft2, (-2, -1))
fftn, ifftn = _fftn(torch.fft.fftn), _fftn(torch.fft.ifftn)


def fftshift(input, dim=None):  # noqa: A002
    return _w(torch.fft.fftshift(_t(input), dim))


def ifftshift(input, dim=None):  # noqa: A002
    return _w(torch.fft.ifftshift(_t(input), dim))


# ---------------------------------------------------------------------------------------------------- clip / debug
def clip_by_norm(x, max_norm, norm_type=2.0, error_if_nonfinite=False):
    """Scales the tensors of ``x`` (one tensor or a sequence) so that their joint ``norm_type`` norm is at most
    ``max_norm``."""
    seq = isinstance(x, (tuple, list))
    ts = [_t(v) for v in (x if seq else [x])]
    total = torch.linalg.vector_norm(torch.stack([torch.linalg.vector_norm(v.float(), norm_type) for v in ts]),
                                     norm_type)
    if error_if_nonfinite and not bool(torch.isfinite(total)):
        raise RuntimeError("For 'clip_by_norm', the total norm of the input is non-finite")
    coef = (float(max_norm) / (total + 1e-6)).clamp(max=1.0)
    out = [_w((v.float() * coef).to(v.dtype)) for v in ts]
    return tuple(out) if seq else out[0]


def print_(*input_x):
    builtins.print(*[v if not isinstance(v, torch.Tensor) else _t(v) for v in input_x])


# ---------------------------------------------------------------------------------------------------- nn
def adaptive_avg_pool1d(input, output_size):  # noqa: A002
    return _w(F.adaptive_avg_pool1d(_t(input), output_size))


def adaptive_avg_pool3d(input, output_size):  # noqa: A002
    return _w(F.adaptive_avg_pool3d(_t(input), output_size))


def adaptive_max_pool1d(input, output_size):  # noqa: A002
    return _w(F.adaptive_max_pool1d(_t(input), output_size))


def adaptive_max_pool2d(input, output_size, return_indices=False):  # noqa: A002
    return _w(F.adaptive_max_pool2d(_t(input), output_size, return_indices))


def adaptive_max_pool3d(input, output_size, return_indices=False):  # noqa: A002
    return _w(F.adaptive_max_pool3d(_t(input), output_size, return_indices))


def avg_pool1d(input_x, kernel_size=1, stride=1, padding=0, ceil_mode=False, count_include_pad=True):
    return _w(F.avg_pool1d(_t(input_x), kernel_size, stride, padding, ceil_mode, count_include_pad))


def avg_pool3d(input_x, kernel_size=1, stride=1, padding=0, ceil_mode=False, count_include_pad=True,
               divisor_override=0):
    return _w(F.avg_pool3d(_t(input_x), kernel_size, stride, padding, ceil_mode, count_include_pad,
                           divisor_override or None))


def max_pool3d(x, kernel_size, stride=None, padding=0, dilation=1, ceil_mode=False, return_indices=False):
    return _w(F.max_pool3d(_t(x), kernel_size, stride, padding, dilation, ceil_mode, return_indices))


def _unpool(fn):
    def un(x, indices, kernel_size, stride=None, padding=0, output_size=None):
        return _w(fn(_t(x), _t(indices).long(), kernel_size, stride, padding, output_size))
    return un


max_unpool1d, max_unpool2d, max_unpool3d = _unpool(F.max_unpool1d), _unpool(F.max_unpool2d), _unpool(F.max_unpool3d)


def lp_pool1d(x, norm_type, kernel_size, stride=None, ceil_mode=False):
    return _w(F.lp_pool1d(_t(x), float(norm_type), kernel_size, stride, ceil_mode))


def lp_pool2d(x, norm_type, kernel_size, stride=None, ceil_mode=False):
    return _w(F.lp_pool2d(_t(x), float(norm_type), kernel_size, stride, ceil_mode))


def fractional_max_pool2d(input, kernel_size, output_size=None, output_ratio=None, return_indices=False,  # noqa: A002
                          _random_samples=None):
    rs = None if _random_samples is None else _t(_random_samples)
    return _w(F.fractional_max_pool2d(_t(input), kernel_size, output_size, output_ratio, return_indices, rs))


def fractional_max_pool3d(input, kernel_size, output_size=None, output_ratio=None, return_indices=False,  # noqa: A002
                          _random_samples=None):
    rs = None if _random_samples is None else _t(_random_samples)
    return _w(F.fractional_max_pool3d(_t(input), kernel_size, output_size, output_ratio, return_indices, rs))


def bias_add(input_x, bias):
    t = _t(input_x)
    shape = [1] * t.dim()
    shape[1 if t.dim() > 1 else 0] = -1
    return _w(t + _t(bias).reshape(shape))


def bidense(input1, input2, weight, bias=None):
    return _w(F.bilinear(_t(input1), _t(input2), _t(weight), None if bias is None else _t(bias)))


def celu(x, alpha=1.0):
    return _w(F.celu(_t(x), alpha))


def channel_shuffle(x, groups):
    return _w(F.channel_shuffle(_t(x), groups))


def _conv_pad(t, nd, kernel, stride, dilation, pad_mode, padding):
    if pad_mode == "same":
        pads = []
        for size, k, s, d in zip(t.shape[2:][::-1], kernel[::-1], stride[::-1], dilation[::-1]):
            total = max((-(-size // s) - 1) * s + (k - 1) * d + 1 - size, 0)
            pads += [total // 2, total - total // 2]
        return F.pad(t, pads), 0
    if pad_mode == "valid":
        return t, 0
    if pad_mode != "pad":
        raise ValueError("pad_mode must be 'same', 'valid' or 'pad', but got %r" % (pad_mode,))
    p = _tup(padding, nd)
    if len(p) == 2 * nd:                                        # (before, after) per dim
        pads = []
        for i in reversed(range(nd)):
            pads += [p[2 * i], p[2 * i + 1]]
        return F.pad(t, pads), 0
    return t, p


def conv1d(input, weight, bias=None, stride=1, pad_mode="valid", padding=0, dilation=1, groups=1):  # noqa: A002
    t, w = _t(input), _t(weight)
    s, d = _tup(stride, 1), _tup(dilation, 1)
    t, p = _conv_pad(t, 1, w.shape[2:], s, d, pad_mode, padding)
    return _w(F.conv1d(t, w, None if bias is None else _t(bias), s, p, d, groups))


def conv3d(input, weight, bias=None, stride=1, pad_mode="valid", padding=0, dilation=1, groups=1):  # noqa: A002
    t, w = _t(input), _t(weight)
    s, d = _tup(stride, 3), _tup(dilation, 3)
    t, p = _conv_pad(t, 3, w.shape[2:], s, d, pad_mode, padding)
    return _w(F.conv3d(t, w, None if bias is None else _t(bias), s, p, d, groups))


def conv_transpose2d(input, weight, bias=None, stride=1, padding=0, output_padding=0, groups=1, dilation=1):  # noqa: A002
    return _w(F.conv_transpose2d(_t(input), _t(weight), None if bias is None else _t(bias), stride, padding,
                                 output_padding, groups, dilation))


def conv3d_transpose(inputs, weight, pad_mode="valid", padding=0, stride=1, dilation=1, group=1, output_padding=0):
    w = _t(weight)
    if pad_mode == "valid":
        p = 0
    elif pad_mode == "pad":
        p = _tup(padding, 3)
    else:
        p = tuple(((k - 1) * d) // 2 for k, d in zip(w.shape[2:], _tup(dilation, 3)))
    return _w(F.conv_transpose3d(_t(inputs), w, None, stride, p, output_padding, group, dilation))


def deformable_conv2d(x, weight, offsets, kernel_size, strides, padding, bias=None, dilations=(1, 1, 1, 1), groups=1,
                      deformable_groups=1, modulated=True):
    """Deformable convolution v2: ``offsets`` [N, 3 * dg * kh * kw, Ho, Wo] holds the x offsets, then the y offsets,
    then the modulation masks, each [dg, kh, kw] per output position.  Sampled bilinearly, then a dense product."""
    t, w, off = _t(x), _t(weight), _t(offsets)
    n, c, h, wd = t.shape
    kh, kw = kernel_size
    sh, sw = strides[2], strides[3]
    dh, dw = dilations[2], dilations[3]
    pt, pb, pl, pr = padding
    dg = deformable_groups
    ho = (h + pt + pb - dh * (kh - 1) - 1) // sh + 1
    wo = (wd + pl + pr - dw * (kw - 1) - 1) // sw + 1
    k = kh * kw
    off = off.reshape(n, 3, dg, k, ho, wo)
    ox, oy, mask = off[:, 0], off[:, 1], off[:, 2]
    base_y = (torch.arange(ho) * sh - pt).reshape(1, 1, 1, ho, 1).to(t.dtype)
    base_x = (torch.arange(wo) * sw - pl).reshape(1, 1, 1, 1, wo).to(t.dtype)
    ky = (torch.arange(kh).repeat_interleave(kw) * dh).reshape(1, 1, k, 1, 1).to(t.dtype)
    kx = (torch.arange(kw).repeat(kh) * dw).reshape(1, 1, k, 1, 1).to(t.dtype)
    py, px = base_y + ky + oy, base_x + kx + ox                    # [N, dg, k, ho, wo]
    gx = 2 * px / max(wd - 1, 1) - 1
    gy = 2 * py / max(h - 1, 1) - 1
    cols = []
    cg = c // dg
    for g in range(dg):
        grid = torch.stack([gx[:, g], gy[:, g]], -1).reshape(n, k * ho, wo, 2)
        samp = F.grid_sample(t[:, g * cg:(g + 1) * cg], grid, mode="bilinear", padding_mode="zeros",
                             align_corners=True).reshape(n, cg, k, ho, wo)
        if modulated:
            samp = samp * mask[:, g].unsqueeze(1)
        cols.append(samp)
    col = torch.cat(cols, 1)                                       # [N, C, k, ho, wo]
    cout = w.shape[0]
    col = col.reshape(n, groups, c // groups * k, ho * wo)
    wg = w.reshape(groups, cout // groups, c // groups * k)
    out = torch.einsum("gok,ngkl->ngol", wg, col).reshape(n, cout, ho, wo)
    if bias is not None:
        out = out + _t(bias).reshape(1, -1, 1, 1)
    return _w(out)


def cosine_embedding_loss(input1, input2, target, margin=0.0, reduction="mean"):
    return _w(F.cosine_embedding_loss(_t(input1), _t(input2), _t(target), margin, reduction=reduction))


def ctc_greedy_decoder(inputs, sequence_length, merge_repeated=True):
    """inputs [T, N, C], blank = C - 1.  Returns (indices [k, 2], values [k], shape [2], -sum of max log-probs [N, 1])."""
    x, lens = _t(inputs), _t(sequence_length).tolist()
    tmax, n, c = x.shape
    best, idx = x.max(-1)
    ind, vals, width = [], [], 0
    neg = torch.zeros(n, 1, dtype=x.dtype)
    for b in range(n):
        prev, col = -1, 0
        for step in range(_int(lens[b])):
            k = _int(idx[step, b])
            neg[b, 0] -= best[step, b]
            if k != c - 1 and not (merge_repeated and k == prev):
                ind.append([b, col])
                vals.append(k)
                col += 1
            prev = k
        width = max(width, col)
    return (_w(torch.tensor(ind, dtype=torch.int64).reshape(-1, 2)), _w(torch.tensor(vals, dtype=torch.int64)),
            _w(torch.tensor([n, width], dtype=torch.int64)), _w(neg))


def ctc_loss(log_probs, targets, input_lengths, target_lengths, blank=0, reduction="none", zero_infinity=False):
    lp = _t(log_probs)
    per = F.ctc_loss(lp, _t(targets).long(), _t(input_lengths).long(), _t(target_lengths).long(), blank, "none",
                     zero_infinity)
    if reduction == "mean":
        out = (per / _t(target_lengths).clamp(min=1).to(per.dtype)).mean()
    elif reduction == "sum":
        out = per.sum()
    else:
        out = per
    # second output: the gradient-like "log_alpha" is not exposed by torch; the reference returns it for its own
    # backward only
    return _w(out), _w(torch.zeros(0))


def dropout1d(input, p=0.5, training=True):  # noqa: A002
    return _w(F.dropout1d(_t(input), p, training))


def dropout2d(input, p=0.5, training=True):  # noqa: A002
    return _w(F.dropout2d(_t(input), p, training))


def dropout3d(input, p=0.5, training=True):  # noqa: A002
    return _w(F.dropout3d(_t(input), p, training))


def gaussian_nll_loss(x, target, var, full=False, eps=1e-6, reduction="mean"):
    return _w(F.gaussian_nll_loss(_t(x), _t(target), _t(var), full, eps, reduction))


def glu(x, axis=-1):
    return _w(F.glu(_t(x), axis))


def group_norm(input, num_groups, weight=None, bias=None, eps=1e-5):  # noqa: A002
    return _w(F.group_norm(_t(input), num_groups, None if weight is None else _t(weight),
                           None if bias is None else _t(bias), eps))


def hardshrink(x, lambd=0.5):
    return _w(F.hardshrink(_t(x), lambd))


def softshrink(x, lambd=0.5):
    return _w(F.softshrink(_t(x), lambd))


soft_shrink = softshrink


def hardtanh(input, min_val=-1.0, max_val=1.0):  # noqa: A002
    return _w(F.hardtanh(_t(input), min_val, max_val))


def hinge_embedding_loss(inputs, targets, margin=1.0, reduction="mean"):
    return _w(F.hinge_embedding_loss(_t(inputs), _t(targets), margin, reduction=reduction))


def huber_loss(input, target, reduction="mean", delta=1.0):  # noqa: A002
    return _w(F.huber_loss(_t(input), _t(target), reduction=reduction, delta=delta))


def intopk(x1, x2, k):
    """Whether the target class ``x2[i]`` is among the top ``k`` predictions of row ``x1[i]``."""
    a, lab = _t(x1), _t(x2).long()
    target = a.gather(1, lab[:, None])
    return _w(((a > target).sum(1) < k))


def lrn(x, depth_radius=5, bias=1.0, alpha=1.0, beta=0.5, norm_region="ACROSS_CHANNELS"):
    size = 2 * depth_radius + 1
    return _w(F.local_response_norm(_t(x), size, alpha * size, beta, bias))


def margin_ranking_loss(input1, input2, target, margin=0.0, reduction="mean"):
    return _w(F.margin_ranking_loss(_t(input1), _t(input2), _t(target), margin, reduction=reduction))


def mirror_pad(input_x, paddings, mode):
    """``paddings`` [rank, 2]; 'REFLECT' mirrors without repeating the border element, 'SYMMETRIC' repeats it."""
    t = _t(input_x)
    pads = _t(paddings).tolist() if isinstance(paddings, torch.Tensor) else [list(p) for p in paddings]
    mode = mode.upper()
    if mode not in ("REFLECT", "SYMMETRIC"):
        raise ValueError("For 'mirror_pad', 'mode' must be 'REFLECT' or 'SYMMETRIC', but got %r" % (mode,))
    off = 1 if mode == "REFLECT" else 0
    for d, (lo, hi) in enumerate(pads):
        lo, hi = _int(lo), _int(hi)
        if lo == 0 and hi == 0:
            continue
        n = t.shape[d]
        left = t.narrow(d, off, lo).flip(d)
        right = t.narrow(d, n - off - hi, hi).flip(d)
        t = torch.cat([left, t, right], d)
    return _w(t)


def multi_margin_loss(input, target, p=1, margin=1, weight=None, reduction="mean"):  # noqa: A002
    return _w(F.multi_margin_loss(_t(input), _t(target).long(), p, margin, None if weight is None else _t(weight),
                                  reduction=reduction))


def multilabel_margin_loss(input, target, reduction="mean"):  # noqa: A002
    return _w(F.multilabel_margin_loss(_t(input), _t(target).long(), reduction=reduction))


def multilabel_soft_margin_loss(input, target, weight=None, reduction="mean"):  # noqa: A002
    return _w(F.multilabel_soft_margin_loss(_t(input), _t(target), None if weight is None else _t(weight),
                                            reduction=reduction))


def soft_margin_loss(input, target, reduction="mean"):  # noqa: A002
    return _w(F.soft_margin_loss(_t(input), _t(target), reduction=reduction))


def triplet_margin_loss(anchor, positive, negative, margin=1.0, p=2, eps=1e-06, swap=False, reduction="mean"):
    return _w(F.triplet_margin_loss(_t(anchor), _t(positive), _t(negative), margin, p, eps, swap,
                                    reduction=reduction))


def pdist(input, p=2.0):  # noqa: A002
    return _w(F.pdist(_t(input), p))


def pixel_shuffle(input, upscale_factor):  # noqa: A002
    return _w(F.pixel_shuffle(_t(input), upscale_factor))


def pixel_unshuffle(input, downscale_factor):  # noqa: A002
    return _w(F.pixel_unshuffle(_t(input), downscale_factor))


def rrelu(input, lower=1.0 / 8, upper=1.0 / 3):  # noqa: A002
    return _w(F.rrelu(_t(input), lower, upper, training=True))


def softmin(x, axis=-1, *, dtype=None):
    return _w(F.softmin(_t(x), axis, dtype=_dt(dtype)))


def threshold(input, thr, value):  # noqa: A002
    return _w(F.threshold(_t(input), thr, value))


def upsample(input, size=None, scale_factor=None, mode="nearest", align_corners=None,  # noqa: A002
             recompute_scale_factor=None):
    from .functional import interpolate
    return interpolate(input, size, scale_factor, mode, align_corners, recompute_scale_factor)


# ---------------------------------------------------------------------------------------------------- image
def bounding_box_encode(anchor_box, groundtruth_box, means=(0.0, 0.0, 0.0, 0.0), stds=(1.0, 1.0, 1.0, 1.0)):
    a, g = _t(anchor_box).float(), _t(groundtruth_box).float()
    aw, ah = a[:, 2] - a[:, 0] + 1, a[:, 3] - a[:, 1] + 1
    gw, gh = g[:, 2] - g[:, 0] + 1, g[:, 3] - g[:, 1] + 1
    ax, ay = (a[:, 0] + a[:, 2]) * 0.5, (a[:, 1] + a[:, 3]) * 0.5
    gx, gy = (g[:, 0] + g[:, 2]) * 0.5, (g[:, 1] + g[:, 3]) * 0.5
    d = torch.stack([(gx - ax) / aw, (gy - ay) / ah, torch.log(gw / aw), torch.log(gh / ah)], 1)
    return _w((d - torch.tensor(means)) / torch.tensor(stds))


def bounding_box_decode(anchor_box, deltas, max_shape, means=(0.0, 0.0, 0.0, 0.0), stds=(1.0, 1.0, 1.0, 1.0),
                        wh_ratio_clip=0.016):
    a, d = _t(anchor_box).float(), _t(deltas).float() * torch.tensor(stds) + torch.tensor(means)
    lim = abs(math.log(wh_ratio_clip))
    dw, dh = d[:, 2].clamp(-lim, lim), d[:, 3].clamp(-lim, lim)
    aw, ah = a[:, 2] - a[:, 0] + 1, a[:, 3] - a[:, 1] + 1
    ax, ay = (a[:, 0] + a[:, 2]) * 0.5, (a[:, 1] + a[:, 3]) * 0.5
    gw, gh = aw * torch.exp(dw), ah * torch.exp(dh)
    gx, gy = ax + aw * d[:, 0], ay + ah * d[:, 1]
    x1, y1 = gx - gw * 0.5 + 0.5, gy - gh * 0.5 + 0.5
    x2, y2 = gx + gw * 0.5 - 0.5, gy + gh * 0.5 - 0.5
    h, w = max_shape
    return _w(torch.stack([x1.clamp(0, w - 1), y1.clamp(0, h - 1), x2.clamp(0, w - 1), y2.clamp(0, h - 1)], 1))


def check_valid(bboxes, img_metas):
    b, m = _t(bboxes).float(), _t(img_metas).float()
    h, w = m[0] * m[2], m[1] * m[2]
    return _w((b[:, 0] >= 0) & (b[:, 1] >= 0) & (b[:, 2] <= w - 1) & (b[:, 3] <= h - 1))


def crop_and_resize(image, boxes, box_indices, crop_size, method="bilinear", extrapolation_value=0.0):
    """image [N, H, W, C]; boxes [K, 4] as normalised (y1, x1, y2, x2); returns [K, crop_h, crop_w, C]."""
    img, bx, bi = _t(image).float(), _t(boxes).float(), _t(box_indices).long()
    n, h, w, c = img.shape
    ch, cw = crop_size
    outs = []
    for k in range(bx.shape[0]):
        y1, x1, y2, x2 = bx[k]
        ys = y1 * (h - 1) + torch.arange(ch) * ((y2 - y1) * (h - 1) / max(ch - 1, 1)) if ch > 1 else \
            torch.tensor([0.5 * (y1 + y2) * (h - 1)])
        xs = x1 * (w - 1) + torch.arange(cw) * ((x2 - x1) * (w - 1) / max(cw - 1, 1)) if cw > 1 else \
            torch.tensor([0.5 * (x1 + x2) * (w - 1)])
        gy = (2 * ys / max(h - 1, 1) - 1).reshape(ch, 1).expand(ch, cw)
        gx = (2 * xs / max(w - 1, 1) - 1).reshape(1, cw).expand(ch, cw)
        grid = torch.stack([gx, gy], -1)[None]
        src = img[bi[k]].permute(2, 0, 1)[None]
        mode = "nearest" if method == "nearest" else "bilinear"
        samp = F.grid_sample(src, grid, mode=mode, padding_mode="zeros", align_corners=True)[0].permute(1, 2, 0)
        outside = ((ys < 0) | (ys > h - 1)).reshape(ch, 1, 1) | ((xs < 0) | (xs > w - 1)).reshape(1, cw, 1)
        outs.append(torch.where(outside, torch.full_like(samp, extrapolation_value), samp))
    return _w(torch.stack(outs))


# ---------------------------------------------------------------------------------------------------- random
def _gen(seed):
    if seed is None:
        return None
    g = torch.Generator()
    g.manual_seed(_int(seed))
    return g


def multinomial_with_replacement(x, seed, offset, numsamples, replacement=False):
    return _w(torch.multinomial(_t(x).float(), _int(numsamples), replacement, generator=_gen(seed + offset)))


def random_categorical(logits, num_sample, seed=0, dtype=mstype.int64):
    p = torch.softmax(_t(logits).float(), -1)
    return _w(torch.multinomial(p, _int(num_sample), True, generator=_gen(seed) if seed else None).to(_dt(dtype)))


def random_gamma(shape, alpha, seed=None):
    a = _t(alpha).float()
    full = tuple(_int(s) for s in (shape.tolist() if isinstance(shape, torch.Tensor) else shape)) + tuple(a.shape)
    return _w(torch._standard_gamma(a.expand(full).contiguous(), generator=_gen(seed)))


def random_poisson(shape, rate, seed=None, dtype=mstype.float32):
    r = _t(rate).float()
    full = tuple(_int(s) for s in (shape.tolist() if isinstance(shape, torch.Tensor) else shape)) + tuple(r.shape)
    return _w(torch.poisson(r.expand(full).contiguous(), generator=_gen(seed)).to(_dt(dtype)))


def standard_laplace(shape, seed=None):
    u = torch.rand(tuple(shape), generator=_gen(seed)) - 0.5
    return _w(-torch.sign(u) * torch.log1p(-2 * u.abs()))


def uniform_candidate_sampler(true_classes, num_true, num_sampled, unique, range_max, seed=0, remove_accidental_hits=False):
    g = _gen(seed) if seed else None
    if unique:
        if num_sampled > range_max:
            raise ValueError("For 'uniform_candidate_sampler', num_sampled must not exceed range_max when unique")
        sampled = torch.randperm(range_max, generator=g)[:num_sampled]
    else:
        sampled = torch.randint(0, range_max, (num_sampled,), generator=g)
    p = num_sampled / range_max if not unique else 1 - (1 - 1.0 / range_max) ** num_sampled
    tc = _t(true_classes)
    return (_w(sampled.to(torch.int64)), _w(torch.full(tuple(tc.shape), p, dtype=torch.float32)),
            _w(torch.full((num_sampled,), p, dtype=torch.float32)))


def log_uniform_candidate_sampler(true_classes, num_true=1, num_sampled=5, unique=True, range_max=5, seed=0):
    g = _gen(seed) if seed else None
    logr = math.log(range_max + 1)
    prob = lambda c: (torch.log((c + 2.0) / (c + 1.0))) / logr
    out = []
    seen = set()
    while len(out) < num_sampled:
        v = _int(torch.exp(torch.rand((), generator=g) * logr)) - 1
        v = min(max(v, 0), range_max - 1)
        if unique and v in seen:
            continue
        seen.add(v)
        out.append(v)
    sampled = torch.tensor(out, dtype=torch.int64)
    tc = _t(true_classes).float()
    return _w(sampled), _w(prob(tc) * num_sampled), _w(prob(sampled.float()) * num_sampled)


def leaky_relu_ext(input, negative_slope=0.01):                                            # noqa: A002
    """``max(x, 0) + negative_slope * min(x, 0)`` (ops/extend/nn_func.py)."""
    return _w(F.leaky_relu(_t(input), float(negative_slope)))


__all__ = [n for n in dir() if not n.startswith("_") and n not in (
    "annotations", "builtins", "math", "numbers", "np", "torch", "F", "mstype")]
