"""Third tier of primitive classes: the long tail of ``mindspore.ops.operations`` (array / math / linear algebra /
neural-network / image / random / optimizer-update / quantisation / debug primitives).  Every class is built from one
table row - its constructor attributes with their defaults, and how to evaluate it - so the class API
(``ops.Cholesky(upper=True)(x)``) and the functional API (``ops.cholesky(x, upper=True)``) share one
implementation.  Attribute names and input orders follow python/mindspore/ops/operations/{array_ops,math_ops,
nn_ops,linalg_ops,image_ops,random_ops,other_ops,debug_ops,sparse_ops,inner_ops,_quant_ops}.py and
ops/auto_generate/gen_ops_prim.py.  Everything here is re-exported from ``ops.operations`` and ``ops``."""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F

from . import function_ext as X
from .primitive import Primitive

__all__ = []
_REQ = object()


def _t(x):
    return x.as_subclass(torch.Tensor) if isinstance(x, torch.Tensor) else torch.as_tensor(x)


def _u(x):
    """Unwraps what the functional layer returned (framework tensors) to plain tensors for ``_run``."""
    if isinstance(x, (tuple, list)):
        return tuple(_u(v) for v in x)
    return _t(x) if isinstance(x, torch.Tensor) else x


def _prim(name, params=(), run=None, doc=None):
    """Creates class ``name``: ``params`` is a sequence of (attribute, default) - ``_REQ`` marks a required one;
    ``run(self, *inputs)`` evaluates it."""
    params = tuple(params)
    names = [p[0] for p in params]

    def __init__(self, *args, **kwargs):
        Primitive.__init__(self, name)
        if len(args) > len(names):
            raise TypeError("%s() takes at most %d arguments (%d given)" % (name, len(names), len(args)))
        vals = dict(zip(names, args))
        for n, d in params:
            if n in vals:
                if n in kwargs:
                    raise TypeError("%s() got multiple values for argument %r" % (name, n))
                continue
            if n in kwargs:
                vals[n] = kwargs.pop(n)
            elif d is _REQ:
                raise TypeError("%s() missing required argument %r" % (name, n))
            else:
                vals[n] = d
        if kwargs:
            raise TypeError("%s() got an unexpected keyword argument %r" % (name, next(iter(kwargs))))
        for n in names:
            self._add_prim_arg(n, vals[n])

    def _run(self, *inputs):
        return _u(run(self, *inputs))

    cls = type(name, (Primitive,), {"__init__": __init__, "_run": _run,
                                    "__doc__": doc or "%s(%s)." % (name, ", ".join(names))})
    globals()[name] = cls
    __all__.append(name)
    return cls


def _fn(name, fn, params=(), n_inputs=None):
    """Primitive whose evaluation is ``fn(*inputs, **attributes)``."""
    keys = [p[0] for p in params]
    _prim(name, params, lambda self, *a: fn(*a, **{k: getattr(self, k) for k in keys}))


# ---------------------------------------------------------------------------------------------------- unary / simple
for _n, _f in {
    "BesselJ0": X.bessel_j0, "BesselJ1": X.bessel_j1, "BesselK0": X.bessel_k0, "BesselK0e": X.bessel_k0e,
    "BesselK1": X.bessel_k1, "BesselK1e": X.bessel_k1e, "BesselY0": X.bessel_y0, "BesselY1": X.bessel_y1,
    "ComplexAbs": lambda x: torch.abs(_t(x)), "ConjugateTranspose": None, "Diag": X.diag,
    "DiagPart": lambda x: torch.diagonal(_t(x).reshape(int(math.isqrt(_t(x).numel())), -1)) if _t(x).dim() != 2
    else torch.diagonal(_t(x)), "Eps": X.eps, "FastGelu": lambda x: _t(x) * torch.sigmoid(1.702 * _t(x)),
    "Geqrf": X.geqrf, "Ger": X.ger, "InvertPermutation": lambda x: torch.argsort(_t(x)),
    "LogMatrixDeterminant": X.log_matrix_determinant, "MatrixDeterminant": X.matrix_determinant,
    "MatrixExp": X.matrix_exp, "Orgqr": X.orgqr, "Trace": lambda x: torch.trace(_t(x)),
    "TupleToArray": lambda x: torch.as_tensor(x), "ScalarToArray": lambda x: torch.as_tensor(x),
    "CheckValid": X.check_valid, "MatrixBandPart": X.matrix_band_part, "Fmax": lambda a, b: torch.fmax(_t(a), _t(b)),
    "Fmin": lambda a, b: torch.fmin(_t(a), _t(b)), "Polar": lambda a, b: torch.polar(_t(a), _t(b)),
    "Complex": lambda a, b: torch.complex(_t(a), _t(b)), "Polygamma": lambda a, x: torch.polygamma(int(_t(a)), _t(x)),
    "Betainc": lambda a, b, x: torch.as_tensor(__import__("scipy.special", fromlist=["betainc"]).betainc(
        _t(a).numpy(), _t(b).numpy(), _t(x).numpy())), "AccumulateNV2": X.accumulate_n, "IdentityN": lambda x: x,
    "MaskedSelect": lambda x, m: torch.masked_select(_t(x), _t(m)),
    "MaskedScatter": lambda x, m, u: _t(x).masked_scatter(_t(m), _t(u)),
    "ListDiff": None, "UnravelIndex": lambda i, d: torch.stack(torch.unravel_index(_t(i), tuple(_t(d).tolist()))),
    "Expand": X.expand, "Fills": X.fills, "EqualCount": lambda a, b: (_t(a) == _t(b)).sum().reshape(1),
    "Coalesce": lambda i, v, s: __import__("importlib").import_module(__package__ + ".sparse_func").coalesce(i, v, s),
    "LuSolve": X.lu_solve, "HSVToRGB": None, "RGBToHSV": None,
    "CheckNumerics": None, "MatrixLogarithm": None, "TridiagonalMatMul": None,
}.items():
    if _f is not None:
        _prim(_n, (), (lambda f: lambda self, *a: f(*a))(_f))

_prim("ConjugateTranspose", (), lambda self, x, perm: _t(x).permute(tuple(perm)).conj())


def _list_diff(self, x, y):
    a, b = _t(x), _t(y)
    keep = ~torch.isin(a, b)
    return a[keep], torch.nonzero(keep).reshape(-1).to(torch.int32)


_prim("ListDiff", (("out_idx", None),), _list_diff)


def _check_numerics(self, x):
    t = _t(x)
    if not bool(torch.isfinite(t).all()):
        raise RuntimeError("For 'CheckNumerics', the input contains NaN or Inf")
    return t


_prim("CheckNumerics", (), _check_numerics)


def _hsv_to_rgb(self, x):
    t = _t(x)
    h, s, v = t[..., 0], t[..., 1], t[..., 2]
    i = torch.floor(h * 6)
    f = h * 6 - i
    p, q, w = v * (1 - s), v * (1 - f * s), v * (1 - (1 - f) * s)
    i = i.long() % 6
    r = torch.stack([v, q, p, p, w, v], -1).gather(-1, i[..., None])[..., 0]
    g = torch.stack([w, v, v, q, p, p], -1).gather(-1, i[..., None])[..., 0]
    b = torch.stack([p, p, w, v, v, q], -1).gather(-1, i[..., None])[..., 0]
    return torch.stack([r, g, b], -1)


def _rgb_to_hsv(self, x):
    t = _t(x)
    r, g, b = t[..., 0], t[..., 1], t[..., 2]
    mx, mn = t.max(-1).values, t.min(-1).values
    d = mx - mn
    safe = torch.where(d == 0, torch.ones_like(d), d)
    h = torch.where(mx == r, ((g - b) / safe) % 6, torch.where(mx == g, (b - r) / safe + 2, (r - g) / safe + 4)) / 6
    h = torch.where(d == 0, torch.zeros_like(h), h)
    s = torch.where(mx == 0, torch.zeros_like(mx), d / torch.where(mx == 0, torch.ones_like(mx), mx))
    return torch.stack([h, s, mx], -1)


_prim("HSVToRGB", (), _hsv_to_rgb)
_prim("RGBToHSV", (), _rgb_to_hsv)


def _matrix_log(self, x):
    import scipy.linalg
    t = _t(x)
    flat = t.reshape((-1,) + tuple(t.shape[-2:]))
    out = [torch.as_tensor(scipy.linalg.logm(m.numpy())) for m in flat]
    return torch.stack(out).reshape(t.shape).to(t.dtype if t.is_complex() else torch.complex64
                                                 if any(o.is_complex() for o in out) else t.dtype)


_prim("MatrixLogarithm", (), _matrix_log)


def _tridiag_matmul(self, superdiag, maindiag, subdiag, rhs):
    sup, main, sub, r = _t(superdiag), _t(maindiag), _t(subdiag), _t(rhs)
    out = main.squeeze(-2).unsqueeze(-1) * r
    out[..., :-1, :] += sup.squeeze(-2)[..., :-1].unsqueeze(-1) * r[..., 1:, :]
    out[..., 1:, :] += sub.squeeze(-2)[..., 1:].unsqueeze(-1) * r[..., :-1, :]
    return out


_prim("TridiagonalMatMul", (), _tridiag_matmul)

# ---------------------------------------------------------------------------------------------------- attribute -> kwarg
_fn("AdaptiveAvgPool2D", lambda x, output_size: F.adaptive_avg_pool2d(_t(x), output_size), [("output_size", _REQ)])
_fn("AdaptiveAvgPool3D", lambda x, output_size: F.adaptive_avg_pool3d(_t(x), output_size), [("output_size", _REQ)])
_fn("AdaptiveMaxPool2D", lambda x, output_size: F.adaptive_max_pool2d(_t(x), output_size, True),
    [("output_size", _REQ)])
_prim("AdaptiveMaxPool3D", (), lambda self, x, output_size: F.adaptive_max_pool3d(
    _t(x), tuple(_t(output_size).tolist()), True))
_fn("AffineGrid", X.affine_grid, [("align_corners", False)])
_fn("BartlettWindow", lambda n, periodic, dtype: X.bartlett_window(int(_t(n)), periodic, dtype=dtype),
    [("periodic", True), ("dtype", None)])
_fn("BlackmanWindow", lambda n, periodic, dtype: X.blackman_window(int(_t(n)), periodic, dtype=dtype),
    [("periodic", True), ("dtype", None)])
_fn("HammingWindow", lambda n, periodic, alpha, beta, dtype: X.hamming_window(int(_t(n)), periodic, alpha, beta,
                                                                              dtype=dtype),
    [("periodic", True), ("alpha", 0.54), ("beta", 0.46), ("dtype", None)])
_fn("BCEWithLogitsLoss", lambda logits, label, weight, pos_weight, reduction: F.binary_cross_entropy_with_logits(
    _t(logits), _t(label), _t(weight), pos_weight=_t(pos_weight), reduction=reduction), [("reduction", "mean")])
_fn("BatchToSpaceND", lambda x, block_shape, crops: X.batch_to_space_nd(x, block_shape, crops),
    [("block_shape", _REQ), ("crops", _REQ)])
_fn("BatchToSpace", lambda x, block_size, crops: X.batch_to_space_nd(x, block_size, crops),
    [("block_size", _REQ), ("crops", _REQ)])
_prim("BatchToSpaceNDV2", (), lambda self, x, block_shape, crops: X.batch_to_space_nd(
    x, _t(block_shape).tolist(), _t(crops).tolist()))
_fn("SpaceToBatchND", lambda x, block_shape, paddings: X.space_to_batch_nd(x, block_shape, paddings),
    [("block_shape", _REQ), ("paddings", _REQ)])
_fn("SpaceToBatch", lambda x, block_size, paddings: X.space_to_batch_nd(x, block_size, paddings),
    [("block_size", _REQ), ("paddings", _REQ)])
_fn("SpaceToDepth", lambda x, block_size: F.pixel_unshuffle(_t(x), block_size), [("block_size", _REQ)])
_fn("DepthToSpace", lambda x, block_size: F.pixel_shuffle(_t(x), block_size), [("block_size", _REQ)])
_fn("Bucketize", lambda x, boundaries: torch.bucketize(_t(x), torch.tensor(boundaries, dtype=_t(x).dtype
                                                                           if _t(x).is_floating_point() else
                                                                           torch.float32)).to(torch.int32)
    if _t(x).is_floating_point() else torch.bucketize(_t(x).float(), torch.tensor(boundaries)).to(torch.int32),
    [("boundaries", _REQ)])
_prim("Bincount", (), lambda self, array, size, weights: torch.bincount(
    _t(array).long(), _t(weights) if _t(weights).numel() else None, minlength=int(_t(size)))[:int(_t(size))])
_fn("CTCGreedyDecoder", X.ctc_greedy_decoder, [("merge_repeated", True)])
_fn("CTCLossV2", lambda lp, tg, il, tl, blank, reduction, zero_infinity: X.ctc_loss(lp, tg, il, tl, blank,
                                                                                    reduction, zero_infinity),
    [("blank", 0), ("reduction", "none"), ("zero_infinity", False)])


def _ctc_loss_sparse(self, x, labels_indices, labels_values, sequence_length):
    """Labels as a sparse [batch, max_len] tensor; blank is the last class.  Returns (loss [N], gradient)."""
    logits = _t(x).detach().clone().requires_grad_(True)
    idx, vals, lens = _t(labels_indices).long(), _t(labels_values).long(), _t(sequence_length).long()
    n = logits.shape[1]
    tl = torch.bincount(idx[:, 0], minlength=n)
    order = torch.argsort(idx[:, 0] * (idx[:, 1].max() + 1 if idx.numel() else 1) + idx[:, 1])
    loss = F.ctc_loss(torch.log_softmax(logits, -1), vals[order], lens, tl, blank=logits.shape[2] - 1,
                      reduction="none", zero_infinity=self.ignore_longer_outputs_than_inputs)
    (grad,) = torch.autograd.grad(loss.sum(), logits)
    return loss.detach(), grad


_prim("CTCLoss", [("preprocess_collapse_repeated", False), ("ctc_merge_repeated", True),
                  ("ignore_longer_outputs_than_inputs", False)], _ctc_loss_sparse)
_fn("Cdist", lambda a, b, p: torch.cdist(_t(a), _t(b), p), [("p", 2.0)])
_fn("CeLU", X.celu, [("alpha", 1.0)])
_fn("ChannelShuffle", lambda x, group: X.channel_shuffle(x, group), [("group", _REQ)])
_fn("Cholesky", X.cholesky, [("upper", False)])
_fn("CholeskyInverse", X.cholesky_inverse, [("upper", False)])
_fn("CholeskySolve", X.cholesky_solve, [("upper", False)])
_fn("Col2Im", lambda x, output_size, kernel_size, dilation, padding, stride: X.col2im(
    x, output_size, kernel_size, dilation, padding, stride),
    [("kernel_size", _REQ), ("dilation", (1, 1)), ("padding", (0, 0)), ("stride", (1, 1))])
_fn("CountNonZero", lambda x, dims: torch.count_nonzero(_t(x), tuple(dims) if dims else None), [("dims", None)])
_fn("CropAndResize", lambda image, boxes, box_index, crop_size, method, extrapolation_value: X.crop_and_resize(
    image, boxes, box_index, tuple(crop_size), method, extrapolation_value),
    [("method", "bilinear"), ("extrapolation_value", 0.0)])
_fn("Cross", lambda a, b, dim: torch.cross(_t(a), _t(b), dim=dim if dim != -65530 else
                                           next(i for i, s in enumerate(_t(a).shape) if s == 3)), [("dim", -65530)])
_fn("Cummax", lambda x, axis: (lambda r: (r.values, r.indices))(torch.cummax(_t(x), axis)), [("axis", _REQ)])
_fn("Cummin", lambda x, axis: (lambda r: (r.values, r.indices))(torch.cummin(_t(x), axis)), [("axis", _REQ)])


def _cum_lse(self, x, axis):
    t = _t(x)
    a = int(_t(axis))
    if self.reverse:
        t = t.flip(a)
    out = torch.logcumsumexp(t, a)
    if self.exclusive:
        out = torch.cat([torch.full_like(out.narrow(a, 0, 1), float("-inf")), out.narrow(a, 0, out.shape[a] - 1)], a)
    return out.flip(a) if self.reverse else out


_prim("CumulativeLogsumexp", [("exclusive", False), ("reverse", False)], _cum_lse)
_prim("Dense", (), lambda self, x, w, b=None: F.linear(_t(x), _t(w), None if b is None else _t(b)))
_fn("Dropout2D", lambda x, keep_prob: (lambda m: (_t(x) * m / keep_prob, m.bool().expand_as(_t(x))))(
    (torch.rand(_t(x).shape[:2] + (1,) * (_t(x).dim() - 2)) < keep_prob).to(_t(x).dtype)), [("keep_prob", 0.5)])
_fn("Dropout3D", lambda x, keep_prob: (lambda m: (_t(x) * m / keep_prob, m.bool().expand_as(_t(x))))(
    (torch.rand(_t(x).shape[:2] + (1,) * (_t(x).dim() - 2)) < keep_prob).to(_t(x).dtype)), [("keep_prob", 0.5)])


def _gen_mask(self, shape, keep_prob):
    g = None
    if self.Seed0 or self.Seed1:
        g = torch.Generator()
        g.manual_seed(int(self.Seed0) * 65537 + int(self.Seed1))
    n = int(math.prod(tuple(shape)))
    bits = torch.rand(n, generator=g) < float(_t(keep_prob))
    pad = (-n) % 128
    bits = torch.cat([bits, torch.zeros(pad, dtype=torch.bool)])
    weights = torch.tensor([1, 2, 4, 8, 16, 32, 64, 128], dtype=torch.uint8)
    return (bits.reshape(-1, 8).to(torch.uint8) * weights).sum(1).to(torch.uint8)


def _do_mask(self, x, mask, keep_prob):
    t = _t(x)
    m = _t(mask)
    bits = ((m[:, None] >> torch.arange(8, dtype=torch.uint8)) & 1).reshape(-1)[:t.numel()].reshape(t.shape)
    return t * bits.to(t.dtype) / float(_t(keep_prob))


_prim("DropoutGenMask", [("Seed0", 0), ("Seed1", 0)], _gen_mask)
_prim("DropoutDoMask", (), _do_mask)


def _edit_distance(self, hi, hv, hs, ti, tv, ts):
    def seqs(idx, vals, shape):
        idx, vals = _t(idx).long(), _t(vals)
        shape = tuple(int(s) for s in _t(shape).tolist())
        out = {}
        for k in range(idx.shape[0]):
            out.setdefault(tuple(idx[k, :-1].tolist()), []).append((int(idx[k, -1]), vals[k].item()))
        return {k: [v for _, v in sorted(s)] for k, s in out.items()}, shape[:-1]
    h, lead = seqs(hi, hv, hs)
    t, _ = seqs(ti, tv, ts)
    res = torch.zeros(lead)
    for key in {**h, **t}:
        a, b = h.get(key, []), t.get(key, [])
        dp = list(range(len(b) + 1))
        for i in range(1, len(a) + 1):
            prev, dp[0] = dp[0], i
            for j in range(1, len(b) + 1):
                cur = min(dp[j] + 1, dp[j - 1] + 1, prev + (a[i - 1] != b[j - 1]))
                prev, dp[j] = dp[j], cur
        d = float(dp[len(b)])
        res[key] = d / len(b) if self.normalize and len(b) else (float("inf") if self.normalize and d else d)
    return res


_prim("EditDistance", [("normalize", True)], _edit_distance)
_fn("Eig", lambda x, compute_v: torch.linalg.eig(_t(x)) if compute_v else (torch.linalg.eigvals(_t(x)),),
    [("compute_v", False)])
_fn("EuclideanNorm", lambda x, axes, keep_dims: torch.linalg.vector_norm(_t(x), 2, tuple(_t(axes).tolist())
                                                                         if isinstance(axes, torch.Tensor) else
                                                                         tuple(axes), keep_dims),
    [("keep_dims", False)])


def _extract_patches(self, x):
    t = _t(x)
    k, s, r = self.ksizes[-2:], self.strides[-2:], self.rates[-2:]
    if self.padding.lower() == "same":
        pads = []
        for size, kk, ss, rr in zip(t.shape[2:][::-1], k[::-1], s[::-1], r[::-1]):
            total = max((-(-size // ss) - 1) * ss + (kk - 1) * rr + 1 - size, 0)
            pads += [total // 2, total - total // 2]
        t = F.pad(t, pads)
    n, c = t.shape[:2]
    cols = F.unfold(t, tuple(k), tuple(r), 0, tuple(s))               # [N, C * kh * kw, L]
    ho = (t.shape[2] - (k[0] - 1) * r[0] - 1) // s[0] + 1
    cols = cols.reshape(n, c, k[0] * k[1], ho, -1).permute(0, 2, 1, 3, 4)
    return cols.reshape(n, k[0] * k[1] * c, ho, -1)


_prim("ExtractImagePatches", [("ksizes", _REQ), ("strides", _REQ), ("rates", _REQ), ("padding", "valid")],
      _extract_patches)
_fn("FillDiagonal", lambda x, fill_value, wrap: _t(x).clone().fill_diagonal_(fill_value, wrap),
    [("fill_value", _REQ), ("wrap", False)])
_fn("GLU", X.glu, [("axis", -1)])
_fn("GridSampler2D", lambda x, grid, interpolation_mode, padding_mode, align_corners: F.grid_sample(
    _t(x), _t(grid), interpolation_mode, padding_mode, align_corners),
    [("interpolation_mode", "bilinear"), ("padding_mode", "zeros"), ("align_corners", False)])
_fn("GridSampler3D", lambda x, grid, interpolation_mode, padding_mode, align_corners: F.grid_sample(
    _t(x), _t(grid), interpolation_mode, padding_mode, align_corners),
    [("interpolation_mode", "bilinear"), ("padding_mode", "zeros"), ("align_corners", False)])
_fn("HShrink", X.hardshrink, [("lambd", 0.5)])
_fn("SoftShrink", X.softshrink, [("lambd", 0.5)])
_fn("Histogram", lambda x, bins, min, max: torch.histc(_t(x).float(), bins, min, max).to(  # noqa: A002
    torch.int32 if not _t(x).is_floating_point() else _t(x).dtype), [("bins", 100), ("min", 0.0), ("max", 0.0)])
_fn("HistogramFixedWidth", lambda x, rng, nbins, dtype: torch.histc(
    _t(x).float().clamp(float(_t(rng)[0]), float(_t(rng)[1])), nbins, float(_t(rng)[0]), float(_t(rng)[1])).to(
    torch.int32), [("nbins", _REQ), ("dtype", "int32")])
_fn("IOU", X.iou, [("mode", "iou")])
_fn("Im2Col", lambda x, ksizes, strides, dilations, pads: (lambda t, k: F.unfold(
    t, k, tuple(dilations) if isinstance(dilations, (tuple, list)) else dilations, pads if isinstance(pads, int) else
    tuple(pads)[:2], tuple(strides) if isinstance(strides, (tuple, list)) else strides).reshape(
    t.shape[0], t.shape[1], k[0] * k[1], -1))(_t(x), tuple(ksizes) if isinstance(ksizes, (tuple, list)) else
                                             (ksizes, ksizes)),
    [("ksizes", _REQ), ("strides", 1), ("dilations", 1), ("pads", 0)])
_fn("InTopK", lambda x1, x2, k: X.intopk(x1, x2, k), [("k", _REQ)])
_fn("IndexAdd", lambda x, indices, y, axis, use_lock, check_index_bound: _t(x).index_add(axis, _t(indices).long(),
                                                                                         _t(y)),
    [("axis", _REQ), ("use_lock", True), ("check_index_bound", True)])
_prim("IndexFill", (), lambda self, x, dim, index, value: _t(x).index_fill(
    int(dim), _t(index).long(), value if not isinstance(value, torch.Tensor) else _t(value).item()))
_fn("IndexPut", lambda x1, x2, indices, accumulate: _t(x1).index_put(tuple(_t(i).long() for i in indices), _t(x2),
                                                                     bool(accumulate)), [("accumulate", 0)])
_fn("InplaceAdd", lambda x, v, indices: X.inplace_add(x, v, indices), [("indices", _REQ)])
_fn("InplaceSub", lambda x, v, indices: X.inplace_sub(x, v, indices), [("indices", _REQ)])


def _inplace_update(x, v, indices):
    t = _t(x).clone()
    idx = [indices] if isinstance(indices, int) else [int(i) for i in (_t(indices).tolist() if isinstance(
        indices, torch.Tensor) else indices)]
    t[idx] = _t(v).to(t.dtype)
    return t


_fn("InplaceUpdate", _inplace_update, [("indices", _REQ)])
_prim("InplaceUpdateV2", (), lambda self, x, indices, v: _inplace_update(x, v, indices))
_fn("InplaceIndexAdd", lambda var, indices, updates, axis: X.inplace_index_add(var, indices, updates, axis),
    [("axis", _REQ)])
_fn("IsClose", lambda a, b, rtol, atol, equal_nan: torch.isclose(_t(a), _t(b), rtol, atol, equal_nan),
    [("rtol", 1e-05), ("atol", 1e-08), ("equal_nan", True)])
_fn("LRN", X.lrn, [("depth_radius", 5), ("bias", 1.0), ("alpha", 1.0), ("beta", 0.5),
                   ("norm_region", "ACROSS_CHANNELS")])
_fn("LogSpace", lambda start, end, steps, base, dtype: X.logspace(start, end, steps, base,
                                                                  dtype=dtype or torch.float32),
    [("steps", 10), ("base", 10), ("dtype", None)])
_fn("LowerBound", lambda s, v, out_type: torch.searchsorted(_t(s), _t(v), right=False).to(torch.int32),
    [("out_type", "int32")])
_fn("UpperBound", lambda s, v, out_type: torch.searchsorted(_t(s), _t(v), right=True).to(torch.int32),
    [("out_type", "int32")])
_fn("SearchSorted", lambda s, v, sorter=None, dtype="int64", right=False: torch.searchsorted(
    _t(s), _t(v), right=right, sorter=None if sorter is None else _t(sorter).long()).to(
    torch.int32 if "32" in str(dtype) else torch.int64), [("dtype", "int64"), ("right", False)])
_fn("LpNorm", lambda x, axis, p, keep_dims, epsilon: torch.linalg.vector_norm(
    _t(x), p, tuple(axis) if isinstance(axis, (tuple, list)) else axis, keep_dims).clamp(min=epsilon),
    [("axis", _REQ), ("p", 2), ("keep_dims", False), ("epsilon", 1e-12)])
_fn("Lstsq", lambda x, a, fast, l2_regularizer: torch.linalg.lstsq(_t(x), _t(a)).solution,
    [("fast", True), ("l2_regularizer", 0.0)])
_fn("LuUnpack", lambda d, p, unpack_data, unpack_pivots: X.lu_unpack(d, p, unpack_data, unpack_pivots),
    [("unpack_data", True), ("unpack_pivots", True)])
_fn("MatrixDiagV3", lambda x, k, num_rows, num_cols, padding_value, align: X.matrix_diag(
    x, k, num_rows, num_cols, float(_t(padding_value)), align), [("align", "RIGHT_LEFT")])
_fn("MatrixDiagPartV3", lambda x, k, padding_value, align: X.matrix_diag_part(x, k, padding_value, align),
    [("align", "RIGHT_LEFT")])
_fn("MatrixSetDiagV3", lambda x, d, k, align: X.matrix_set_diag(x, d, k, align), [("align", "RIGHT_LEFT")])
_fn("MatrixInverse", lambda x, adjoint: torch.linalg.inv(_t(x).mH if adjoint else _t(x)), [("adjoint", False)])
_fn("MatrixPower", lambda x, n: torch.linalg.matrix_power(_t(x), n), [("n", _REQ)])
_fn("MatrixSolve", lambda m, r, adjoint: X.matrix_solve(m, r, adjoint), [("adjoint", False)])
_fn("MatrixSolveLs", lambda m, r, l2, fast: torch.linalg.solve(
    _t(m).mH @ _t(m) + float(_t(l2)) * torch.eye(_t(m).shape[-1], dtype=_t(m).dtype), _t(m).mH @ _t(r)),
    [("fast", True)])
_fn("MatrixTriangularSolve", lambda m, r, lower, adjoint: torch.linalg.solve_triangular(
    _t(m).mH if adjoint else _t(m), _t(r), upper=(not lower) != bool(adjoint)), [("lower", True), ("adjoint", False)])


def _pool_pad(t, nd, k, s, pad_mode, pad=0):
    if pad_mode.lower() == "same":
        pads = []
        for size, kk, ss in zip(t.shape[2:][::-1], k[::-1], s[::-1]):
            total = max((-(-size // ss) - 1) * ss + kk - size, 0)
            pads += [total // 2, total - total // 2]
        return F.pad(t, pads, value=float("-inf")), 0
    return t, (pad if pad_mode.lower() == "pad" else 0)


def _last(v, n):
    v = tuple(v) if isinstance(v, (tuple, list)) else (v,) * n
    return v[-n:]


def _max_pool_argmax(self, x):
    t = _t(x)
    k, s = _last(self.kernel_size, 2), _last(self.strides, 2)
    t, p = _pool_pad(t, 2, k, s, self.pad_mode)
    out, idx = F.max_pool2d(t, k, s, p, return_indices=True)
    return out, idx.to(torch.int32)


_prim("MaxPoolWithArgmax", [("kernel_size", 1), ("strides", 1), ("pad_mode", "valid"), ("data_format", "NCHW")],
      _max_pool_argmax)
_fn("MaxPoolWithArgmaxV2", lambda x, kernel_size, strides, pads, dilation, ceil_mode, argmax_type: (
    lambda r: (r[0], r[1].to(torch.int64)))(F.max_pool2d(_t(x), _last(kernel_size, 2), _last(strides or kernel_size,
                                                                                             2), _last(pads, 2),
                                                         _last(dilation, 2), ceil_mode, True)),
    [("kernel_size", _REQ), ("strides", None), ("pads", 0), ("dilation", (1, 1)), ("ceil_mode", False),
     ("argmax_type", "int64")])
_fn("MaxPool3DWithArgmax", lambda x, ksize, strides, pads, dilation, ceil_mode, data_format, argmax_type: (
    lambda r: (r[0], r[1].to(torch.int64)))(F.max_pool3d(_t(x), _last(ksize, 3), _last(strides, 3), _last(pads, 3),
                                                         _last(dilation, 3), ceil_mode, True)),
    [("ksize", _REQ), ("strides", _REQ), ("pads", 0), ("dilation", (1, 1, 1)), ("ceil_mode", False),
     ("data_format", "NCDHW"), ("argmax_type", "int64")])


def _pool3d(fn):
    def run(self, x):
        t = _t(x)
        k, s = _last(self.kernel_size, 3), _last(self.strides, 3)
        if self.pad_mode.lower() == "same":
            pads = []
            for size, kk, ss in zip(t.shape[2:][::-1], k[::-1], s[::-1]):
                total = max((-(-size // ss) - 1) * ss + kk - size, 0)
                pads += [total // 2, total - total // 2]
            t = F.pad(t, pads, value=float("-inf") if fn is F.max_pool3d else 0.0)
            p = 0
        else:
            pl = self.pad_list if isinstance(self.pad_list, (tuple, list)) else (self.pad_list,) * 6
            p = tuple(pl[::2]) if len(pl) == 6 else _last(pl, 3)
            p = p if self.pad_mode.lower() == "pad" else 0
        if fn is F.max_pool3d:
            return fn(t, k, s, p, 1, bool(self.ceil_mode))
        return fn(t, k, s, p, bool(self.ceil_mode), self.count_include_pad, self.divisor_override or None)
    return run


_prim("MaxPool3D", [("kernel_size", 1), ("strides", 1), ("pad_mode", "VALID"), ("pad_list", 0), ("ceil_mode", None),
                    ("data_format", "NCDHW")], _pool3d(F.max_pool3d))
_prim("AvgPool3D", [("kernel_size", 1), ("strides", 1), ("pad_mode", "valid"), ("pad_list", 0), ("ceil_mode", False),
                    ("count_include_pad", True), ("divisor_override", 0), ("data_format", "NCDHW")],
      _pool3d(F.avg_pool3d))
_prim("MaxUnpool2D", [("ksize", _REQ), ("strides", 0), ("pads", 0), ("output_shape", ()), ("data_format", "NCHW")],
      lambda self, x, argmax: F.max_unpool2d(_t(x), _t(argmax).long(), _last(self.ksize, 2),
                                             _last(self.strides or self.ksize, 2), _last(self.pads, 2),
                                             tuple(self.output_shape)[-2:] if self.output_shape else None))
_prim("MaxUnpool3D", [("ksize", _REQ), ("strides", 0), ("pads", 0), ("output_shape", ()), ("data_format", "NCDHW")],
      lambda self, x, argmax: F.max_unpool3d(_t(x), _t(argmax).long(), _last(self.ksize, 3),
                                             _last(self.strides or self.ksize, 3), _last(self.pads, 3),
                                             tuple(self.output_shape)[-3:] if self.output_shape else None))
_fn("Meshgrid", lambda xs, indexing: torch.meshgrid(*[_t(v) for v in xs], indexing=indexing), [("indexing", "xy")])
_fn("MirrorPad", lambda x, paddings, mode: X.mirror_pad(x, paddings, mode), [("mode", "REFLECT")])
_fn("MultiMarginLoss", lambda x, target, weight=None, p=1, margin=1.0, reduction="mean": X.multi_margin_loss(
    x, target, p, margin, weight, reduction), [("p", 1), ("margin", 1.0), ("reduction", "mean")])
_fn("MultilabelMarginLoss", lambda x, target, reduction: (X.multilabel_margin_loss(x, target, reduction),
                                                          torch.zeros_like(_t(target), dtype=torch.int32)),
    [("reduction", "mean")])
_fn("SoftMarginLoss", X.soft_margin_loss, [("reduction", "mean")])
_fn("TripletMarginLoss", lambda a, pz, n, margin, p, swap, eps, reduction: X.triplet_margin_loss(
    a, pz, n, float(_t(margin)), p, eps, swap, reduction), [("p", 2), ("swap", False), ("eps", 1e-06),
                                                            ("reduction", "mean")])
_fn("Mvlgamma", lambda x, p: torch.mvlgamma(_t(x), p), [("p", _REQ)])
_fn("NanToNum", lambda x, nan, posinf, neginf: torch.nan_to_num(_t(x), nan, posinf, neginf),
    [("nan", None), ("posinf", None), ("neginf", None)])
_fn("NthElement", lambda x, n, reverse: torch.sort(_t(x), -1, descending=reverse).values[..., int(_t(n))],
    [("reverse", False)])
_fn("NuclearNorm", lambda x, dim, keepdim: torch.linalg.matrix_norm(_t(x), "nuc", tuple(dim) if dim is not None else
                                                                    (-2, -1), keepdim),
    [("dim", None), ("keepdim", False)])
_fn("Ormqr", lambda x, tau, other, left, transpose: X.ormqr(x, tau, other, left, transpose),
    [("left", True), ("transpose", False)])
_fn("Padding", X.padding, [("pad_dim_size", 8)])
_prim("ParallelConcat", (), lambda self, values: torch.cat([_t(v) for v in values], 0))
_fn("Pdist", X.pdist, [("p", 2.0)])
_fn("Qr", lambda x, full_matrices: torch.linalg.qr(_t(x), "complete" if full_matrices else "reduced"),
    [("full_matrices", False)])
_fn("Quantile", lambda x, q, dim, keep_dims, ignore_nan: (torch.nanquantile if ignore_nan else torch.quantile)(
    _t(x), _t(q).to(_t(x).dtype), dim, keep_dims), [("dim", None), ("keep_dims", False), ("ignore_nan", False)])
_fn("ReduceStd", lambda x, axis, unbiased, keep_dims: (lambda t, d: (
    torch.std(t, d, unbiased=unbiased, keepdim=keep_dims), torch.mean(t, d, keepdim=keep_dims)))(
    _t(x), (tuple(axis) if isinstance(axis, (tuple, list)) else axis) if axis not in ((), None) else
    tuple(range(_t(x).dim()))), [("axis", ()), ("unbiased", True), ("keep_dims", False)])
_fn("Renorm", lambda x, p, dim, maxnorm: torch.renorm(_t(x), p, dim, maxnorm),
    [("p", _REQ), ("dim", _REQ), ("maxnorm", _REQ)])
_fn("ReverseSequence", lambda x, seq_lengths, seq_dim, batch_dim: X.reverse_sequence(x, seq_lengths, seq_dim,
                                                                                     batch_dim),
    [("seq_dim", _REQ), ("batch_dim", 0)])
_fn("Roll", lambda x, shift, axis: torch.roll(_t(x), shift, axis), [("shift", _REQ), ("axis", _REQ)])
_fn("STFT", lambda x, window, n_fft, hop_length, win_length, normalized, onesided, return_complex: X.stft(
    x, n_fft, hop_length, win_length, window, False, "REFLECT", normalized, onesided, return_complex),
    [("n_fft", _REQ), ("hop_length", None), ("win_length", None), ("normalized", False), ("onesided", True),
     ("return_complex", True)])
_prim("ScalarCast", (), lambda self, x, dtype: X._dt(dtype) and torch.as_tensor(x).to(X._dt(dtype)).item())
_prim("ScalarToTensor", (), lambda self, x, dtype=None: torch.as_tensor(x, dtype=X._dt(dtype)))
_fn("Svd", lambda x, full_matrices, compute_uv: X.svd(x, full_matrices, compute_uv) if compute_uv else
    (X.svd(x, full_matrices, False),), [("full_matrices", False), ("compute_uv", True)])
_fn("TrilIndices", lambda row, col, offset, dtype: torch.tril_indices(row, col, offset).to(X._dt(dtype)
                                                                                           or torch.int32),
    [("row", _REQ), ("col", _REQ), ("offset", 0), ("dtype", None)])
_fn("TriuIndices", lambda row, col, offset, dtype: torch.triu_indices(row, col, offset).to(X._dt(dtype)
                                                                                           or torch.int32),
    [("row", _REQ), ("col", _REQ), ("offset", 0), ("dtype", None)])
_fn("UniqueConsecutive", lambda x, return_idx, return_counts, axis: (lambda r: r if isinstance(r, tuple) else (r,))(
    torch.unique_consecutive(_t(x), return_inverse=return_idx, return_counts=return_counts, dim=axis)),
    [("return_idx", False), ("return_counts", False), ("axis", None)])
_prim("UniqueWithPad", (), lambda self, x, pad_num: X.unique_with_pad(x, pad_num))
_fn("Unpack", lambda x, axis: torch.unbind(_t(x), axis), [("axis", 0)])
_fn("UpsampleNearest3D", lambda x, output_size=None, scales=None: F.interpolate(
    _t(x), size=tuple(output_size) if output_size else None, scale_factor=tuple(scales) if scales else None,
    mode="nearest"))
_fn("UpsampleTrilinear3D", lambda x, output_size=None, scales=None, align_corners=False: F.interpolate(
    _t(x), size=tuple(output_size) if output_size else None, scale_factor=tuple(scales) if scales else None,
    mode="trilinear", align_corners=align_corners), [("align_corners", False)])
_fn("ResizeBicubic", lambda x, size, align_corners, half_pixel_centers: F.interpolate(
    _t(x), size=tuple(int(s) for s in (_t(size).tolist() if isinstance(size, torch.Tensor) else size)),
    mode="bicubic", align_corners=align_corners), [("align_corners", False), ("half_pixel_centers", False)])
_fn("ResizeArea", lambda x, size, align_corners: F.interpolate(
    _t(x).permute(0, 3, 1, 2), size=tuple(int(s) for s in (_t(size).tolist() if isinstance(size, torch.Tensor)
                                                          else size)), mode="area").permute(0, 2, 3, 1),
    [("align_corners", False)])
_fn("ResizeLinear1D", lambda x, size, coordinate_transformation_mode: F.interpolate(
    _t(x), size=tuple(int(s) for s in (_t(size).tolist() if isinstance(size, torch.Tensor) else size)),
    mode="linear", align_corners=coordinate_transformation_mode == "align_corners"),
    [("coordinate_transformation_mode", "align_corners")])
_fn("ResizeNearestNeighborV2", lambda x, size, align_corners, half_pixel_centers: F.interpolate(
    _t(x), size=tuple(int(s) for s in (_t(size).tolist() if isinstance(size, torch.Tensor) else size)),
    mode="nearest"), [("align_corners", False), ("half_pixel_centers", False)])


def _conv3d(self, x, w):
    s, d = _last(self.stride, 3), _last(self.dilation, 3)
    pad = self.pad if isinstance(self.pad, (tuple, list)) else (self.pad,) * 6
    return X.conv3d(x, w, None, s, self.pad_mode.lower(), tuple(pad) if self.pad_mode.lower() == "pad" else 0, d,
                    self.group)


_prim("Conv3D", [("out_channel", _REQ), ("kernel_size", _REQ), ("mode", 1), ("pad_mode", "valid"), ("pad", 0),
                 ("stride", 1), ("dilation", 1), ("group", 1), ("data_format", "NCDHW")], _conv3d)
_prim("Conv3DTranspose", [("in_channel", _REQ), ("out_channel", _REQ), ("kernel_size", _REQ), ("mode", 1),
                          ("pad_mode", "valid"), ("pad", 0), ("stride", 1), ("dilation", 1), ("group", 1),
                          ("output_padding", 0), ("data_format", "NCDHW")],
      lambda self, x, w: X.conv3d_transpose(x, w, self.pad_mode.lower(), _last(self.pad, 3) if not isinstance(
          self.pad, int) else self.pad, _last(self.stride, 3), _last(self.dilation, 3), self.group,
          self.output_padding))


def _conv2d_bprop_input(self, dout, w, input_size):
    s, d = _last(self.stride, 2), _last(self.dilation, 2)
    size = tuple(int(v) for v in (_t(input_size).tolist() if isinstance(input_size, torch.Tensor) else input_size))
    k = _t(w).shape[2:]
    if self.pad_mode.lower() == "same":
        pads = [max((-(-size[2 + i] // s[i]) - 1) * s[i] + (k[i] - 1) * d[i] + 1 - size[2 + i], 0) for i in range(2)]
        lo = [p // 2 for p in pads]
        full = torch.nn.grad.conv2d_input((size[0], size[1], size[2] + pads[0], size[3] + pads[1]), _t(w), _t(dout),
                                          s, 0, d, self.group)
        return full[:, :, lo[0]:lo[0] + size[2], lo[1]:lo[1] + size[3]]
    p = 0 if self.pad_mode.lower() == "valid" else (_last(self.pad, 2) if not isinstance(self.pad, int) else self.pad)
    return torch.nn.grad.conv2d_input(size, _t(w), _t(dout), s, p, d, self.group)


_prim("Conv2DBackpropInput", [("out_channel", _REQ), ("kernel_size", _REQ), ("pad_mode", "valid"), ("pad", 0),
                              ("pad_list", None), ("mode", 1), ("stride", 1), ("dilation", 1), ("group", 1),
                              ("data_format", "NCHW")], _conv2d_bprop_input)
def _depthwise_conv(self, x, w):
    """``w`` is [channel_multiplier, C, kh, kw]; every input channel gets its own ``channel_multiplier`` filters."""
    t, k = _t(x), _t(w)
    c = t.shape[1]
    k = k.permute(1, 0, 2, 3).reshape(c * k.shape[0], 1, *k.shape[2:])
    s, d = _last(self.stride, 2), _last(self.dilation, 2)
    t, p = X._conv_pad(t, 2, k.shape[2:], s, d, self.pad_mode.lower(), self.pad)
    return F.conv2d(t, k, None, s, p, d, c)


_prim("DepthwiseConv2dNative", [("channel_multiplier", _REQ), ("kernel_size", _REQ), ("mode", 3),
                                ("pad_mode", "valid"), ("pad", 0), ("stride", 1), ("dilation", 1), ("group", 1)],
      _depthwise_conv)


def _roi_align(self, features, rois):
    """features [N, C, H, W]; rois [K, 5] = (batch index, x1, y1, x2, y2); average of ``sample_num`` x ``sample_num``
    bilinear samples per output bin."""
    f, r = _t(features), _t(rois).float()
    ph, pw, scale = self.pooled_height, self.pooled_width, self.spatial_scale
    sn = max(int(self.sample_num), 1)
    end = 1.0 if self.roi_end_mode else 0.0
    n, c, h, w = f.shape
    outs = []
    for k in range(r.shape[0]):
        b = int(r[k, 0])
        x1, y1 = r[k, 1] * scale, r[k, 2] * scale
        x2, y2 = (r[k, 3] + end) * scale, (r[k, 4] + end) * scale
        rw, rh = torch.clamp(x2 - x1, min=1.0), torch.clamp(y2 - y1, min=1.0)
        ys = y1 + (torch.arange(ph * sn) + 0.5) * rh / (ph * sn)
        xs = x1 + (torch.arange(pw * sn) + 0.5) * rw / (pw * sn)
        gy = (2 * ys / max(h - 1, 1) - 1).reshape(-1, 1).expand(ph * sn, pw * sn)
        gx = (2 * xs / max(w - 1, 1) - 1).reshape(1, -1).expand(ph * sn, pw * sn)
        samp = F.grid_sample(f[b:b + 1].float(), torch.stack([gx, gy], -1)[None], mode="bilinear",
                             padding_mode="border", align_corners=True)
        outs.append(F.avg_pool2d(samp, sn)[0])
    return torch.stack(outs).to(f.dtype) if outs else f.new_zeros((0, c, ph, pw))


_prim("ROIAlign", [("pooled_height", _REQ), ("pooled_width", _REQ), ("spatial_scale", _REQ), ("sample_num", 2),
                   ("roi_end_mode", 1)], _roi_align)


def _nms(boxes, scores, thr):
    order = torch.argsort(scores, descending=True)
    keep = []
    area = (boxes[:, 2] - boxes[:, 0]) * (boxes[:, 3] - boxes[:, 1])
    alive = torch.ones(boxes.shape[0], dtype=torch.bool)
    for i in order.tolist():
        if not alive[i]:
            continue
        keep.append(i)
        lt = torch.maximum(boxes[i, :2], boxes[:, :2])
        rb = torch.minimum(boxes[i, 2:4], boxes[:, 2:4])
        wh = (rb - lt).clamp(min=0)
        inter = wh[:, 0] * wh[:, 1]
        iou = inter / (area[i] + area - inter).clamp(min=1e-12)
        alive &= ~(iou > thr)
        alive[i] = False
    return keep


def _nms_with_mask(self, bboxes):
    b = _t(bboxes).float()
    order = torch.argsort(b[:, 4], descending=True)
    sorted_b = b[order]
    keep = _nms(sorted_b[:, :4], sorted_b[:, 4], self.iou_threshold)
    mask = torch.zeros(b.shape[0], dtype=torch.bool)
    mask[keep] = True
    return sorted_b.to(_t(bboxes).dtype), order.to(torch.int32), mask


_prim("NMSWithMask", [("iou_threshold", 0.5)], _nms_with_mask)


def _nms_v3(self, boxes, scores, max_output_size, iou_threshold, score_threshold):
    b, s = _t(boxes).float(), _t(scores).float()
    ok = torch.nonzero(s > float(_t(score_threshold))).reshape(-1)
    keep = [int(ok[i]) for i in _nms(b[ok], s[ok], float(_t(iou_threshold)))][:int(_t(max_output_size))]
    return torch.tensor(keep, dtype=torch.int32)


_prim("NonMaxSuppressionV3", (), _nms_v3)

# ---------------------------------------------------------------------------------------------------- scatter / segment
for _r in ("Add", "Sub", "Mul", "Div", "Max", "Min"):
    _low = _r.lower()
    if hasattr(X, "scatter_nd_" + _low):
        _prim("ScatterNd" + _r, [("use_locking", False)],
              (lambda f: lambda self, x, i, u: f(x, i, u))(getattr(X, "scatter_nd_" + _low)))
    if _r != "Add" and hasattr(X, "tensor_scatter_" + _low):
        _prim("TensorScatter" + _r, (), (lambda f: lambda self, x, i, u: f(x, i, u))(
            getattr(X, "tensor_scatter_" + _low)))
for _r in ("Update", "Mul", "Div", "Max", "Min"):
    _prim("Scatter" + _r, [("use_locking", False if _r != "Update" else True)],
          (lambda f: lambda self, x, i, u: f(x, i, u))(getattr(X, "scatter_" + _r.lower())))


def _scatter_rows(sign):
    def run(self, x, indices, updates):
        t = _t(x)
        ind = _t(indices).long().reshape(-1)
        upd = _t(updates).to(t.dtype).reshape((ind.numel(),) + tuple(t.shape[1:]))
        with torch.no_grad():
            t.index_add_(0, ind, sign * upd)
        return t
    return run


_prim("ScatterAdd", [("use_locking", False)], _scatter_rows(1))
_prim("ScatterSub", [("use_locking", False)], _scatter_rows(-1))


def _scatter_nd_update(self, x, indices, updates):
    t = _t(x)
    with torch.no_grad():
        t.index_put_(X._nd_index(indices), _t(updates).to(t.dtype))
    return t


_prim("ScatterNdUpdate", [("use_locking", True)], _scatter_nd_update)
_prim("ScatterNonAliasingAdd", (), lambda self, x, i, u: _t(x).index_put(X._nd_index(i), _t(u).to(_t(x).dtype),
                                                                        accumulate=True))
_fn("ScatterAddWithAxis", lambda x, i, u, axis: _t(x).scatter_add(axis, _t(i).long(), _t(u)), [("axis", 0)])
_fn("TensorScatterElements", lambda x, i, u, axis, reduction: X.tensor_scatter_elements(x, i, u, axis, reduction),
    [("axis", 0), ("reduction", "none")])


def _sorted_segment(reduce):
    def run(self, x, segment_ids):
        t, ids = _t(x), _t(segment_ids).long()
        n = int(ids.max()) + 1 if ids.numel() else 0
        idx = ids.reshape((-1,) + (1,) * (t.dim() - 1)).expand_as(t)
        if reduce == "mean":
            out = torch.zeros((n,) + tuple(t.shape[1:]), dtype=t.dtype).scatter_add(0, idx, t)
            cnt = torch.bincount(ids, minlength=n).clamp(min=1).reshape((-1,) + (1,) * (t.dim() - 1))
            return out / cnt.to(t.dtype)
        init = {"sum": 0, "prod": 1, "amax": X._min_of(t.dtype), "amin": X._max_of(t.dtype)}[reduce]
        out = torch.full((n,) + tuple(t.shape[1:]), init, dtype=t.dtype).scatter_reduce(0, idx, t, reduce)
        if reduce in ("amax", "amin"):
            empty = torch.bincount(ids, minlength=n) == 0
            out[empty] = 0
        return out
    return run


for _n, _r in (("SegmentSum", "sum"), ("SegmentProd", "prod"), ("SegmentMax", "amax"), ("SegmentMin", "amin"),
               ("SegmentMean", "mean")):
    _prim(_n, (), _sorted_segment(_r))
for _n in ("Max", "Min", "Prod"):
    _prim("UnsortedSegment" + _n, (), (lambda f: lambda self, x, ids, n: f(x, ids, n))(
        getattr(X, "unsorted_segment_" + _n.lower())))

# ---------------------------------------------------------------------------------------------------- sparse <-> dense
_prim("SparseToDense", (), lambda self, indices, values, dense_shape: torch.zeros(
    tuple(int(s) for s in (_t(dense_shape).tolist() if isinstance(dense_shape, torch.Tensor) else dense_shape)),
    dtype=_t(values).dtype).index_put(X._nd_index(indices), _t(values)))
_prim("SparseTensorDenseAdd", (), lambda self, i, v, s, d: _t(d).index_put(X._nd_index(i), _t(v).to(_t(d).dtype),
                                                                          accumulate=True))


def _sparse_dense_matmul(self, indices, values, sparse_shape, dense):
    shape = tuple(int(s) for s in (_t(sparse_shape).tolist() if isinstance(sparse_shape, torch.Tensor)
                                   else sparse_shape))
    sp = torch.zeros(shape, dtype=_t(values).dtype).index_put(X._nd_index(indices), _t(values), accumulate=True)
    d = _t(dense)
    return (sp.mH if self.adjoint_st else sp) @ (d.mH if self.adjoint_dt else d)


_prim("SparseTensorDenseMatmul", [("adjoint_st", False), ("adjoint_dt", False)], _sparse_dense_matmul)

# ---------------------------------------------------------------------------------------------------- random


def _seeded(self):
    s0, s1 = int(getattr(self, "seed", 0) or 0), int(getattr(self, "seed2", getattr(self, "offset", 0)) or 0)
    if not s0 and not s1:
        return None
    g = torch.Generator()
    g.manual_seed(s0 * 65537 + s1)
    return g


_prim("Bernoulli", [("seed", -1), ("offset", 0)], lambda self, x, p=0.5: torch.bernoulli(
    torch.full_like(_t(x), float(p), dtype=torch.float32) if not isinstance(p, torch.Tensor) else
    _t(p).float().expand_as(_t(x)), generator=_seeded(self) if self.seed not in (-1, 0) else None).to(_t(x).dtype))
_prim("Cauchy", [("size", _REQ), ("median", 0.0), ("sigma", 1.0)], lambda self: torch.empty(
    tuple(self.size)).cauchy_(self.median, self.sigma))
_prim("Gamma", [("seed", 0), ("seed2", 0)], lambda self, shape, alpha, beta: torch._standard_gamma(
    _t(alpha).float().expand(tuple(shape) if tuple(shape)[-_t(alpha).dim():] == tuple(_t(alpha).shape) else
                             tuple(shape) + tuple(_t(alpha).shape)).contiguous(), generator=_seeded(self))
      / _t(beta).float())
_prim("Poisson", [("seed", 0), ("seed2", 0)], lambda self, shape, mean: torch.poisson(
    _t(mean).float().expand(tuple(shape)).contiguous(), generator=_seeded(self)).to(torch.int32))
_prim("RandomGamma", [("seed", 0), ("seed2", 0)], lambda self, shape, alpha: X.random_gamma(
    shape, alpha, (self.seed * 65537 + self.seed2) or None))
_prim("RandomPoisson", [("seed", 0), ("seed2", 0), ("dtype", None)], lambda self, shape, rate: X.random_poisson(
    shape, rate, (self.seed * 65537 + self.seed2) or None, self.dtype or torch.int64))
_prim("RandomCategorical", [("dtype", None)], lambda self, logits, num_sample, seed: X.random_categorical(
    logits, int(num_sample), int(seed), self.dtype or torch.int64))
_prim("RandomShuffle", [("seed", 0), ("seed2", 0)], lambda self, x: _t(x)[torch.randperm(
    _t(x).shape[0], generator=_seeded(self))])


def _choice_with_mask(self, x):
    t = _t(x)
    idx = torch.nonzero(t)
    n = min(int(self.count), idx.shape[0])
    pick = torch.randperm(idx.shape[0], generator=_seeded(self))[:n]
    out = torch.zeros((int(self.count), t.dim()), dtype=torch.int32)
    out[:n] = idx[pick].to(torch.int32)
    mask = torch.zeros(int(self.count), dtype=torch.bool)
    mask[:n] = True
    return out, mask


_prim("RandomChoiceWithMask", [("count", 256), ("seed", 0), ("seed2", 0)], _choice_with_mask)
_prim("Randperm", [("max_length", 1), ("pad", -1), ("dtype", None)], lambda self, n: torch.cat([
    torch.randperm(int(_t(n))), torch.full((self.max_length - int(_t(n)),), self.pad, dtype=torch.int64)]).to(
    X._dt(self.dtype) or torch.int32))
_prim("RandpermV2", [("dtype", None)], lambda self, n, seed=-1, offset=0: torch.randperm(
    int(n if not isinstance(n, torch.Tensor) else _t(n)), generator=X._gen(int(seed) + int(offset))
    if int(seed) >= 0 else None).to(X._dt(self.dtype) or torch.int64))
_prim("StandardLaplace", [("seed", 0), ("seed2", 0)], lambda self, shape: X.standard_laplace(
    tuple(shape), (self.seed * 65537 + self.seed2) or None))
_prim("TruncatedNormal", [("seed", 0), ("seed2", 0), ("dtype", None)], lambda self, shape: torch.nn.init.trunc_normal_(
    torch.empty(tuple(int(s) for s in (_t(shape).tolist() if isinstance(shape, torch.Tensor) else shape)),
                dtype=X._dt(self.dtype) or torch.float32), 0.0, 1.0, -2.0, 2.0, generator=_seeded(self)))
_prim("ParameterizedTruncatedNormal", [("seed", 0), ("seed2", 0)],
      lambda self, shape, mean, stdevs, mn, mx: torch.stack([torch.nn.init.trunc_normal_(
          torch.empty(tuple(int(s) for s in _t(shape).tolist()[1:])), float(_t(mean).reshape(-1)[i % _t(mean).numel()]),
          float(_t(stdevs).reshape(-1)[i % _t(stdevs).numel()]), float(_t(mn).reshape(-1)[i % _t(mn).numel()]),
          float(_t(mx).reshape(-1)[i % _t(mx).numel()]), generator=_seeded(self))
          for i in range(int(_t(shape)[0]))]))
_prim("NonDeterministicInts", [("dtype", None)], lambda self, shape: torch.randint(
    torch.iinfo(X._dt(self.dtype) or torch.int64).min, torch.iinfo(X._dt(self.dtype) or torch.int64).max,
    tuple(int(s) for s in _t(shape).tolist()), dtype=X._dt(self.dtype) or torch.int64))
_prim("LogNormalReverse", [("mean", 1.0), ("std", 2.0)], lambda self, x: torch.empty_like(_t(x)).log_normal_(
    self.mean, self.std))
_prim("MultinomialWithReplacement", [("numsamples", _REQ), ("replacement", False)],
      lambda self, x, seed, offset: X.multinomial_with_replacement(x, int(_t(seed)), int(_t(offset)),
                                                                   self.numsamples, self.replacement))
_prim("UniformCandidateSampler", [("num_true", _REQ), ("num_sampled", _REQ), ("unique", _REQ), ("range_max", _REQ),
                                  ("seed", 0), ("remove_accidental_hits", False)],
      lambda self, true_classes: X.uniform_candidate_sampler(true_classes, self.num_true, self.num_sampled,
                                                             self.unique, self.range_max, self.seed,
                                                             self.remove_accidental_hits))
_prim("LogUniformCandidateSampler", [("num_true", 1), ("num_sampled", 5), ("unique", True), ("range_max", 5),
                                     ("seed", 0)],
      lambda self, true_classes: X.log_uniform_candidate_sampler(true_classes, self.num_true, self.num_sampled,
                                                                 self.unique, self.range_max, self.seed))


def _accidental_hits(self, true_classes, sampled):
    tc, sc = _t(true_classes), _t(sampled)
    rows, ids = [], []
    for r in range(tc.shape[0]):
        for j in range(sc.shape[0]):
            if bool((tc[r] == sc[j]).any()):
                rows.append(r)
                ids.append(j)
    n = len(rows)
    return (torch.tensor(rows, dtype=torch.int32), torch.tensor(ids, dtype=torch.int32),
            torch.full((n,), -torch.finfo(torch.float32).max))


_prim("ComputeAccidentalHits", [("num_true", 1)], _accidental_hits)

# ---------------------------------------------------------------------------------------------------- optimizer updates


def _upd(t, value):
    with torch.no_grad():
        _t(t).copy_(value)
    return _t(t)


def _s(v, like):
    return _t(v).to(like.dtype) if isinstance(v, torch.Tensor) else torch.as_tensor(v, dtype=like.dtype)


def _apply_adamax(self, var, m, v, beta1_power, lr, beta1, beta2, eps, grad):
    vv, g = _t(var), _t(grad)
    b1, b2 = _s(beta1, vv), _s(beta2, vv)
    m2 = b1 * _t(m) + (1 - b1) * g
    v2 = torch.maximum(b2 * _t(v), g.abs())
    return _upd(var, vv - _s(lr, vv) / (1 - _s(beta1_power, vv)) * m2 / (v2 + _s(eps, vv))), _upd(m, m2), _upd(v, v2)


def _apply_adadelta(self, var, accum, accum_update, lr, rho, eps, grad):
    vv, g = _t(var), _t(grad)
    r, e = _s(rho, vv), _s(eps, vv)
    a2 = r * _t(accum) + (1 - r) * g * g
    upd = torch.sqrt(_t(accum_update) + e) / torch.sqrt(a2 + e) * g
    au2 = r * _t(accum_update) + (1 - r) * upd * upd
    return _upd(var, vv - _s(lr, vv) * upd), _upd(accum, a2), _upd(accum_update, au2)


def _apply_adagrad(self, var, accum, lr, grad):
    vv, g = _t(var), _t(grad)
    a2 = _t(accum) + g * g if getattr(self, "update_slots", True) else _t(accum)
    eps = getattr(self, "epsilon", None)
    den = torch.sqrt(a2) + eps if eps is not None else torch.sqrt(a2)
    return _upd(var, vv - _s(lr, vv) * g / den), _upd(accum, a2)


def _apply_adagrad_da(self, var, gacc, gsq, grad, lr, l1, l2, global_step):
    vv, g = _t(var), _t(grad)
    ga, gs = _t(gacc) + g, _t(gsq) + g * g
    step = _s(global_step, vv)
    l1v, l2v, lrv = _s(l1, vv), _s(l2, vv), _s(lr, vv)
    tmp = torch.sign(ga) * torch.clamp(ga.abs() - l1v * step, min=0) if float(l1v) > 0 else ga
    return _upd(var, -lrv * tmp / (l2v * step * lrv + torch.sqrt(gs))), _upd(gacc, ga), _upd(gsq, gs)


def _apply_amsgrad(self, var, m, v, vhat, beta1_power, beta2_power, lr, *rest):
    if len(rest) == 1:
        b1, b2, eps, grad = self.beta1, self.beta2, self.epsilon, rest[0]
    else:
        b1, b2, eps, grad = rest
    vv, g = _t(var), _t(grad)
    b1, b2 = _s(b1, vv), _s(b2, vv)
    lr_t = _s(lr, vv) * torch.sqrt(1 - _s(beta2_power, vv)) / (1 - _s(beta1_power, vv))
    m2 = b1 * _t(m) + (1 - b1) * g
    v2 = b2 * _t(v) + (1 - b2) * g * g
    vh = torch.maximum(_t(vhat), v2)
    return _upd(var, vv - lr_t * m2 / (torch.sqrt(vh) + _s(eps, vv))), _upd(m, m2), _upd(v, v2), _upd(vhat, vh)


def _apply_add_sign(self, var, m, lr, alpha, sign_decay, beta, grad):
    vv, g = _t(var), _t(grad)
    b = _s(beta, vv)
    m2 = b * _t(m) + (1 - b) * g
    return _upd(var, vv - _s(lr, vv) * (_s(alpha, vv) + _s(sign_decay, vv) * torch.sign(g) * torch.sign(m2)) * g), \
        _upd(m, m2)


def _apply_power_sign(self, var, m, lr, logbase, sign_decay, beta, grad):
    vv, g = _t(var), _t(grad)
    b = _s(beta, vv)
    m2 = b * _t(m) + (1 - b) * g
    return _upd(var, vv - _s(lr, vv) * torch.exp(_s(logbase, vv) * _s(sign_decay, vv) * torch.sign(g)
                                                 * torch.sign(m2)) * g), _upd(m, m2)


def _apply_centered_rmsprop(self, var, mg, ms, mom, grad, lr, rho, momentum, eps):
    vv, g = _t(var), _t(grad)
    r = _s(rho, vv)
    mg2 = r * _t(mg) + (1 - r) * g
    ms2 = r * _t(ms) + (1 - r) * g * g
    mom2 = _s(momentum, vv) * _t(mom) + _s(lr, vv) * g / torch.sqrt(ms2 - mg2 * mg2 + _s(eps, vv))
    _upd(mg, mg2), _upd(ms, ms2), _upd(mom, mom2)
    return _upd(var, vv - mom2)


def _apply_rmsprop(self, var, ms, mom, lr, grad, rho, momentum, eps):
    vv, g = _t(var), _t(grad)
    r = _s(rho, vv)
    ms2 = r * _t(ms) + (1 - r) * g * g
    mom2 = _s(momentum, vv) * _t(mom) + _s(lr, vv) * g / torch.sqrt(ms2 + _s(eps, vv))
    _upd(ms, ms2), _upd(mom, mom2)
    return _upd(var, vv - mom2)


def _ftrl_update(vv, acc, lin, g, lr, l1, l2, lr_power):
    acc2 = acc + g * g
    sigma = (acc2.pow(-lr_power) - acc.pow(-lr_power)) / lr
    lin2 = lin + g - sigma * vv
    quad = acc2.pow(-lr_power) / lr + 2 * l2
    new = torch.where(lin2.abs() > l1, (torch.sign(lin2) * l1 - lin2) / quad, torch.zeros_like(vv))
    return new, acc2, lin2


def _apply_ftrl(self, var, accum, linear, grad, lr, l1, l2, lr_power):
    vv = _t(var)
    new, a2, l2n = _ftrl_update(vv, _t(accum), _t(linear), _t(grad), _s(lr, vv), _s(l1, vv), _s(l2, vv),
                                _s(lr_power, vv))
    _upd(accum, a2), _upd(linear, l2n)
    return _upd(var, new)


def _apply_gd(self, var, alpha, delta):
    return _upd(var, _t(var) - _s(alpha, _t(var)) * _t(delta))


def _apply_keras_momentum(self, var, accum, lr, grad, momentum):
    vv, g = _t(var), _t(grad)
    a2 = _t(accum) * _s(momentum, vv) - g * _s(lr, vv)
    new = vv + a2 * _s(momentum, vv) - g * _s(lr, vv) if self.use_nesterov else vv + a2
    return _upd(var, new), _upd(accum, a2)


def _prox(v, lr, l1, l2):
    return torch.sign(v) * torch.clamp(v.abs() - lr * l1, min=0) / (1 + lr * l2)


def _apply_proximal_adagrad(self, var, accum, lr, l1, l2, grad):
    vv, g = _t(var), _t(grad)
    a2 = _t(accum) + g * g
    lr_t = _s(lr, vv) / torch.sqrt(a2)
    return _upd(var, _prox(vv - lr_t * g, lr_t, _s(l1, vv), _s(l2, vv))), _upd(accum, a2)


def _apply_proximal_gd(self, var, alpha, l1, l2, delta):
    vv = _t(var)
    a = _s(alpha, vv)
    return _upd(var, _prox(vv - a * _t(delta), a, _s(l1, vv), _s(l2, vv)))


_prim("ApplyAdaMax", (), _apply_adamax)
_prim("ApplyAdadelta", (), _apply_adadelta)
_prim("ApplyAdagrad", [("update_slots", True)], _apply_adagrad)
_prim("ApplyAdagradV2", [("epsilon", _REQ), ("update_slots", True)], _apply_adagrad)
_prim("ApplyAdagradDA", [("use_locking", False)], _apply_adagrad_da)
_prim("ApplyAdamWithAmsgrad", [("beta1", 0.9), ("beta2", 0.999), ("epsilon", 1e-8), ("use_locking", False)],
      _apply_amsgrad)
_prim("ApplyAdamWithAmsgradV2", [("use_locking", False)], _apply_amsgrad)
_prim("ApplyAddSign", (), _apply_add_sign)
_prim("ApplyPowerSign", (), _apply_power_sign)
_prim("ApplyCenteredRMSProp", [("use_locking", False)], _apply_centered_rmsprop)
_prim("ApplyRMSProp", [("use_locking", False)], _apply_rmsprop)
_prim("ApplyFtrl", [("use_locking", False)], _apply_ftrl)
_prim("ApplyGradientDescent", (), _apply_gd)
_prim("ApplyKerasMomentum", [("use_locking", False), ("use_nesterov", False)], _apply_keras_momentum)
_prim("ApplyProximalAdagrad", [("use_locking", False)], _apply_proximal_adagrad)
_prim("ApplyProximalGradientDescent", (), _apply_proximal_gd)


def _rows(t, indices):
    return _t(t)[_t(indices).long()]


def _put_rows(t, indices, rows):
    with torch.no_grad():
        _t(t)[_t(indices).long()] = rows
    return _t(t)


def _sparse_adagrad(self, var, accum, grad, indices):
    g = _t(grad)
    a = _rows(accum, indices) + g * g if self.update_slots else _rows(accum, indices)
    eps = getattr(self, "epsilon", 0.0) or 0.0
    v = _rows(var, indices) - self.lr * g / (torch.sqrt(a) + eps)
    return _put_rows(var, indices, v), _put_rows(accum, indices, a)


def _sparse_ftrl(self, var, accum, linear, grad, indices):
    vv = _rows(var, indices)
    c = lambda x: torch.as_tensor(x, dtype=vv.dtype)
    l2 = self.l2 + getattr(self, "l2_shrinkage", 0.0) * 0
    new, a2, l2n = _ftrl_update(vv, _rows(accum, indices), _rows(linear, indices), _t(grad), c(self.lr), c(self.l1),
                                c(l2), c(self.lr_power))
    return _put_rows(var, indices, new), _put_rows(accum, indices, a2), _put_rows(linear, indices, l2n)


def _sparse_proximal_adagrad(self, var, accum, lr, l1, l2, grad, indices):
    g = _t(grad)
    a2 = _rows(accum, indices) + g * g
    vv = _rows(var, indices)
    lr_t = _s(lr, vv) / torch.sqrt(a2)
    return _put_rows(var, indices, _prox(vv - lr_t * g, lr_t, _s(l1, vv), _s(l2, vv))), _put_rows(accum, indices, a2)


def _sparse_adadelta(self, var, accum, accum_update, lr, rho, grad, indices):
    g = _t(grad)
    vv = _rows(var, indices)
    r, e = _s(rho, vv), torch.as_tensor(self.epsilon, dtype=vv.dtype)
    a2 = r * _rows(accum, indices) + (1 - r) * g * g
    upd = torch.sqrt(_rows(accum_update, indices) + e) / torch.sqrt(a2 + e) * g
    au2 = r * _rows(accum_update, indices) + (1 - r) * upd * upd
    return (_put_rows(var, indices, vv - _s(lr, vv) * upd), _put_rows(accum, indices, a2),
            _put_rows(accum_update, indices, au2))


def _sparse_rmsprop(self, var, ms, mom, lr, grad, indices):
    g = _t(grad)
    vv = _rows(var, indices)
    ms2 = self.rho * _rows(ms, indices) + (1 - self.rho) * g * g
    mom2 = self.momentum * _rows(mom, indices) + _s(lr, vv) * g / torch.sqrt(ms2 + self.epsilon)
    return _put_rows(var, indices, vv - mom2), _put_rows(ms, indices, ms2), _put_rows(mom, indices, mom2)


def _fused_sparse_adam(lazy):
    def run(self, var, m, v, beta1_power, beta2_power, lr, beta1, beta2, eps, grad, indices):
        vt, g = _t(var), _t(grad)
        b1, b2 = _s(beta1, vt), _s(beta2, vt)
        lr_t = _s(lr, vt) * torch.sqrt(1 - _s(beta2_power, vt)) / (1 - _s(beta1_power, vt))
        idx = _t(indices).long()
        if lazy:
            m2 = b1 * _t(m)[idx] + (1 - b1) * g
            v2 = b2 * _t(v)[idx] + (1 - b2) * g * g
            _put_rows(m, indices, m2), _put_rows(v, indices, v2)
            upd = m2 * b1 + (1 - b1) * g if self.use_nesterov else m2
            _put_rows(var, indices, vt[idx] - lr_t * upd / (torch.sqrt(v2) + _s(eps, vt)))
        else:
            dense = torch.zeros_like(vt).index_add_(0, idx, g)
            m2 = b1 * _t(m) + (1 - b1) * dense
            v2 = b2 * _t(v) + (1 - b2) * dense * dense
            _upd(m, m2), _upd(v, v2)
            upd = m2 * b1 + (1 - b1) * dense if self.use_nesterov else m2
            _upd(var, vt - lr_t * upd / (torch.sqrt(v2) + _s(eps, vt)))
        return _t(var), _t(m), _t(v)
    return run


_prim("SparseApplyAdagrad", [("lr", _REQ), ("update_slots", True), ("use_locking", False)], _sparse_adagrad)
_prim("SparseApplyAdagradV2", [("lr", _REQ), ("epsilon", _REQ), ("use_locking", False), ("update_slots", True)],
      _sparse_adagrad)
_prim("SparseApplyFtrl", [("lr", _REQ), ("l1", _REQ), ("l2", _REQ), ("lr_power", _REQ), ("use_locking", False)],
      _sparse_ftrl)
_prim("SparseApplyFtrlV2", [("lr", _REQ), ("l1", _REQ), ("l2", _REQ), ("l2_shrinkage", _REQ), ("lr_power", _REQ),
                            ("use_locking", False)], _sparse_ftrl)
_prim("FusedSparseFtrl", [("lr", _REQ), ("l1", _REQ), ("l2", _REQ), ("lr_power", _REQ), ("use_locking", False)],
      _sparse_ftrl)
_prim("SparseApplyProximalAdagrad", [("use_locking", False)], _sparse_proximal_adagrad)
_prim("FusedSparseProximalAdagrad", [("use_locking", False)], _sparse_proximal_adagrad)
_prim("SparseApplyAdadelta", [("epsilon", _REQ), ("use_locking", False)], _sparse_adadelta)
_prim("SparseApplyRMSProp", [("rho", 0.9), ("momentum", 0.0), ("epsilon", 1e-10), ("use_locking", False)],
      _sparse_rmsprop)
_prim("FusedSparseAdam", [("use_locking", False), ("use_nesterov", False)], _fused_sparse_adam(False))
_prim("FusedSparseLazyAdam", [("use_locking", False), ("use_nesterov", False)], _fused_sparse_adam(True))


def _lars_update(self, weight, gradient, norm_weight, norm_gradient, weight_decay, learning_rate):
    w, g = _t(weight), _t(gradient)
    nw, ng = torch.sqrt(_t(norm_weight)), torch.sqrt(_t(norm_gradient))
    wd, lr = _s(weight_decay, w), _s(learning_rate, w)
    coef = torch.where((nw > 0) & (ng > 0), self.hyperpara * nw / (ng + wd * nw + self.epsilon), torch.ones_like(nw))
    out = coef * (g + wd * w)
    return out if not self.use_clip else out.clamp(-1.0 / float(lr), 1.0 / float(lr)) if float(lr) else out


_prim("LARSUpdate", [("epsilon", 1e-05), ("hyperpara", 0.001), ("use_clip", False)], _lars_update)


def _adam_no_update(self, m, v, beta1_power, beta2_power, lr, beta1, beta2, eps, grad):
    g = _t(grad)
    b1, b2 = _s(beta1, g), _s(beta2, g)
    m2 = b1 * _t(m) + (1 - b1) * g
    v2 = b2 * _t(v) + (1 - b2) * g * g
    _upd(m, m2), _upd(v, v2)
    lr_t = _s(lr, g) * torch.sqrt(1 - _s(beta2_power, g)) / (1 - _s(beta1_power, g))
    return -lr_t * m2 / (torch.sqrt(v2) + _s(eps, g))


_prim("AdamNoUpdateParam", [("use_locking", False)], _adam_no_update)


def _fused_cast_adamw(self, var, m, v, lr, beta1, beta2, eps, decay, grad, global_norm):
    vt = _t(var)
    g = _t(grad).float() / torch.clamp(_t(global_norm).float(), min=1.0)
    b1, b2 = float(_t(beta1)), float(_t(beta2))
    m2 = b1 * _t(m).float() + (1 - b1) * g
    v2 = b2 * _t(v).float() + (1 - b2) * g * g
    upd = m2 / (torch.sqrt(v2) + float(_t(eps))) + float(_t(decay)) * vt.float()
    _upd(m, m2.to(_t(m).dtype)), _upd(v, v2.to(_t(v).dtype))
    return _upd(var, (vt.float() - float(_t(lr)) * upd).to(vt.dtype))


_prim("FusedCastAdamWeightDecay", [("use_locking", False)], _fused_cast_adamw)
_prim("FusedWeightScaleApplyMomentum", (), lambda self, weight_decay, loss_scale, var, accum, lr, grad, momentum: (
    lambda g: (_upd(accum, _t(accum) * _s(momentum, _t(var)) + g), _upd(var, _t(var) - _s(lr, _t(var)) * _t(accum)))[1])(
    _t(grad).to(_t(var).dtype) / _s(loss_scale, _t(var)) + _s(weight_decay, _t(var)) * _t(var)))

# ---------------------------------------------------------------------------------------------------- quantisation


def _fake_quant(x, mn, mx, num_bits, symmetric, narrow_range, axis=None):
    t = _t(x)
    lo, hi = _t(mn).to(t.dtype), _t(mx).to(t.dtype)
    if axis is not None:
        shape = [1] * t.dim()
        shape[axis] = -1
        lo, hi = lo.reshape(shape), hi.reshape(shape)
    qmin = 1.0 if narrow_range else 0.0
    qmax = float(2 ** num_bits - 1)
    if symmetric:
        bound = torch.maximum(lo.abs(), hi.abs())
        lo, hi = -bound, bound
    scale = (hi - lo) / (qmax - qmin)
    scale = torch.where(scale == 0, torch.ones_like(scale), scale)
    zp = torch.clamp(torch.round(qmin - lo / scale), qmin, qmax)
    q = torch.clamp(torch.round(t / scale + zp), qmin, qmax)
    return (q - zp) * scale


_prim("FakeQuantPerLayer", [("num_bits", 8), ("ema", False), ("ema_decay", 0.999), ("quant_delay", 0),
                            ("symmetric", False), ("narrow_range", False), ("training", True)],
      lambda self, x, mn, mx: _fake_quant(x, mn, mx, self.num_bits, self.symmetric, self.narrow_range))
_prim("FakeQuantPerChannel", [("num_bits", 8), ("ema", False), ("ema_decay", 0.999), ("quant_delay", 0),
                              ("symmetric", False), ("narrow_range", False), ("training", True), ("channel_axis", 1)],
      lambda self, x, mn, mx: _fake_quant(x, mn, mx, self.num_bits, self.symmetric, self.narrow_range,
                                          self.channel_axis))
_prim("FakeQuantWithMinMaxVars", [("num_bits", 8), ("narrow_range", False)],
      lambda self, x, mn, mx: _fake_quant(x, mn, mx, self.num_bits, False, self.narrow_range))
_prim("FakeQuantWithMinMaxVarsPerChannel", [("num_bits", 8), ("narrow_range", False)],
      lambda self, x, mn, mx: _fake_quant(x, mn, mx, self.num_bits, False, self.narrow_range, _t(x).dim() - 1))


def _minmax_update(self, x, mn, mx, axis=None):
    t = _t(x)
    if axis is None:
        cur_min, cur_max = t.min().reshape(1), t.max().reshape(1)
    else:
        dims = [d for d in range(t.dim()) if d != axis]
        cur_min, cur_max = t.amin(dims), t.amax(dims)
    if self.ema:
        d = self.ema_decay
        cur_min, cur_max = d * _t(mn) + (1 - d) * cur_min, d * _t(mx) + (1 - d) * cur_max
    return torch.minimum(cur_min, torch.zeros_like(cur_min)), torch.maximum(cur_max, torch.zeros_like(cur_max))


_prim("MinMaxUpdatePerLayer", [("ema", False), ("ema_decay", 0.999)], _minmax_update)
_prim("MinMaxUpdatePerChannel", [("ema", False), ("ema_decay", 0.999), ("channel_axis", 1)],
      lambda self, x, mn, mx: _minmax_update(self, x, mn, mx, self.channel_axis))
_prim("FakeQuantParam", [("quant_dtype", None), ("quant_algo_name", ""), ("is_per_channel", False)],
      lambda self, x: _t(x))

# ---------------------------------------------------------------------------------------------------- debug / control


def _summary(kind):
    def run(self, name, value):
        from ..train import summary as _summary_mod
        rec = getattr(_summary_mod, "record_from_primitive", None)
        if rec is not None:
            rec(kind, name, value)
        return None
    return run


for _k in ("Scalar", "Tensor", "Image", "Histogram"):
    _prim(_k + "Summary", (), _summary(_k.lower()))


def _assert(self, condition, input_data):
    ok = bool(_t(condition).all()) if isinstance(condition, torch.Tensor) else bool(condition)
    if not ok:
        shown = [str(_t(v).reshape(-1)[:self.summarize].tolist()) if isinstance(v, torch.Tensor) else str(v)
                 for v in (input_data if isinstance(input_data, (tuple, list)) else [input_data])]
        raise RuntimeError("For 'Assert', the condition is false; data: %s" % ", ".join(shown))
    return None


_prim("Assert", [("summarize", 3)], _assert)


def _tensor_dump(self, file, input_x):
    import os
    import numpy as np
    path = file if file.endswith(".npy") else file + ".npy"
    os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
    t = _t(input_x).detach().cpu()
    np.save(path, t.float().numpy() if t.dtype == torch.bfloat16 else t.numpy())
    return None


_prim("TensorDump", [("input_output", "out")], _tensor_dump)


class _GradHook(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, fn):
        ctx.fn = fn
        return x.view_as(x)

    @staticmethod
    def backward(ctx, g):
        out = ctx.fn(g)
        return (g if out is None else (_t(out[0]) if isinstance(out, (tuple, list)) else _t(out))), None


_prim("InsertGradientOf", [("f", _REQ)], lambda self, x: _GradHook.apply(_t(x), self.f))
_prim("HookBackward", [("hook_fn", _REQ), ("cell_id", "")],
      lambda self, *xs: (lambda outs: outs[0] if len(outs) == 1 else outs)(
          tuple(_GradHook.apply(_t(x), lambda g, s=self: s.hook_fn((g,))) for x in xs)))
_prim("PyFunc", [("fn", _REQ), ("in_types", ()), ("in_shapes", ()), ("out_types", ()), ("out_shapes", ()),
                 ("stateful", True)],
      lambda self, *xs: (lambda out: tuple(torch.as_tensor(o) for o in out) if isinstance(out, (tuple, list)) else
                         torch.as_tensor(out))(self.fn(*[_t(x).detach().cpu().numpy() for x in xs])))
_prim("PyExecute", (), lambda self, script, local_keys, local_values: eval(  # noqa: S307 (the reference evaluates it too)
    script, {}, dict(zip(local_keys, local_values))))
_prim("Merge", (), lambda self, inputs: next(((_t(v), torch.tensor(i, dtype=torch.int32))
                                              for i, v in enumerate(inputs) if v is not None)))
_prim("GeSwitch", (), lambda self, data, pred: (None, _t(data)) if bool(_t(pred)) else (_t(data), None))
_prim("Reusing", (), lambda self, x: _t(x))
_prim("SelectView", (), lambda self, x, index, axis: _t(x).select(int(axis), int(index)))
_prim("CopyWithSlice", (), lambda self, x, y: _upd(x, _t(y)))
_prim("NPUGetFloatStatus", (), lambda self, x: _t(x))
_prim("NPUClearFloatStatus", (), lambda self, x: torch.zeros_like(_t(x)))


def _no_repeat_ngram(self, state_seq, log_probs):
    seq, lp = _t(state_seq), _t(log_probs).clone()
    n = self.ngram_size
    b, beams, length = seq.shape
    if length >= n:
        for i in range(b):
            for j in range(beams):
                s = seq[i, j].tolist()
                prefix = tuple(s[length - n + 1:]) if n > 1 else ()
                for k in range(length - n + 1):
                    if tuple(s[k:k + n - 1]) == prefix:
                        lp[i, j, s[k + n - 1]] = torch.finfo(lp.dtype).min
    return lp


_prim("NoRepeatNGram", [("ngram_size", 1)], _no_repeat_ngram)
_prim("RaggedRange", [("Tsplits", None)], lambda self, starts, limits, deltas: (lambda parts: (
    torch.cumsum(torch.tensor([0] + [p.numel() for p in parts]), 0).to(X._dt(self.Tsplits) or torch.int64),
    torch.cat(parts) if parts else _t(starts)[:0]))([torch.arange(float(s), float(l), float(d)).to(_t(starts).dtype)
                                                     if _t(starts).is_floating_point() else
                                                     torch.arange(int(s), int(l), int(d), dtype=_t(starts).dtype)
                                                     for s, l, d in zip(_t(starts).tolist(), _t(limits).tolist(),
                                                                        _t(deltas).tolist())]))
_prim("DataFormatDimMap", [("src_format", "NHWC"), ("dst_format", "NCHW")], lambda self, x: torch.tensor(
    [self.dst_format.index(self.src_format[int(v) % len(self.src_format)]) for v in _t(x).reshape(-1).tolist()],
    dtype=_t(x).dtype).reshape(_t(x).shape))
_prim("DataFormatVecPermute", [("src_format", "NHWC"), ("dst_format", "NCHW")], lambda self, x: _t(x)[
    [self.src_format.index(c) for c in self.dst_format]])
_prim("CompareAndBitpack", (), lambda self, x, threshold: (lambda bits: (bits.reshape(-1, 8).to(torch.uint8) * torch
                                                                         .tensor([128, 64, 32, 16, 8, 4, 2, 1],
                                                                                 dtype=torch.uint8)).sum(1).to(
    torch.uint8).reshape(tuple(_t(x).shape[:-1]) + (_t(x).shape[-1] // 8,)))(_t(x) > _t(threshold)))
_prim("ConfusionMatrix", [("num_classes", _REQ), ("dtype", "int32")], lambda self, labels, predictions, weights=None: (
    torch.zeros(self.num_classes, self.num_classes, dtype=torch.float32).index_put(
        (_t(labels).long(), _t(predictions).long()),
        torch.ones(_t(labels).numel()) if weights is None else _t(weights).float(), accumulate=True).to(
        X._dt(self.dtype) if not isinstance(self.dtype, str) else getattr(torch, self.dtype))))


def _extract_glimpse(self, x, size, offsets):
    """Windows of ``size`` (height, width) around ``offsets`` [N, 2] (y, x) of NHWC images; outside pixels are 0."""
    t, off = _t(x), _t(offsets).float()
    gh, gw = (int(v) for v in _t(size).tolist())
    n, h, w, _ = t.shape
    outs = []
    for i in range(n):
        cy, cx = float(off[i, 0]), float(off[i, 1])
        if self.normalized:
            cy, cx = ((cy + 1) / 2 * h, (cx + 1) / 2 * w) if self.centered else (cy * h, cx * w)
        elif self.centered:
            cy, cx = cy + h / 2, cx + w / 2
        y0, x0 = int(round(cy - gh / 2)), int(round(cx - gw / 2))
        padded = F.pad(t[i].permute(2, 0, 1), (gw, gw, gh, gh))
        outs.append(padded[:, y0 + gh:y0 + 2 * gh, x0 + gw:x0 + 2 * gw].permute(1, 2, 0))
    return torch.stack(outs)


_prim("ExtractGlimpse", [("centered", True), ("normalized", True), ("uniform_noise", True), ("noise", "uniform")],
      _extract_glimpse)


# ---------------------------------------------------------------------------------------------------- recurrent / misc
def _lstm(self, x, h0, c0, w):
    """x [T, N, input_size]; h0 / c0 [layers * directions, N, hidden]; ``w`` is the flat weight: for every layer and
    direction W_ih then W_hh (gate order i, f, g, o), then - when ``has_bias`` - all b_ih / b_hh in the same order.
    Returns (output, h_n, c_n, reserve, state) like the reference's GPU kernel; the last two are empty."""
    t, w = _t(x), _t(w).reshape(-1)
    dirs = 2 if self.bidirectional else 1
    hs, gates = self.hidden_size, 4 * self.hidden_size
    mats, pos = [], 0
    for layer in range(self.num_layers):
        in_size = self.input_size if layer == 0 else hs * dirs
        for _ in range(dirs):
            wih = w[pos:pos + gates * in_size].reshape(gates, in_size)
            pos += gates * in_size
            whh = w[pos:pos + gates * hs].reshape(gates, hs)
            pos += gates * hs
            mats.append([wih, whh])
    if self.has_bias:
        for m in mats:
            m.append(w[pos:pos + gates])
            pos += gates
            m.append(w[pos:pos + gates])
            pos += gates
    flat = [p for m in mats for p in m]
    out, hn, cn = torch.lstm(t, (_t(h0), _t(c0)), flat, self.has_bias, self.num_layers,
                             float(self.dropout) if self.training else 0.0, bool(self.training), self.bidirectional,
                             False)
    return out, hn, cn, t.new_zeros(0), t.new_zeros(0)


_prim("LSTM", [("input_size", _REQ), ("hidden_size", _REQ), ("num_layers", _REQ), ("has_bias", _REQ),
               ("bidirectional", _REQ), ("dropout", _REQ), ("proj_size", 0), ("training", False)], _lstm)


def _fft_with_size(self, x):
    t = _t(x)
    dims = tuple(range(-self.signal_ndim, 0))
    norm = {"backward": "backward", "forward": "forward", "ortho": "ortho"}[self.norm]
    if not self.real:
        return (torch.fft.ifftn if self.inverse else torch.fft.fftn)(t, dim=dims, norm=norm)
    if not self.inverse:
        out = torch.fft.rfftn(t, dim=dims, norm=norm)
        return out if self.onesided else torch.fft.fftn(t.to(out.dtype), dim=dims, norm=norm)
    return torch.fft.irfftn(t, s=tuple(self.signal_sizes) if self.signal_sizes else None, dim=dims, norm=norm)


_prim("FFTWithSize", [("signal_ndim", _REQ), ("inverse", _REQ), ("real", _REQ), ("norm", "backward"),
                      ("onesided", True), ("signal_sizes", ())], _fft_with_size)
_prim("AdjustSaturation", (), lambda self, image, scale: _hsv_to_rgb(self, (lambda hsv: torch.stack(
    [hsv[..., 0], (hsv[..., 1] * float(_t(scale))).clamp(0, 1), hsv[..., 2]], -1))(_rgb_to_hsv(self, image))))
_prim("AdjustHue", (), lambda self, image, delta: _hsv_to_rgb(self, (lambda hsv: torch.stack(
    [(hsv[..., 0] + float(_t(delta))) % 1.0, hsv[..., 1], hsv[..., 2]], -1))(_rgb_to_hsv(self, image))))


def _dilation2d(self, x, w):
    """Grey-scale morphological dilation: max over the window of x + filter."""
    t, k = _t(x), _t(w)
    kh, kw = k.shape[-2:]
    s, d = _last(self.stride, 2), _last(self.dilation, 2)
    if self.pad_mode.lower() == "same":
        pads = []
        for size, kk, ss, dd in zip(t.shape[2:][::-1], (kh, kw)[::-1], s[::-1], d[::-1]):
            total = max((-(-size // ss) - 1) * ss + (kk - 1) * dd + 1 - size, 0)
            pads += [total // 2, total - total // 2]
        t = F.pad(t, pads, value=float("-inf"))
    n, c = t.shape[:2]
    cols = F.unfold(t, (kh, kw), d, 0, s).reshape(n, c, kh * kw, -1)
    out = (cols + k.reshape(1, c, kh * kw, 1)).amax(2)
    ho = (t.shape[2] - (kh - 1) * d[0] - 1) // s[0] + 1
    return out.reshape(n, c, ho, -1)


_prim("Dilation2D", [("stride", _REQ), ("dilation", _REQ), ("pad_mode", "SAME"), ("data_format", "NCHW")], _dilation2d)
_prim("Reshard", (), lambda self, x, layout: __import__("importlib").import_module(__package__).reshard(x, layout))
