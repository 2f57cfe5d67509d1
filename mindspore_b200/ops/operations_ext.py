"""Second tier of primitives: everything that has a distributed ``*Info`` in the reference
(frontend/parallel/ops_info/*.cc ``REGISTER`` entries) but is not on a training hot path - extended arithmetic,
scatter / segment families, 3-D convolution and pooling, quantisation helpers, detection helpers and the
inference-time attention / KV-cache operators.  Each is a thin ``Primitive`` over torch ops; attribute names and
input orders follow python/mindspore/ops/operations/{math_ops,array_ops,nn_ops,_inner_ops}.py and
ops/auto_generate/gen_ops_prim.py.  Everything here is re-exported from ``ops.operations``."""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F

from . import fused
from .primitive import Primitive, prim_attr_register

__all__ = []


def _export(cls):
    __all__.append(cls.__name__)
    return cls


def _simple(name, fn, doc=None):
    def __init__(self):
        Primitive.__init__(self, name)

    def _run(self, *args):
        return fn(*args)

    cls = type(name, (Primitive,), {"__init__": __init__, "_run": _run, "__doc__": doc or "%s." % name})
    globals()[name] = cls
    __all__.append(name)
    return cls


def _tt(x, like):
    return x if isinstance(x, torch.Tensor) else torch.as_tensor(x, device=like.device)


# ------------------------------------------------------------------------------------------------ arithmetic
_simple("BesselJ0", torch.special.bessel_j0)
_simple("BesselJ1", torch.special.bessel_j1)
_simple("Igamma", lambda a, x: torch.special.gammainc(a, x))
_simple("Igammac", lambda a, x: torch.special.gammaincc(a, x))
_simple("NextAfter", torch.nextafter)
if "Zeta" not in globals():
    _simple("Zeta", torch.special.zeta)
_simple("Gcd", torch.gcd)
_simple("LeftShift", torch.bitwise_left_shift)
_simple("RightShift", torch.bitwise_right_shift)
_simple("AddExt", lambda x, y, alpha=1: torch.add(x, _tt(y, x), alpha=alpha))
_simple("SubExt", lambda x, y, alpha=1: torch.sub(x, _tt(y, x), alpha=alpha))
_simple("DivMod", lambda x, y, rounding_mode=None: torch.div(x, _tt(y, x), rounding_mode=rounding_mode))
_simple("ClampScalar", lambda x, lo=None, hi=None: torch.clamp(x, lo, hi))
_simple("SumExt", lambda x, dim=None, keepdim=False, dtype=None:
        torch.sum(x, dtype=dtype) if dim is None else torch.sum(x, dim=dim, keepdim=keepdim, dtype=dtype))
_simple("Cholesky", lambda x, upper=False: torch.linalg.cholesky(x, upper=bool(upper)))
_simple("TensorDot", lambda a, b, axes=2: torch.tensordot(a, b, dims=axes))
_simple("Cdist", lambda x, y, p=2.0: torch.cdist(x, y, p=float(p)))
_simple("IndexSelect", lambda x, axis, index: torch.index_select(x, int(axis), index.long()))
_simple("RepeatElements", lambda x, rep=1, axis=0: torch.repeat_interleave(x, int(rep), dim=int(axis)))
_simple("SliceExt", lambda x, dim, start, end, step=1: x[(slice(None),) * (dim % x.dim()) + (slice(start, end, step),)])
_simple("SplitTensor", lambda x, split_size, dim=0: tuple(torch.split(x, int(split_size), dim=dim)))
_simple("SplitWithSize", lambda x, sizes, dim=0: tuple(torch.split(x, [int(s) for s in sizes], dim=dim)))
_simple("StackExt", lambda xs, dim=0: torch.stack(list(xs), dim=dim))
_simple("TopkExt", lambda x, k, dim=-1, largest=True, sorted=True:  # noqa: A002
        tuple(torch.topk(x, int(k), dim=dim, largest=largest, sorted=sorted)))
_simple("OneHotExt", lambda x, num_classes=-1: F.one_hot(x.long(), int(num_classes)))
_simple("LinSpaceExt", lambda start, end, steps, dtype=None: torch.linspace(float(start), float(end), int(steps),
                                                                          dtype=dtype))
_simple("BatchMatMulExt", lambda a, b: torch.matmul(a, b))
_simple("HShrink", lambda x, lambd=0.5: F.hardshrink(x, lambd))
_simple("SoftShrink", lambda x, lambd=0.5: F.softshrink(x, lambd))
_simple("Cummax", lambda x, axis=0: tuple(torch.cummax(x, dim=axis)))
_simple("Cummin", lambda x, axis=0: tuple(torch.cummin(x, dim=axis)))


@_export
class Betainc(Primitive):
    """Regularised incomplete beta function I_x(a, b) by the continued fraction of Lentz (fp64 internally)."""

    def __init__(self):
        super().__init__("Betainc")

    def _run(self, a, b, x):
        dt = x.dtype
        a, b, x = (t.double() for t in torch.broadcast_tensors(a, b, x))
        swap = x > (a + 1) / (a + b + 2)
        aa, bb, xx = torch.where(swap, b, a), torch.where(swap, a, b), torch.where(swap, 1 - x, x)
        lbeta = torch.lgamma(aa) + torch.lgamma(bb) - torch.lgamma(aa + bb)
        front = torch.exp(aa * torch.log(xx.clamp_min(1e-300)) + bb * torch.log1p(-xx.clamp_max(1 - 1e-16)) - lbeta) / aa
        tiny = 1e-300
        f, c, d = torch.ones_like(xx), torch.ones_like(xx), torch.zeros_like(xx)
        for i in range(200):
            m = i // 2
            if i == 0:
                num = torch.ones_like(xx)
            elif i % 2 == 0:
                num = m * (bb - m) * xx / ((aa + 2 * m - 1) * (aa + 2 * m))
            else:
                num = -(aa + m) * (aa + bb + m) * xx / ((aa + 2 * m) * (aa + 2 * m + 1))
            d = 1 + num * d
            d = torch.where(d.abs() < tiny, torch.full_like(d, tiny), d)
            d = 1 / d
            c = 1 + num / c
            c = torch.where(c.abs() < tiny, torch.full_like(c, tiny), c)
            f = f * c * d
        res = front * (f - 1)
        res = torch.where(swap, 1 - res, res)
        res = torch.where(x <= 0, torch.zeros_like(res), torch.where(x >= 1, torch.ones_like(res), res))
        return res.to(dt)


@_export
class PopulationCount(Primitive):
    def __init__(self):
        super().__init__("PopulationCount")

    def _run(self, x):
        bits = x.element_size() * 8
        v = x.to(torch.int64) & ((1 << bits) - 1 if bits < 64 else -1)
        cnt = torch.zeros_like(v)
        for i in range(bits):
            cnt += (v >> i) & 1
        return cnt.to(torch.uint8)


@_export
class Gamma(Primitive):
    """Samples Gamma(alpha, beta) of the given shape (python/mindspore/ops/operations/random_ops.py ``Gamma``)."""

    @prim_attr_register
    def __init__(self, seed=0, seed2=0):
        pass

    def _run(self, shape, alpha, beta):
        alpha = alpha.float().expand(tuple(shape)) if isinstance(alpha, torch.Tensor) else torch.full(tuple(shape), float(alpha))
        beta = beta if isinstance(beta, torch.Tensor) else torch.tensor(float(beta))
        return torch._standard_gamma(alpha.contiguous()) / beta.to(alpha.device)


# ------------------------------------------------------------------------------------------------ scatter family
def _scatter_param(name, reduce):
    """Scatter*(input_x: Parameter, indices, updates): rows of ``input_x`` selected by ``indices`` are combined with
    ``updates`` in place (indices of any shape; updates.shape = indices.shape + input_x.shape[1:])."""

    def __init__(self, use_locking=False):
        Primitive.__init__(self, name)
        self.add_prim_attr("use_locking", use_locking)

    def _run(self, x, indices, updates):
        idx = indices.reshape(-1).long()
        upd = updates.reshape((idx.numel(),) + tuple(x.shape[1:])).to(x.dtype)
        with torch.no_grad():
            if reduce == "update":
                x.index_copy_(0, idx, upd)
            elif reduce == "add":
                x.index_add_(0, idx, upd)
            elif reduce == "sub":
                x.index_add_(0, idx, -upd)
            else:
                full = idx.reshape((-1,) + (1,) * (x.dim() - 1)).expand_as(upd)
                if reduce == "div":
                    x.scatter_reduce_(0, full, 1.0 / upd, reduce="prod", include_self=True)
                else:
                    x.scatter_reduce_(0, full, upd, reduce={"mul": "prod", "max": "amax", "min": "amin"}[reduce],
                                      include_self=True)
        return x

    cls = type(name, (Primitive,), {"__init__": __init__, "_run": _run, "__doc__": _scatter_param.__doc__})
    globals()[name] = cls
    __all__.append(name)


for _n, _r in (("ScatterUpdate", "update"), ("ScatterAdd", "add"), ("ScatterSub", "sub"), ("ScatterMul", "mul"),
               ("ScatterDiv", "div"), ("ScatterMax", "max"), ("ScatterMin", "min")):
    _scatter_param(_n, _r)


def _nd_index(indices):
    return tuple(indices.long()[..., i] for i in range(indices.shape[-1]))


def _scatter_nd(name, reduce, inplace):
    def __init__(self, use_locking=False):
        Primitive.__init__(self, name)

    def _run(self, x, indices, updates):
        out = x if inplace else x.clone()
        ix = _nd_index(indices)
        upd = updates.to(out.dtype)
        with torch.no_grad() if inplace else torch.enable_grad():
            if reduce == "update":
                out.index_put_(ix, upd)
            elif reduce in ("add", "sub"):
                out.index_put_(ix, upd if reduce == "add" else -upd, accumulate=True)
            else:
                # flatten the indexed prefix and reduce with scatter_reduce
                k = indices.shape[-1]
                strides = [1] * k
                for i in range(k - 2, -1, -1):
                    strides[i] = strides[i + 1] * out.shape[i + 1]
                flat = sum(indices.long()[..., i] * strides[i] for i in range(k)).reshape(-1)
                tail = tuple(out.shape[k:])
                o2 = out.reshape((-1,) + tail)
                u2 = upd.reshape((flat.numel(),) + tail)
                full = flat.reshape((-1,) + (1,) * len(tail)).expand_as(u2)
                if reduce == "div":
                    u2, red = 1.0 / u2, "prod"
                else:
                    red = {"mul": "prod", "max": "amax", "min": "amin"}[reduce]
                res = o2.scatter_reduce(0, full, u2, reduce=red, include_self=True)
                if inplace:
                    out.copy_(res.reshape(out.shape))
                else:
                    out = res.reshape(out.shape)
        return out

    cls = type(name, (Primitive,), {"__init__": __init__, "_run": _run,
                                    "__doc__": "%s(input_x, indices[..., K], updates)." % name})
    globals()[name] = cls
    __all__.append(name)


for _n, _r in (("ScatterNdUpdate", "update"), ("ScatterNdAdd", "add"), ("ScatterNdSub", "sub")):
    _scatter_nd(_n, _r, True)
for _n, _r in (("TensorScatterSub", "sub"), ("TensorScatterMul", "mul"), ("TensorScatterDiv", "div"),
               ("TensorScatterMax", "max"), ("TensorScatterMin", "min")):
    _scatter_nd(_n, _r, False)


def _segment(name, red, init):
    def __init__(self):
        Primitive.__init__(self, name)

    def _run(self, x, segment_ids, num_segments):
        n = int(num_segments)
        ids = segment_ids.reshape(-1).long()
        lead = segment_ids.dim()
        flat = x.reshape((ids.numel(),) + tuple(x.shape[lead:]))
        out = torch.full((n,) + tuple(flat.shape[1:]), init(x.dtype), dtype=x.dtype, device=x.device)
        full = ids.reshape((-1,) + (1,) * (flat.dim() - 1)).expand_as(flat)
        return out.scatter_reduce(0, full, flat, reduce=red, include_self=True)

    cls = type(name, (Primitive,), {"__init__": __init__, "_run": _run,
                                    "__doc__": "%s(x, segment_ids, num_segments)." % name})
    globals()[name] = cls
    __all__.append(name)


def _lowest(dt):
    return torch.finfo(dt).min if dt.is_floating_point else torch.iinfo(dt).min


def _highest(dt):
    return torch.finfo(dt).max if dt.is_floating_point else torch.iinfo(dt).max


_segment("UnsortedSegmentMax", "amax", _lowest)
_segment("UnsortedSegmentMin", "amin", _highest)
_segment("UnsortedSegmentProd", "prod", lambda dt: 1)


def _inplace_rows(name, mode):
    def __init__(self, indices):
        Primitive.__init__(self, name)
        self.add_prim_attr("indices", indices)
        self.indices = (indices,) if isinstance(indices, int) else tuple(indices)

    def _run(self, x, v):
        out = x.clone()
        idx = torch.as_tensor(self.indices, device=x.device)
        if mode == "update":
            out[idx] = v.to(x.dtype)
        else:
            out[idx] = out[idx] + (v if mode == "add" else -v).to(x.dtype)
        return out

    cls = type(name, (Primitive,), {"__init__": __init__, "_run": _run, "__doc__": "%s(indices)(x, v)." % name})
    globals()[name] = cls
    __all__.append(name)


_inplace_rows("InplaceAdd", "add")
_inplace_rows("InplaceSub", "sub")
_inplace_rows("InplaceUpdate", "update")


# ------------------------------------------------------------------------------------------------ nn: conv / pool / norm
def _triple(v):
    return (v,) * 3 if isinstance(v, int) else tuple(v)[-3:]


def _pair(v):
    return (v,) * 2 if isinstance(v, int) else tuple(v)[-2:]


@_export
class Conv3D(Primitive):
    @prim_attr_register
    def __init__(self, out_channel, kernel_size, mode=1, pad_mode="valid", pad=0, stride=1, dilation=1, group=1,
                 data_format="NCDHW"):
        pass

    def _run(self, x, w, bias=None):
        st, dl = _triple(self.stride), _triple(self.dilation)
        if self.pad_mode == "same":
            pads = []
            for i in range(3):
                size, k = x.shape[2 + i], (w.shape[2 + i] - 1) * dl[i] + 1
                total = max((math.ceil(size / st[i]) - 1) * st[i] + k - size, 0)
                pads = [total // 2, total - total // 2] + pads
            x = F.pad(x, pads)
            padding = 0
        elif self.pad_mode == "pad":
            p = self.pad
            if isinstance(p, int):
                padding = p
            else:
                x = F.pad(x, [p[4], p[5], p[2], p[3], p[0], p[1]])
                padding = 0
        else:
            padding = 0
        return F.conv3d(x, w, bias, st, padding, dl, self.group)


def _pool3d(name, fn):
    def __init__(self, kernel_size=1, strides=1, pad_mode="valid", pad_list=0, ceil_mode=None, data_format="NCDHW",
                 count_include_pad=True, divisor_override=0):
        Primitive.__init__(self, name)
        self.kernel_size, self.strides, self.pad_mode = _triple(kernel_size), _triple(strides), pad_mode.lower()
        self.pad_list, self.ceil_mode = pad_list, bool(ceil_mode)
        self.count_include_pad = count_include_pad

    def _run(self, x):
        if self.pad_mode == "same":
            pads = []
            for i in range(3):
                size, k, s = x.shape[2 + i], self.kernel_size[i], self.strides[i]
                total = max((math.ceil(size / s) - 1) * s + k - size, 0)
                pads = [total // 2, total - total // 2] + pads
            x = F.pad(x, pads, value=float("-inf") if fn is F.max_pool3d else 0.0)
            padding = 0
        elif self.pad_mode == "pad":
            padding = self.pad_list if isinstance(self.pad_list, int) else tuple(self.pad_list)[::2]
        else:
            padding = 0
        if fn is F.max_pool3d:
            return fn(x, self.kernel_size, self.strides, padding, ceil_mode=self.ceil_mode)
        return fn(x, self.kernel_size, self.strides, padding, ceil_mode=self.ceil_mode,
                  count_include_pad=self.count_include_pad)

    cls = type(name, (Primitive,), {"__init__": __init__, "_run": _run, "__doc__": "%s over NCDHW input." % name})
    globals()[name] = cls
    __all__.append(name)


_pool3d("MaxPool3D", F.max_pool3d)
_pool3d("AvgPool3D", F.avg_pool3d)


@_export
class Conv2DBackpropInput(Primitive):
    """Gradient of Conv2D with respect to its input: (dout, weight, input_size) -> dx."""

    @prim_attr_register
    def __init__(self, out_channel, kernel_size, pad_mode="valid", pad=0, pad_list=None, mode=1, stride=1, dilation=1,
                 group=1, data_format="NCHW"):
        pass

    def _run(self, dout, w, input_size):
        st, dl = _pair(self.stride), _pair(self.dilation)
        size = tuple(int(s) for s in input_size)
        if self.pad_mode == "same":
            pad = []
            for i in range(2):
                k = (w.shape[2 + i] - 1) * dl[i] + 1
                total = max((math.ceil(size[2 + i] / st[i]) - 1) * st[i] + k - size[2 + i], 0)
                pad.append(total // 2)
        elif self.pad_mode == "pad":
            p = self.pad
            pad = [p, p] if isinstance(p, int) else [p[0], p[2]]
        else:
            pad = [0, 0]
        return torch.nn.grad.conv2d_input(size, w, dout, st, pad, dl, self.group)


@_export
class Convolution(Primitive):
    """Generic N-d convolution (ops/auto_generate ``Convolution``): (input, weight, bias, stride, padding, dilation,
    transposed, output_padding, groups)."""

    def __init__(self):
        super().__init__("Convolution")

    def _run(self, x, w, bias=None, stride=1, padding=0, dilation=1, transposed=False, output_padding=0, groups=1):
        nd = x.dim() - 2
        fwd = {1: F.conv1d, 2: F.conv2d, 3: F.conv3d}[nd]
        bwd = {1: F.conv_transpose1d, 2: F.conv_transpose2d, 3: F.conv_transpose3d}[nd]
        if transposed:
            return bwd(x, w, bias, stride, padding, output_padding, groups, dilation)
        return fwd(x, w, bias, stride, padding, dilation, groups)


@_export
class GroupNorm(Primitive):
    def __init__(self):
        super().__init__("GroupNorm")

    def _run(self, x, num_groups, gamma=None, beta=None, eps=1e-5):
        y = F.group_norm(x, int(num_groups), gamma, beta, eps)
        g = x.float().reshape(x.shape[0], int(num_groups), -1)
        mean, var = g.mean(-1), g.var(-1, unbiased=False)
        return y, mean, torch.rsqrt(var + eps)


@_export
class LayerNormV3(Primitive):
    """LayerNorm that returns (y, mean, rstd)."""

    @prim_attr_register
    def __init__(self, begin_norm_axis=1, begin_params_axis=1, epsilon=1e-7):
        pass

    def _run(self, x, gamma, beta):
        ax = self.begin_norm_axis % x.dim()
        dims = tuple(range(ax, x.dim()))
        y = fused.layer_norm(x, gamma, beta, self.epsilon) if ax == x.dim() - 1 else \
            F.layer_norm(x, tuple(x.shape[ax:]), gamma, beta, self.epsilon)
        xf = x.float()
        mean = xf.mean(dims, keepdim=True)
        return y, mean, torch.rsqrt(xf.var(dims, unbiased=False, keepdim=True) + self.epsilon)


@_export
class Activation(Primitive):
    """Activation selected by name (the reference's ``ActivationInfo`` family)."""

    _FN = {"relu": F.relu, "relu6": F.relu6, "sigmoid": torch.sigmoid, "tanh": torch.tanh, "gelu": F.gelu,
           "fast_gelu": lambda x: x * torch.sigmoid(1.702 * x), "silu": F.silu, "swish": F.silu, "elu": F.elu,
           "hswish": F.hardswish, "hsigmoid": F.hardsigmoid, "mish": F.mish, "softplus": F.softplus}

    @prim_attr_register
    def __init__(self, activation_type="relu"):
        pass

    def _run(self, x):
        return self._FN[self.activation_type.lower()](x)


@_export
class GridSampler2D(Primitive):
    @prim_attr_register
    def __init__(self, interpolation_mode="bilinear", padding_mode="zeros", align_corners=False):
        pass

    def _run(self, x, grid):
        return F.grid_sample(x, grid, mode=self.interpolation_mode, padding_mode=self.padding_mode,
                             align_corners=self.align_corners)


@_export
class CropAndResize(Primitive):
    """(image NHWC, boxes [n, 4] normalised y1 x1 y2 x2, box_index [n], crop_size (h, w)) -> [n, h, w, C]."""

    @prim_attr_register
    def __init__(self, method="bilinear", extrapolation_value=0.0):
        pass

    def _run(self, image, boxes, box_index, crop_size):
        ch, cw = int(crop_size[0]), int(crop_size[1])
        n = boxes.shape[0]
        img = image.permute(0, 3, 1, 2).float()[box_index.long()]
        y1, x1, y2, x2 = (boxes[:, i].float() for i in range(4))
        ty = torch.linspace(0, 1, ch, device=image.device) if ch > 1 else torch.full((1,), 0.5, device=image.device)
        tx = torch.linspace(0, 1, cw, device=image.device) if cw > 1 else torch.full((1,), 0.5, device=image.device)
        ys = y1[:, None] + (y2 - y1)[:, None] * ty[None]
        xs = x1[:, None] + (x2 - x1)[:, None] * tx[None]
        grid = torch.stack([xs[:, None, :].expand(n, ch, cw) * 2 - 1, ys[:, :, None].expand(n, ch, cw) * 2 - 1], -1)
        mode = "bilinear" if self.method.startswith("bilinear") else "nearest"
        out = F.grid_sample(img, grid, mode=mode, padding_mode="zeros", align_corners=True)
        outside = (grid.abs() > 1).any(-1)[:, None].expand_as(out)
        out = torch.where(outside, torch.full_like(out, self.extrapolation_value), out)
        return out.permute(0, 2, 3, 1)


@_export
class ROIAlign(Primitive):
    """(features NCHW, rois [n, 5] = batch index, x1, y1, x2, y2) -> [n, C, pooled_h, pooled_w], average of
    ``sample_num`` x ``sample_num`` bilinear samples per bin."""

    @prim_attr_register
    def __init__(self, pooled_height, pooled_width, spatial_scale, sample_num=2, roi_end_mode=1):
        pass

    def _run(self, feat, rois):
        n, (ph, pw), s = rois.shape[0], (self.pooled_height, self.pooled_width), max(1, int(self.sample_num))
        H, W = feat.shape[2:]
        off = 1.0 if self.roi_end_mode == 1 else 0.0
        x1, y1 = rois[:, 1] * self.spatial_scale, rois[:, 2] * self.spatial_scale
        x2, y2 = (rois[:, 3] + off) * self.spatial_scale, (rois[:, 4] + off) * self.spatial_scale
        bw, bh = (x2 - x1).clamp_min(1e-6) / pw, (y2 - y1).clamp_min(1e-6) / ph
        iy = (torch.arange(ph * s, device=feat.device).float() + 0.5) / s
        ix = (torch.arange(pw * s, device=feat.device).float() + 0.5) / s
        ys = y1[:, None] + iy[None] * bh[:, None]
        xs = x1[:, None] + ix[None] * bw[:, None]
        gx = (xs / max(W - 1, 1)) * 2 - 1
        gy = (ys / max(H - 1, 1)) * 2 - 1
        grid = torch.stack([gx[:, None, :].expand(n, ph * s, pw * s), gy[:, :, None].expand(n, ph * s, pw * s)], -1)
        samples = F.grid_sample(feat.float()[rois[:, 0].long()], grid, mode="bilinear", padding_mode="border",
                                align_corners=True)
        return F.avg_pool2d(samples, s).to(feat.dtype)


# ------------------------------------------------------------------------------------------------ detection helpers
@_export
class IOU(Primitive):
    @prim_attr_register
    def __init__(self, mode="iou"):
        pass

    def _run(self, anchors, gt):
        a, g = anchors.float(), gt.float()
        area_a = (a[:, 2] - a[:, 0] + 1) * (a[:, 3] - a[:, 1] + 1)
        area_g = (g[:, 2] - g[:, 0] + 1) * (g[:, 3] - g[:, 1] + 1)
        lt = torch.maximum(g[:, None, :2], a[None, :, :2])
        rb = torch.minimum(g[:, None, 2:], a[None, :, 2:])
        wh = (rb - lt + 1).clamp_min(0)
        inter = wh[..., 0] * wh[..., 1]
        denom = (area_g[:, None] + area_a[None] - inter) if self.mode == "iou" else area_g[:, None]
        return (inter / denom.clamp_min(1e-9)).to(anchors.dtype)


@_export
class BoundingBoxEncode(Primitive):
    @prim_attr_register
    def __init__(self, means=(0.0, 0.0, 0.0, 0.0), stds=(1.0, 1.0, 1.0, 1.0)):
        pass

    def _run(self, anchor, gt):
        a, g = anchor.float(), gt.float()
        aw, ah = a[:, 2] - a[:, 0] + 1, a[:, 3] - a[:, 1] + 1
        gw, gh = g[:, 2] - g[:, 0] + 1, g[:, 3] - g[:, 1] + 1
        ax, ay = (a[:, 0] + a[:, 2]) * 0.5, (a[:, 1] + a[:, 3]) * 0.5
        gx, gy = (g[:, 0] + g[:, 2]) * 0.5, (g[:, 1] + g[:, 3]) * 0.5
        d = torch.stack([(gx - ax) / aw, (gy - ay) / ah, torch.log(gw / aw), torch.log(gh / ah)], 1)
        m, s = (torch.tensor(v, device=d.device) for v in (self.means, self.stds))
        return ((d - m) / s).to(anchor.dtype)


@_export
class BoundingBoxDecode(Primitive):
    @prim_attr_register
    def __init__(self, max_shape, means=(0.0, 0.0, 0.0, 0.0), stds=(1.0, 1.0, 1.0, 1.0), wh_ratio_clip=0.016):
        pass

    def _run(self, anchor, deltas):
        a = anchor.float()
        m, s = (torch.tensor(v, device=a.device) for v in (self.means, self.stds))
        d = deltas.float() * s + m
        lim = abs(math.log(self.wh_ratio_clip))
        dw, dh = d[:, 2].clamp(-lim, lim), d[:, 3].clamp(-lim, lim)
        aw, ah = a[:, 2] - a[:, 0] + 1, a[:, 3] - a[:, 1] + 1
        ax, ay = (a[:, 0] + a[:, 2]) * 0.5, (a[:, 1] + a[:, 3]) * 0.5
        gx, gy, gw, gh = ax + d[:, 0] * aw, ay + d[:, 1] * ah, aw * torch.exp(dw), ah * torch.exp(dh)
        H, W = self.max_shape[0], self.max_shape[1]
        out = torch.stack([(gx - gw * 0.5 + 0.5).clamp(0, W - 1), (gy - gh * 0.5 + 0.5).clamp(0, H - 1),
                           (gx + gw * 0.5 - 0.5).clamp(0, W - 1), (gy + gh * 0.5 - 0.5).clamp(0, H - 1)], 1)
        return out.to(anchor.dtype)


@_export
class CheckValid(Primitive):
    def __init__(self):
        super().__init__("CheckValid")

    def _run(self, bboxes, img_metas):
        h, w = img_metas[0] * img_metas[2], img_metas[1] * img_metas[2]
        b = bboxes.float()
        return (b[:, 0] >= 0) & (b[:, 1] >= 0) & (b[:, 2] <= w - 1) & (b[:, 3] <= h - 1)


@_export
class RandomChoiceWithMask(Primitive):
    """Indices of up to ``count`` randomly chosen True elements, padded with zeros, and the validity mask."""

    @prim_attr_register
    def __init__(self, count=256, seed=0, seed2=0):
        pass

    def _run(self, x):
        idx = torch.nonzero(x)
        perm = torch.randperm(idx.shape[0], device=x.device)[:self.count]
        chosen = idx[perm]
        n = chosen.shape[0]
        out = torch.zeros((self.count, x.dim()), dtype=torch.int32, device=x.device)
        out[:n] = chosen.to(torch.int32)
        mask = torch.zeros(self.count, dtype=torch.bool, device=x.device)
        mask[:n] = True
        return out, mask


@_export
class UniformCandidateSampler(Primitive):
    @prim_attr_register
    def __init__(self, num_true, num_sampled, unique, range_max, seed=0, remove_accidental_hits=False):
        pass

    def _run(self, true_classes):
        dev = true_classes.device
        if self.unique:
            sampled = torch.randperm(self.range_max, device=dev)[:self.num_sampled]
            p = 1.0 - (1.0 - 1.0 / self.range_max) ** self.num_sampled
        else:
            sampled = torch.randint(0, self.range_max, (self.num_sampled,), device=dev)
            p = self.num_sampled / self.range_max
        return (sampled.to(true_classes.dtype), torch.full(true_classes.shape, p, device=dev),
                torch.full((self.num_sampled,), p, device=dev))


# ------------------------------------------------------------------------------------------------ quantisation
def _round_half_away(x):
    return torch.sign(x) * torch.floor(x.abs() + 0.5)


@_export
class Quant(Primitive):
    """y = clamp(round(x * scale + offset), -128, 127) as int8."""

    @prim_attr_register
    def __init__(self, scale, offset, sqrt_mode=False, round_mode="Round", dst_type=torch.int8):
        pass

    def _run(self, x):
        s = self.scale * self.scale if self.sqrt_mode else self.scale
        v = x.float() * s + self.offset
        v = {"Round": _round_half_away, "Floor": torch.floor, "Ceil": torch.ceil, "Trunc": torch.trunc}[self.round_mode](v)
        return v.clamp(-128, 127).to(torch.int8)


@_export
class QuantV2(Primitive):
    def __init__(self):
        super().__init__("QuantV2")

    def _run(self, x, scale, offset, sqrt_mode=False, rounding_mode="ROUND", dst_type=torch.int8):
        s = scale * scale if sqrt_mode else scale
        return _round_half_away(x.float() * s + offset).clamp(-128, 127).to(torch.int8)


@_export
class Dequant(Primitive):
    @prim_attr_register
    def __init__(self, sqrt_mode=False, relu_flag=False, dtype=torch.float16):
        pass

    def _run(self, x, deq_scale):
        s = deq_scale.float()
        y = x.float() * (s * s if self.sqrt_mode else s)
        return (F.relu(y) if self.relu_flag else y).to(self.dtype)


@_export
class AntiQuant(Primitive):
    """y = (x + offset) * scale, int8 -> float."""

    @prim_attr_register
    def __init__(self, scale, offset, sqrt_mode=False, dtype=torch.float16):
        pass

    def _run(self, x):
        s = self.scale * self.scale if self.sqrt_mode else self.scale
        return ((x.float() + self.offset) * s).to(self.dtype)


@_export
class DynamicQuantExt(Primitive):
    """Per-token symmetric int8 quantisation: (x, smooth_scales=None) -> (int8 x, fp32 scale per row)."""

    def __init__(self):
        super().__init__("DynamicQuantExt")

    def _run(self, x, smooth_scales=None):
        xf = x.float() * (smooth_scales.float() if smooth_scales is not None else 1.0)
        scale = xf.abs().amax(-1, keepdim=True).clamp_min(1e-12) / 127.0
        return _round_half_away(xf / scale).clamp(-128, 127).to(torch.int8), scale.squeeze(-1)


def _fake_quant(x, lo, hi, num_bits, symmetric, narrow_range, channel_axis=None):
    qmin = (1 if narrow_range else 0)
    qmax = 2 ** num_bits - 1
    if symmetric:
        m = torch.maximum(lo.abs(), hi.abs())
        lo, hi = -m, m
    lo, hi = torch.minimum(lo, torch.zeros_like(lo)), torch.maximum(hi, torch.zeros_like(hi))
    scale = ((hi - lo) / (qmax - qmin)).clamp_min(1e-12)
    zp = torch.round(qmin - lo / scale).clamp(qmin, qmax)
    if channel_axis is not None:
        shape = [1] * x.dim()
        shape[channel_axis] = -1
        scale, zp, lo, hi = (t.reshape(shape) for t in (scale, zp, lo, hi))
    q = torch.round(x / scale + zp).clamp(qmin, qmax)
    y = (q - zp) * scale
    # straight-through estimator inside [lo, hi], zero gradient outside
    inside = ((x >= (qmin - zp) * scale) & (x <= (qmax - zp) * scale)).to(x.dtype)
    return x * inside + (y - x * inside).detach()


@_export
class FakeQuantPerLayer(Primitive):
    @prim_attr_register
    def __init__(self, num_bits=8, ema=False, ema_decay=0.999, quant_delay=0, symmetric=False, narrow_range=False,
                 training=True):
        pass

    def _run(self, x, min_val, max_val):
        return _fake_quant(x, min_val.reshape(()), max_val.reshape(()), self.num_bits, self.symmetric,
                           self.narrow_range)


@_export
class FakeQuantPerChannel(Primitive):
    @prim_attr_register
    def __init__(self, num_bits=8, ema=False, ema_decay=0.999, quant_delay=0, symmetric=False, narrow_range=False,
                 training=True, channel_axis=1):
        pass

    def _run(self, x, min_val, max_val):
        return _fake_quant(x, min_val, max_val, self.num_bits, self.symmetric, self.narrow_range, self.channel_axis)


@_export
class MinMaxUpdatePerLayer(Primitive):
    @prim_attr_register
    def __init__(self, ema=False, ema_decay=0.999):
        pass

    def _run(self, x, min_val, max_val):
        lo, hi = x.min().reshape(1), x.max().reshape(1)
        if self.ema:
            lo = min_val * self.ema_decay + lo * (1 - self.ema_decay)
            hi = max_val * self.ema_decay + hi * (1 - self.ema_decay)
        return torch.minimum(lo, torch.zeros_like(lo)), torch.maximum(hi, torch.zeros_like(hi))


@_export
class MinMaxUpdatePerChannel(Primitive):
    @prim_attr_register
    def __init__(self, ema=False, ema_decay=0.999, channel_axis=1):
        pass

    def _run(self, x, min_val, max_val):
        dims = [d for d in range(x.dim()) if d != self.channel_axis % x.dim()]
        lo, hi = x.amin(dims), x.amax(dims)
        if self.ema:
            lo = min_val * self.ema_decay + lo * (1 - self.ema_decay)
            hi = max_val * self.ema_decay + hi * (1 - self.ema_decay)
        return torch.minimum(lo, torch.zeros_like(lo)), torch.maximum(hi, torch.zeros_like(hi))


@_export
class QuantBatchMatmul(Primitive):
    """int8 x int8 -> int32 accumulate, then * scale (+ offset, + bias) -> dtype."""

    @prim_attr_register
    def __init__(self, transpose_x1=False, transpose_x2=False, dtype=torch.float16):
        pass

    def _run(self, x1, x2, scale, offset=None, bias=None, pertoken_scale=None):
        a = x1.transpose(-1, -2) if self.transpose_x1 else x1
        b = x2.transpose(-1, -2) if self.transpose_x2 else x2
        acc = torch.matmul(a.double(), b.double())                # exact for int8 products at any practical K
        if bias is not None:
            acc = acc + bias.double()
        y = acc * scale.double()
        if pertoken_scale is not None:
            y = y * pertoken_scale.double().unsqueeze(-1)
        if offset is not None:
            y = y + offset.double()
        return y.to(self.dtype)


@_export
class WeightQuantBatchMatmul(Primitive):
    """x (fp16/bf16) @ dequant(weight int8/int4-in-int8): weight * antiquant_scale + antiquant_offset, optional
    grouping along K by ``antiquant_group_size``."""

    @prim_attr_register
    def __init__(self, transpose_x=False, transpose_weight=False, antiquant_group_size=0):
        pass

    def _run(self, x, weight, antiquant_scale, antiquant_offset=None, quant_scale=None, quant_offset=None, bias=None):
        w = weight.float()
        if self.transpose_weight:
            w = w.transpose(-1, -2)
        sc = antiquant_scale.float()
        off = antiquant_offset.float() if antiquant_offset is not None else None
        g = self.antiquant_group_size
        if g and sc.dim() == 2 and sc.shape[0] * g == w.shape[-2]:
            sc = sc.repeat_interleave(g, 0)
            off = off.repeat_interleave(g, 0) if off is not None else None
        w = (w + off) * sc if off is not None else w * sc
        a = x.transpose(-1, -2) if self.transpose_x else x
        y = torch.matmul(a.float(), w)
        if bias is not None:
            y = y + bias.float()
        return y.to(x.dtype)


# ------------------------------------------------------------------------------------------------ transformer blocks
_ACT = {"relu": F.relu, "gelu": F.gelu, "fastgelu": lambda x: x * torch.sigmoid(1.702 * x), "silu": F.silu,
        "swiglu": None, "geglu": None, "reglu": None}


@_export
class FFN(Primitive):
    """y = act(x @ w1 + b1) @ w2 + b2; gated activations split w1's output in halves (value, gate)."""

    @prim_attr_register
    def __init__(self, activation="gelu", inner_precise=0):
        pass

    def _run(self, x, w1, w2, expert_tokens=None, bias1=None, bias2=None, *unused):
        h = torch.matmul(x, w1)
        if bias1 is not None:
            h = h + bias1
        act = self.activation.lower()
        if act in ("swiglu", "geglu", "reglu"):
            a, g = h.chunk(2, -1)
            h = a * {"swiglu": F.silu, "geglu": F.gelu, "reglu": F.relu}[act](g)
        else:
            h = _ACT[act](h)
        y = torch.matmul(h, w2)
        return y + bias2 if bias2 is not None else y


FFNExt = type("FFNExt", (FFN,), {"__doc__": FFN.__doc__})
__all__.append("FFNExt")


@_export
class GroupedMatmul(Primitive):
    """Per-group x_i @ w_i.  split_item 0: lists in, lists out; 3: one x [M, K] whose rows are cut by the cumulative
    ``group_list`` and one stacked weight [G, K, N] -> one y [M, N]."""

    @prim_attr_register
    def __init__(self, split_item=0, group_type=-1, transpose_a=False, transpose_b=False):
        pass

    def _run(self, x, weight, bias=None, scale=None, offset=None, antiquant_scale=None, antiquant_offset=None,
             group_list=None):
        def mm(a, b, i):
            a = a.transpose(-1, -2) if self.transpose_a else a
            b = b.transpose(-1, -2) if self.transpose_b else b
            y = torch.matmul(a, b)
            if bias is not None:
                y = y + (bias[i] if isinstance(bias, (list, tuple)) or bias.dim() > 1 else bias)
            return y
        if isinstance(x, (list, tuple)) and len(x) > 1:
            return [mm(a, w, i) for i, (a, w) in enumerate(zip(x, weight))]
        xs = x[0] if isinstance(x, (list, tuple)) else x
        ws = weight[0] if isinstance(weight, (list, tuple)) else weight
        ends = [int(v) for v in (group_list.tolist() if isinstance(group_list, torch.Tensor) else group_list)]
        out = xs.new_empty(xs.shape[0], ws.shape[-2] if self.transpose_b else ws.shape[-1])
        start = 0
        for g, end in enumerate(ends):
            if end > start:
                out[start:end] = mm(xs[start:end], ws[g], g)
            start = end
        return [out] if isinstance(x, (list, tuple)) else out


@_export
class MoeFinalizeRouting(Primitive):
    """out[t] = skip1[t] + skip2[t] + sum_k scales[t, k] * (expanded_x[expanded_row_idx[k * T + t]] + bias[expert[t, k]])."""

    def __init__(self):
        super().__init__("MoeFinalizeRouting")

    def _run(self, expanded_x, skip1, skip2, bias, scales, expanded_row_idx, expanded_expert_idx):
        T, Kk = scales.shape
        out = skip1.clone() if skip1 is not None else torch.zeros(T, expanded_x.shape[-1], dtype=expanded_x.dtype,
                                                                   device=expanded_x.device)
        if skip2 is not None:
            out = out + skip2
        for k in range(Kk):
            rows = expanded_x[expanded_row_idx[k * T:(k + 1) * T].long()]
            if bias is not None:
                rows = rows + bias[expanded_expert_idx[:, k].long()]
            out = out + scales[:, k:k + 1].to(rows.dtype) * rows
        return out


@_export
class GenerateEodMask(Primitive):
    """Positions / masks reset at every end-of-document token (1 where ``x == eod_token_id``)."""

    @prim_attr_register
    def __init__(self, eod_token_id=0):
        pass

    def _run(self, x):
        is_eod = x == self.eod_token_id
        seg = torch.cumsum(is_eod.long(), -1) - is_eod.long()               # document index of every token
        pos = torch.arange(x.shape[-1], device=x.device).expand_as(x)
        start = torch.zeros_like(pos)
        first = torch.ones_like(is_eod)
        first[..., 1:] = is_eod[..., :-1]
        start = torch.cummax(torch.where(first, pos, torch.zeros_like(pos)), -1).values
        same_doc = seg[..., :, None] == seg[..., None, :]
        causal = torch.tril(torch.ones(x.shape[-1], x.shape[-1], dtype=torch.bool, device=x.device))
        return pos - start, ~(same_doc & causal)


# ------------------------------------------------------------------------------------------------ inference: KV cache
@_export
class KVCacheMgr(Primitive):
    """past[b, :, index[b], :] = cur[b, :, 0, :] (decode step) - in place on ``past``."""

    def __init__(self):
        super().__init__("KVCacheMgr")

    def _run(self, past, cur, index):
        with torch.no_grad():
            b = torch.arange(past.shape[0], device=past.device)
            past[b, :, index.long().reshape(-1), :] = cur[:, :, 0, :].to(past.dtype)
        return past


@_export
class KVCacheScatterUpdate(Primitive):
    def __init__(self):
        super().__init__("KVCacheScatterUpdate")

    def _run(self, var, indices, updates, axis=-2, reduce="none"):
        ax = axis % var.dim()
        with torch.no_grad():
            for b in range(var.shape[0]):
                start = int(indices.reshape(-1)[b])
                sl = [b] + [slice(None)] * (var.dim() - 1)
                sl[ax] = slice(start, start + updates.shape[ax])
                if reduce == "add":
                    var[tuple(sl)] += updates[b].to(var.dtype)
                else:
                    var[tuple(sl)] = updates[b].to(var.dtype)
        return var


@_export
class DecoderKVCache(Primitive):
    """cache[b, ..., valid_seq_len[b], :] = update[b, ..., 0, :] for a one-token decode step."""

    def __init__(self):
        super().__init__("DecoderKVCache")

    def _run(self, cache, update, valid_seq_len, batch_index=None, seq_len_axis=2, new_max_seq_len=None,
             cur_max_seq_len=None):
        ax = int(seq_len_axis if not isinstance(seq_len_axis, torch.Tensor) else seq_len_axis.reshape(-1)[0])
        with torch.no_grad():
            for b in range(cache.shape[0]):
                sl = [b] + [slice(None)] * (cache.dim() - 1)
                pos = int(valid_seq_len.reshape(-1)[b])
                sl[ax] = slice(pos, pos + update.shape[ax])
                cache[tuple(sl)] = update[b].to(cache.dtype)
        return cache


@_export
class PromptKVCache(Primitive):
    """cache[batch_index[b], ..., :S, :] = update[b] (prefill), zero padded beyond ``valid_seq_len``."""

    def __init__(self):
        super().__init__("PromptKVCache")

    def _run(self, cache, update, valid_seq_len, batch_index, seq_len_axis=2, new_max_seq_len=None,
             cur_max_seq_len=None):
        ax = int(seq_len_axis if not isinstance(seq_len_axis, torch.Tensor) else seq_len_axis.reshape(-1)[0])
        with torch.no_grad():
            for b in range(update.shape[0]):
                dst = int(batch_index.reshape(-1)[b])
                if dst < 0:
                    continue
                sl = [dst] + [slice(None)] * (cache.dim() - 1)
                sl[ax] = slice(0, update.shape[ax])
                cache[tuple(sl)] = update[b].to(cache.dtype)
        return cache


@_export
class ReshapeAndCache(Primitive):
    """Writes this step's keys / values [T, heads * D] into the paged caches [blocks, block_size, heads, D] at
    ``slot_mapping`` (slot = block * block_size + offset)."""

    def __init__(self):
        super().__init__("ReshapeAndCache")

    def _run(self, key, value, key_cache, value_cache, slot_mapping):
        nb, bs, h, d = key_cache.shape
        slots = slot_mapping.reshape(-1).long()
        ok = slots >= 0
        with torch.no_grad():
            key_cache.view(nb * bs, h, d)[slots[ok]] = key.reshape(-1, h, d)[ok].to(key_cache.dtype)
            value_cache.view(nb * bs, h, d)[slots[ok]] = value.reshape(-1, h, d)[ok].to(value_cache.dtype)
        return key


def _gather_pages(cache, table, length):
    """[blocks, block_size, kvh, D] + block table row -> [length, kvh, D]."""
    bs = cache.shape[1]
    n = (length + bs - 1) // bs
    return cache[table[:n].long()].reshape(n * bs, cache.shape[2], cache.shape[3])[:length]


@_export
class PagedAttention(Primitive):
    """Decode attention over paged KV caches: query [B, 1 or S_q, heads * D], caches [blocks, block_size, kv_heads,
    D], block_tables [B, max_blocks], context_lens [B] -> [B, S_q, heads * D]."""

    @prim_attr_register
    def __init__(self, head_num, scale_value=1.0, kv_head_num=0):
        pass

    def _run(self, query, key_cache, value_cache, block_tables, context_lens, antiquant_scale=None,
             antiquant_offset=None, attn_mask=None):
        B, Sq, HD = query.shape
        H = self.head_num
        D = HD // H
        kvh = key_cache.shape[2]
        out = torch.empty_like(query)
        for b in range(B):
            L = int(context_lens[b])
            k = _gather_pages(key_cache, block_tables[b], L).float()          # [L, kvh, D]
            v = _gather_pages(value_cache, block_tables[b], L).float()
            if kvh != H:
                k, v = k.repeat_interleave(H // kvh, 1), v.repeat_interleave(H // kvh, 1)
            q = query[b].reshape(Sq, H, D).float()
            s = torch.einsum("qhd,khd->hqk", q, k) * self.scale_value
            if attn_mask is not None:
                m = attn_mask[b] if attn_mask.dim() == 3 else attn_mask
                s = s + m[..., :Sq, :L].float() * -1e4 if m.dtype != torch.bool else s.masked_fill(m[..., :Sq, :L], -1e30)
            elif Sq > 1:                                                       # causal inside the new tokens
                qpos = torch.arange(L - Sq, L, device=s.device)[:, None]
                s = s.masked_fill(torch.arange(L, device=s.device)[None] > qpos, float("-inf"))
            out[b] = torch.einsum("hqk,khd->qhd", torch.softmax(s, -1), v).reshape(Sq, HD).to(query.dtype)
        return out


PagedAttentionMask = type("PagedAttentionMask", (PagedAttention,), {
    "__doc__": "PagedAttention with an additive alibi-style mask as the extra input.",
    "_run": lambda self, query, key_cache, value_cache, block_tables, context_lens, alibi_mask=None, *a:
        PagedAttention._run(self, query, key_cache, value_cache, block_tables, context_lens, None, None, None)
        if alibi_mask is None else _paged_with_bias(self, query, key_cache, value_cache, block_tables, context_lens,
                                                    alibi_mask)})
__all__.append("PagedAttentionMask")


def _paged_with_bias(self, query, key_cache, value_cache, block_tables, context_lens, bias):
    B, Sq, HD = query.shape
    H = self.head_num
    D = HD // H
    kvh = key_cache.shape[2]
    out = torch.empty_like(query)
    for b in range(B):
        L = int(context_lens[b])
        k = _gather_pages(key_cache, block_tables[b], L).float()
        v = _gather_pages(value_cache, block_tables[b], L).float()
        if kvh != H:
            k, v = k.repeat_interleave(H // kvh, 1), v.repeat_interleave(H // kvh, 1)
        q = query[b].reshape(Sq, H, D).float()
        s = torch.einsum("qhd,khd->hqk", q, k) * self.scale_value + bias[b, :, :Sq, :L].float()
        out[b] = torch.einsum("hqk,khd->qhd", torch.softmax(s, -1), v).reshape(Sq, HD).to(query.dtype)
    return out


def _dense_attention(q, k, v, scale, mask=None, causal=False, actual_kv=None):
    """q [B, H, Sq, D], k / v [B, KVH, Skv, D] -> [B, H, Sq, D] in fp32 math."""
    H, KVH = q.shape[1], k.shape[1]
    if H != KVH:
        k, v = k.repeat_interleave(H // KVH, 1), v.repeat_interleave(H // KVH, 1)
    s = torch.matmul(q.float(), k.float().transpose(-1, -2)) * scale
    Sq, Skv = s.shape[-2:]
    if causal:
        qpos = torch.arange(Skv - Sq, Skv, device=s.device)[:, None]
        s = s.masked_fill(torch.arange(Skv, device=s.device)[None] > qpos, float("-inf"))
    if mask is not None:
        m = mask
        while m.dim() < 4:
            m = m.unsqueeze(0 if m.dim() == 2 else 1)
        s = s.masked_fill(m.bool()[..., :Sq, :Skv], float("-inf"))
    if actual_kv is not None:
        lens = torch.as_tensor(actual_kv, device=s.device).reshape(-1, 1, 1, 1)
        s = s.masked_fill(torch.arange(Skv, device=s.device).reshape(1, 1, 1, -1) >= lens, float("-inf"))
    return torch.matmul(torch.softmax(s, -1), v.float())


def _to_bnsd(t, layout, heads):
    if layout == "BSH":
        B, S, Hd = t.shape
        return t.reshape(B, S, heads, Hd // heads).permute(0, 2, 1, 3)
    if layout == "BSND":
        return t.permute(0, 2, 1, 3)
    return t


def _from_bnsd(t, layout):
    if layout == "BSH":
        B, N, S, D = t.shape
        return t.permute(0, 2, 1, 3).reshape(B, S, N * D)
    if layout == "BSND":
        return t.permute(0, 2, 1, 3)
    return t


@_export
class PromptFlashAttention(Primitive):
    """Prefill attention (full prompt): inputs in BSH / BNSD / BSND, optional mask (True = masked), GQA through
    ``num_key_value_heads``; causal when ``sparse_mode`` is 2 or 3 or ``next_tokens`` is 0."""

    @prim_attr_register
    def __init__(self, num_heads, scale_value=1.0, pre_tokens=2147483647, next_tokens=0, input_layout="BSH",
                 num_key_value_heads=0, sparse_mode=0, inner_precise=1):
        pass

    def _run(self, query, key, value, attn_mask=None, actual_seq_lengths=None, actual_seq_lengths_kv=None,
             pse_shift=None, *unused):
        kvh = self.num_key_value_heads or self.num_heads
        q = _to_bnsd(query, self.input_layout, self.num_heads)
        k = _to_bnsd(key, self.input_layout, kvh)
        v = _to_bnsd(value, self.input_layout, kvh)
        causal = attn_mask is None and (self.sparse_mode in (2, 3) or self.next_tokens == 0)
        if causal and q.dtype == torch.bfloat16 and q.is_cuda and q.shape[-1] == 128 and actual_seq_lengths_kv is None:
            o = fused.flash_attention(q.permute(0, 2, 1, 3).contiguous(), k.permute(0, 2, 1, 3).contiguous(),
                                      v.permute(0, 2, 1, 3).contiguous(), True, self.scale_value).permute(0, 2, 1, 3)
        else:
            o = _dense_attention(q, k, v, self.scale_value, attn_mask, causal, actual_seq_lengths_kv).to(query.dtype)
        return _from_bnsd(o, self.input_layout)


@_export
class IncreFlashAttention(Primitive):
    """Decode attention: one query token per sequence against the whole (dense) KV cache; ``actual_seq_lengths``
    gives the valid cache length per batch entry."""

    @prim_attr_register
    def __init__(self, num_heads, input_layout="BSH", scale_value=1.0, num_key_value_heads=0, block_size=0,
                 inner_precise=1):
        pass

    def _run(self, query, key, value, attn_mask=None, actual_seq_lengths=None, pse_shift=None, *unused):
        kvh = self.num_key_value_heads or self.num_heads
        key = key[0] if isinstance(key, (list, tuple)) else key
        value = value[0] if isinstance(value, (list, tuple)) else value
        q = _to_bnsd(query, self.input_layout, self.num_heads)
        k = _to_bnsd(key, self.input_layout, kvh)
        v = _to_bnsd(value, self.input_layout, kvh)
        o = _dense_attention(q, k, v, self.scale_value, attn_mask, False, actual_seq_lengths).to(query.dtype)
        return _from_bnsd(o, self.input_layout)


@_export
class FusedInferAttentionScore(Primitive):
    """One entry point for prefill (S_q > 1) and decode (S_q = 1); returns (attention_out, softmax_lse)."""

    @prim_attr_register
    def __init__(self, num_heads, scale_value=1.0, pre_tokens=2147483647, next_tokens=2147483647, input_layout="BSH",
                 num_key_value_heads=0, sparse_mode=0, inner_precise=1, block_size=0, antiquant_mode=0,
                 softmax_lse_flag=False):
        pass

    def _run(self, query, key, value, pse_shift=None, attn_mask=None, actual_seq_lengths=None,
             actual_seq_lengths_kv=None, *unused):
        kvh = self.num_key_value_heads or self.num_heads
        key = key[0] if isinstance(key, (list, tuple)) else key
        value = value[0] if isinstance(value, (list, tuple)) else value
        q = _to_bnsd(query, self.input_layout, self.num_heads)
        k = _to_bnsd(key, self.input_layout, kvh)
        v = _to_bnsd(value, self.input_layout, kvh)
        causal = attn_mask is None and q.shape[2] > 1 and (self.sparse_mode in (2, 3) or self.next_tokens == 0)
        o = _dense_attention(q, k, v, self.scale_value, attn_mask, causal, actual_seq_lengths_kv).to(query.dtype)
        lse = torch.zeros(q.shape[0], q.shape[1], q.shape[2], 1, device=q.device)
        if self.softmax_lse_flag:
            kk = k.repeat_interleave(q.shape[1] // k.shape[1], 1) if k.shape[1] != q.shape[1] else k
            lse = torch.logsumexp(torch.matmul(q.float(), kk.float().transpose(-1, -2)) * self.scale_value, -1,
                                  keepdim=True)
        return _from_bnsd(o, self.input_layout), lse


@_export
class WKV(Primitive):
    """RWKV-4 time mixing: out[t] = (sum_{i<t} e^{-(t-1-i) w + k_i} v_i + e^{u + k_t} v_t) / (same with v = 1), computed
    with the running-maximum recurrence; returns (out, state a, state b, state p)."""

    def __init__(self):
        super().__init__("WKV")

    def _run(self, w, u, k, v, sp, sq, sm):
        B, T, C = k.shape
        w = -torch.exp(w.float())
        u, k, v = u.float(), k.float(), v.float()
        p, q, o = sp.float().clone(), sq.float().clone(), sm.float().clone()
        out = torch.empty(B, T, C, device=k.device)
        for t in range(T):
            kt, vt = k[:, t], v[:, t]
            no = torch.maximum(o, u + kt)
            A, Bc = torch.exp(o - no), torch.exp(u + kt - no)
            out[:, t] = (A * p + Bc * vt) / (A * q + Bc)
            no = torch.maximum(w + o, kt)
            A, Bc = torch.exp(w + o - no), torch.exp(kt - no)
            p, q, o = A * p + Bc * vt, A * q + Bc, no
        return out.to(sp.dtype), p, q, o


# ------------------------------------------------------------------------------------------------ parallel placeholders
def _identity_prim(name, doc):
    def __init__(self, *args, **kwargs):
        Primitive.__init__(self, name)
        for k, v in kwargs.items():
            self.add_prim_attr(k, v)

    def _run(self, *xs):
        return xs[0] if len(xs) == 1 else xs

    cls = type(name, (Primitive,), {"__init__": __init__, "_run": _run, "__doc__": doc})
    globals()[name] = cls
    __all__.append(name)


_identity_prim("AShardIdentity", "Identity whose only purpose is to carry a sharding strategy (layout change point).")
_identity_prim("BatchParallel", "Identity marking an op that may only be split along the batch dim.")
_identity_prim("StandAlone", "Identity marking an op that must run un-split on every device.")
_identity_prim("SelfDefineShard", "Identity carrying a user-defined layout pair (Custom-op sharding hook).")
_identity_prim("VirtualDataset", "Marks the dataset outputs: their layout is the dataset strategy.")
_identity_prim("VirtualOutput", "Marks the network outputs for layout inference.")


@_export
class GetNext(Primitive):
    """Pops the next element of the dataset queue named ``shared_name`` (``dataset_helper`` registers queues)."""

    _queues = {}

    @prim_attr_register
    def __init__(self, types=None, shapes=None, output_num=1, shared_name=""):
        pass

    def _run(self):
        it = self._queues.get(self.shared_name)
        if it is None:
            raise RuntimeError("GetNext: no dataset queue named %r has been registered" % self.shared_name)
        item = next(it)
        return tuple(item) if isinstance(item, (list, tuple)) else (item,)


@_export
class Custom(Primitive):
    """User-defined operator: ``func`` is a Python callable on tensors (func_type "pyfunc" / "hybrid"); ``bprop``
    optionally supplies the gradient (python/mindspore/ops/operations/custom_ops.py ``Custom``).  Compiled
    ``aot`` entries are loaded with ``ctypes`` from ``"path.so:symbol"`` and called with raw pointers:
    int fn(int nparam, void** params, int* ndims, int64_t** shapes, const char** dtypes, void* stream, void* extra)."""

    def __init__(self, func, out_shape=None, out_dtype=None, func_type="pyfunc", bprop=None, reg_info=None):
        super().__init__("Custom")
        self.func, self.out_shape, self.out_dtype, self.func_type, self.bprop = func, out_shape, out_dtype, func_type, bprop
        self._aot = None
        if func_type == "aot":
            import ctypes
            path, sym = func.rsplit(":", 1)
            self._aot = getattr(ctypes.CDLL(path), sym)
            self._aot.restype = ctypes.c_int

    def _run(self, *xs):
        if self._aot is None:
            if self.bprop is None:
                return self.func(*xs)
            outer = self

            class _Fn(torch.autograd.Function):
                @staticmethod
                def forward(ctx, *a):
                    ctx.save_for_backward(*a)
                    with torch.no_grad():
                        out = outer.func(*a)
                    ctx.out = out
                    return out

                @staticmethod
                def backward(ctx, dout):
                    g = outer.bprop(*ctx.saved_tensors, ctx.out, dout)
                    return tuple(g) if isinstance(g, (list, tuple)) else (g,)
            return _Fn.apply(*xs)
        import ctypes
        shapes = self.out_shape(*[tuple(x.shape) for x in xs]) if callable(self.out_shape) else self.out_shape
        dtypes = self.out_dtype(*[x.dtype for x in xs]) if callable(self.out_dtype) else self.out_dtype
        single = not isinstance(shapes[0], (list, tuple))
        shapes = [shapes] if single else list(shapes)
        dtypes = [dtypes] * len(shapes) if not isinstance(dtypes, (list, tuple)) else list(dtypes)
        outs = [torch.empty(tuple(s), dtype=d, device=xs[0].device) for s, d in zip(shapes, dtypes)]
        ts = [x.contiguous() for x in xs] + outs
        n = len(ts)
        params = (ctypes.c_void_p * n)(*[t.data_ptr() for t in ts])
        ndims = (ctypes.c_int * n)(*[t.dim() for t in ts])
        shp = [(ctypes.c_int64 * max(t.dim(), 1))(*t.shape) for t in ts]
        shp_ptrs = (ctypes.POINTER(ctypes.c_int64) * n)(*[ctypes.cast(s, ctypes.POINTER(ctypes.c_int64)) for s in shp])
        names = (ctypes.c_char_p * n)(*[str(t.dtype).replace("torch.", "").encode() for t in ts])
        stream = torch.cuda.current_stream().cuda_stream if ts[0].is_cuda else 0
        rc = self._aot(n, params, ndims, shp_ptrs, names, ctypes.c_void_p(stream), None)
        if rc != 0:
            raise RuntimeError("Custom aot function %s returned %d" % (self.func, rc))
        return outs[0] if single else tuple(outs)


@_export
class DropoutGenMask(Primitive):
    """Bit-packed keep mask (uint8, 8 elements per byte, padded to a multiple of 128 bits) for ``shape``."""

    @prim_attr_register
    def __init__(self, Seed0=0, Seed1=0):
        pass

    def _run(self, shape, keep_prob):
        n = 1
        for d in shape:
            n *= int(d)
        padded = (n + 127) // 128 * 128
        kp = float(keep_prob)
        bits = (torch.rand(padded) < kp).to(torch.uint8).reshape(-1, 8)
        weights = torch.tensor([1, 2, 4, 8, 16, 32, 64, 128], dtype=torch.uint8)
        return (bits * weights).sum(1).to(torch.uint8)


@_export
class DropoutDoMask(Primitive):
    """y = x * mask / keep_prob with the bit-packed mask of ``DropoutGenMask``."""

    def __init__(self):
        super().__init__("DropoutDoMask")

    def _run(self, x, mask, keep_prob):
        kp = float(keep_prob)
        m = mask.to(x.device).reshape(-1, 1)
        bits = ((m >> torch.arange(8, device=x.device, dtype=torch.uint8)) & 1).reshape(-1)[:x.numel()]
        return x * bits.reshape(x.shape).to(x.dtype) / kp
