"""Primitive operator classes (``mindspore.ops.operations`` / ``ops.<Name>()``).

Names and constructor attributes follow the reference so that shard strategies, the OperatorInfo
registry of the parallel planner and user code keyed on primitive names keep working.  Execution
is a torch call, or - for the hot ops on CUDA bf16 tensors - one of the sm_100a kernels through
``ops.fused``.

Parity: mindspore/python/mindspore/ops/operations/{math_ops,array_ops,nn_ops,other_ops}.py and the
yaml op definitions under mindspore/core/ops/ops_def/.
"""
from __future__ import annotations

import math
import numbers

import numpy as np
import torch
import torch.nn.functional as F

from ..common import dtype as mstype
from ..common.tensor import Tensor
from . import fused
from .primitive import Primitive, PrimitiveWithInfer, prim_attr_register


def _t(x, like=None):
    """Scalar / numpy -> tensor on the device (and float dtype) of ``like``."""
    if isinstance(x, torch.Tensor):
        return x
    if like is not None and isinstance(like, torch.Tensor):
        if isinstance(x, (bool, np.bool_)):
            return torch.tensor(bool(x), device=like.device)
        if isinstance(x, numbers.Integral):
            return torch.tensor(int(x), device=like.device,
                                dtype=like.dtype if like.dtype != torch.bool else torch.int64)
        if isinstance(x, numbers.Real):
            return torch.tensor(float(x), device=like.device,
                                dtype=like.dtype if like.is_floating_point() else torch.float32)
    return torch.as_tensor(x)


def _axis(a):
    if isinstance(a, torch.Tensor):
        a = a.tolist()
    if isinstance(a, list):
        a = tuple(a)
    return a


def _make_unary(name, fn):
    def __init__(self):
        Primitive.__init__(self, name)

    def _run(self, x):
        return fn(x)

    return type(name, (Primitive,), {"__init__": __init__, "_run": _run, "__doc__": "Elementwise %s." % name})


def _make_binary(name, fn):
    def __init__(self):
        Primitive.__init__(self, name)

    def _run(self, x, y):
        if not isinstance(x, torch.Tensor):
            x = _t(x, y)
        elif not isinstance(y, torch.Tensor):
            y = _t(y, x)
        return fn(x, y)

    return type(name, (Primitive,), {"__init__": __init__, "_run": _run, "__doc__": "Broadcasting %s." % name})


_UNARY = {
    "Abs": torch.abs, "Neg": torch.neg, "Exp": torch.exp, "Expm1": torch.expm1, "Log": torch.log,
    "Log1p": torch.log1p, "Sqrt": torch.sqrt, "Rsqrt": torch.rsqrt, "Square": torch.square, "Sign": torch.sign,
    "Sin": torch.sin, "Cos": torch.cos, "Tan": torch.tan, "Asin": torch.asin, "ACos": torch.acos,
    "Atan": torch.atan, "Sinh": torch.sinh, "Cosh": torch.cosh, "Tanh": torch.tanh, "Asinh": torch.asinh,
    "Acosh": torch.acosh, "Atanh": torch.atanh, "Erf": torch.erf, "Erfc": torch.erfc, "Erfinv": torch.erfinv,
    "Floor": torch.floor, "Ceil": torch.ceil, "Round": torch.round, "Trunc": torch.trunc, "Rint": torch.round,
    "Reciprocal": torch.reciprocal, "Inv": torch.reciprocal, "Invert": torch.bitwise_not,
    "LogicalNot": torch.logical_not, "IsNan": torch.isnan, "IsInf": torch.isinf, "IsFinite": torch.isfinite,
    "Sigmoid": torch.sigmoid, "ReLU": torch.relu, "ReLU6": F.relu6, "SiLU": F.silu, "Mish": F.mish,
    "Softplus": F.softplus, "Softsign": F.softsign, "HSigmoid": F.hardsigmoid, "HSwish": F.hardswish,
    "SeLU": F.selu, "Lgamma": torch.lgamma, "Digamma": torch.digamma, "OnesLike": torch.ones_like,
    "ZerosLike": torch.zeros_like, "Identity": lambda x: x + 0 if isinstance(x, torch.Tensor) else x,
    "StopGradient": lambda x: x.detach(), "Conj": torch.conj, "Real": torch.real, "Imag": torch.imag,
    "BesselI0": torch.special.i0, "BesselI0e": torch.special.i0e, "BesselI1": torch.special.i1,
    "BesselI1e": torch.special.i1e, "Sinc": torch.sinc, "Logit": torch.logit, "FastGeLU": fused.gelu_tanh,
    "Angle": torch.angle, "PopulationCount": lambda x: torch.tensor(
        np.vectorize(lambda v: bin(int(v) & 0xFFFFFFFFFFFFFFFF).count("1"))(x.cpu().numpy()), device=x.device),
}

_BINARY = {
    "Add": torch.add, "Sub": torch.sub, "Mul": torch.mul, "Div": torch.div, "RealDiv": torch.true_divide,
    "FloorDiv": torch.floor_divide, "FloorMod": torch.remainder, "Mod": torch.fmod, "Pow": torch.pow,
    "Maximum": torch.maximum, "Minimum": torch.minimum, "Equal": torch.eq, "NotEqual": torch.ne,
    "Greater": torch.gt, "GreaterEqual": torch.ge, "Less": torch.lt, "LessEqual": torch.le,
    "LogicalAnd": torch.logical_and, "LogicalOr": torch.logical_or, "LogicalXor": torch.logical_xor,
    "BitwiseAnd": torch.bitwise_and, "BitwiseOr": torch.bitwise_or, "BitwiseXor": torch.bitwise_xor,
    "Atan2": torch.atan2, "SquaredDifference": lambda x, y: (x - y) ** 2, "Xdivy": lambda x, y: torch.where(
        x == 0, torch.zeros_like(x), x / y), "Xlogy": torch.xlogy, "TruncateDiv": lambda x, y: torch.div(
        x, y, rounding_mode="trunc"), "TruncateMod": torch.fmod, "DivNoNan": lambda x, y: torch.where(
        y == 0, torch.zeros_like(x), x / y), "MulNoNan": lambda x, y: torch.where(y == 0, torch.zeros_like(x), x * y),
    "Hypot": torch.hypot, "Gcd": torch.gcd, "Lcm": torch.lcm, "NextAfter": torch.nextafter,
    "LeftShift": torch.bitwise_left_shift, "RightShift": torch.bitwise_right_shift, "Heaviside": torch.heaviside,
    "ApproximateEqual": lambda x, y: (x - y).abs() < 1e-5, "Igamma": torch.special.gammainc,
    "Igammac": torch.special.gammaincc, "Zeta": torch.special.zeta,
}

for _n, _f in _UNARY.items():
    globals()[_n] = _make_unary(_n, _f)
for _n, _f in _BINARY.items():
    globals()[_n] = _make_binary(_n, _f)
TensorAdd = globals()["Add"]


# ------------------------------------------------------------------------------------ math with attrs
class AddN(Primitive):
    def __init__(self):
        super().__init__("AddN")

    def _run(self, xs):
        out = xs[0]
        for x in xs[1:]:
            out = out + x
        return out


class Cast(Primitive):
    def __init__(self):
        super().__init__("Cast")

    def _run(self, x, dtype):
        if not isinstance(x, torch.Tensor):
            return Tensor(x, dtype=dtype)
        return x.to(dtype)


class MatMul(Primitive):
    @prim_attr_register
    def __init__(self, transpose_a=False, transpose_b=False):
        self.init_prim_io_names(["x1", "x2"], ["output"])

    def _run(self, a, b):
        return fused.matmul(a, b, self.transpose_a, self.transpose_b)


class BatchMatMul(MatMul):
    def _run(self, a, b):
        if a.dim() == b.dim():
            return fused.matmul(a, b, self.transpose_a, self.transpose_b) if a.dim() in (2, 3) else torch.matmul(
                a.transpose(-1, -2) if self.transpose_a else a, b.transpose(-1, -2) if self.transpose_b else b)
        return torch.matmul(a.transpose(-1, -2) if self.transpose_a else a,
                            b.transpose(-1, -2) if self.transpose_b else b)


class MatMulExt(Primitive):
    def __init__(self):
        super().__init__("MatMulExt")

    def _run(self, a, b):
        return torch.matmul(a, b)


class BiasAdd(Primitive):
    @prim_attr_register
    def __init__(self, data_format="NCHW"):
        pass

    def _run(self, x, b):
        if x.dim() > 2 and self.data_format == "NCHW":
            return x + b.reshape((1, -1) + (1,) * (x.dim() - 2))
        return x + b


class _Reduce(Primitive):
    _fn = None

    @prim_attr_register
    def __init__(self, keep_dims=False):
        pass

    def _run(self, x, axis=()):
        axis = _axis(axis)
        fn = type(self)._fn
        if axis is None or axis == ():
            out = fn(x)
            return out.reshape((1,) * x.dim()) if self.keep_dims else out
        return fn(x, dim=axis, keepdim=self.keep_dims)


class ReduceSum(_Reduce):
    _fn = staticmethod(torch.sum)

    @prim_attr_register
    def __init__(self, keep_dims=False, skip_mode=False):
        pass


class ReduceMean(_Reduce):
    _fn = staticmethod(torch.mean)


class ReduceMax(_Reduce):
    _fn = staticmethod(torch.amax)


class ReduceMin(_Reduce):
    _fn = staticmethod(torch.amin)


class ReduceAll(_Reduce):
    _fn = staticmethod(torch.all)


class ReduceAny(_Reduce):
    _fn = staticmethod(torch.any)


class ReduceProd(_Reduce):
    def _run(self, x, axis=()):
        axis = _axis(axis)
        if axis is None or axis == ():
            return torch.prod(x)
        if isinstance(axis, int):
            return torch.prod(x, dim=axis, keepdim=self.keep_dims)
        out = x
        for a in sorted(axis, reverse=True):
            out = torch.prod(out, dim=a, keepdim=self.keep_dims)
        return out


class CumSum(Primitive):
    @prim_attr_register
    def __init__(self, exclusive=False, reverse=False):
        pass

    def _run(self, x, axis):
        if self.reverse:
            x = torch.flip(x, (axis,))
        out = torch.cumsum(x, axis)
        if self.exclusive:
            out = out - x
        if self.reverse:
            out = torch.flip(out, (axis,))
        return out


class CumProd(CumSum):
    def _run(self, x, axis):
        return torch.cumprod(x, axis)


class Argmax(Primitive):
    @prim_attr_register
    def __init__(self, axis=-1, output_type=mstype.int32):
        pass

    def _run(self, x):
        return torch.argmax(x, dim=self.axis).to(self.output_type)


class Argmin(Argmax):
    def _run(self, x):
        return torch.argmin(x, dim=self.axis).to(self.output_type)


class ArgMaxWithValue(Primitive):
    @prim_attr_register
    def __init__(self, axis=0, keep_dims=False):
        pass

    def _run(self, x):
        v, i = torch.max(x, dim=self.axis, keepdim=self.keep_dims)
        return i.to(torch.int32), v


class ArgMinWithValue(ArgMaxWithValue):
    def _run(self, x):
        v, i = torch.min(x, dim=self.axis, keepdim=self.keep_dims)
        return i.to(torch.int32), v


class TopK(Primitive):
    @prim_attr_register
    def __init__(self, sorted=True):
        pass

    def _run(self, x, k):
        v, i = torch.topk(x, int(k), dim=-1, sorted=self.sorted)
        return v, i.to(torch.int32)


class Sort(Primitive):
    @prim_attr_register
    def __init__(self, axis=-1, descending=False):
        pass

    def _run(self, x):
        v, i = torch.sort(x, dim=self.axis, descending=self.descending)
        return v, i.to(torch.int32)


class Lerp(Primitive):
    def __init__(self):
        super().__init__("Lerp")

    def _run(self, s, e, w):
        return torch.lerp(s, e, _t(w, s))


class Addcmul(Primitive):
    def __init__(self):
        super().__init__("Addcmul")

    def _run(self, x, a, b, value):
        return x + value * a * b


class Addcdiv(Primitive):
    def __init__(self):
        super().__init__("Addcdiv")

    def _run(self, x, a, b, value):
        return x + value * a / b


class SquareSumAll(Primitive):
    def __init__(self):
        super().__init__("SquareSumAll")

    def _run(self, x, y):
        return (x * x).sum(), (y * y).sum()


class L2Loss(Primitive):
    def __init__(self):
        super().__init__("L2Loss")

    def _run(self, x):
        return (x.float() ** 2).sum() / 2


class L2Normalize(Primitive):
    @prim_attr_register
    def __init__(self, axis=0, epsilon=1e-4):
        pass

    def _run(self, x):
        ax = self.axis if isinstance(self.axis, int) else self.axis[0]
        return x / torch.sqrt(torch.clamp((x * x).sum(ax, keepdim=True), min=self.epsilon))


class Einsum(Primitive):
    @prim_attr_register
    def __init__(self, equation):
        pass

    def _run(self, xs):
        return torch.einsum(self.equation, *xs)


class LinSpace(Primitive):
    def __init__(self):
        super().__init__("LinSpace")

    def _run(self, start, stop, num):
        return torch.linspace(float(start), float(stop), int(num))


class Range(Primitive):
    @prim_attr_register
    def __init__(self, maxlen=1000000):
        pass

    def _run(self, start, limit, delta):
        vals = [v.item() if isinstance(v, torch.Tensor) else v for v in (start, limit, delta)]
        dt = torch.float32 if any(isinstance(v, float) for v in vals) else torch.int32
        return torch.arange(*vals, dtype=dt)


class Eye(Primitive):
    def __init__(self):
        super().__init__("Eye")

    def _run(self, n, m, t):
        return torch.eye(n, m, dtype=t)


class ClipByNorm(Primitive):
    @prim_attr_register
    def __init__(self, axis=None):
        pass

    def _run(self, x, clip_norm):
        n = torch.sqrt((x.float() ** 2).sum()) if self.axis is None else torch.sqrt(
            (x.float() ** 2).sum(self.axis, keepdim=True))
        cn = _t(clip_norm, x).float()
        return (x * (cn / torch.maximum(n, cn))).to(x.dtype)


class FloatStatus(Primitive):
    def __init__(self):
        super().__init__("FloatStatus")

    def _run(self, x):
        return (~torch.isfinite(x)).any().float().reshape(1)


class NPUAllocFloatStatus(Primitive):
    def __init__(self):
        super().__init__("NPUAllocFloatStatus")

    def _run(self):
        return torch.zeros(8)


class AllFinite(Primitive):
    def __init__(self):
        super().__init__("AllFinite")

    def _run(self, xs):
        ok = torch.tensor(True, device=xs[0].device)
        for x in xs:
            ok = ok & torch.isfinite(x).all()
        return ~ok


# ------------------------------------------------------------------------------------ array ops
class Reshape(Primitive):
    def __init__(self):
        super().__init__("Reshape")

    def _run(self, x, shape):
        return x.reshape(tuple(int(s) for s in _axis(shape)))


class Shape(Primitive):
    def __init__(self):
        super().__init__("Shape")

    def _run(self, x):
        return tuple(x.shape)


class TensorShape(Shape):
    def _run(self, x):
        return torch.tensor(tuple(x.shape), dtype=torch.int64)


DynamicShape = TensorShape


class Rank(Primitive):
    def __init__(self):
        super().__init__("Rank")

    def _run(self, x):
        return x.dim()


class Size(Primitive):
    def __init__(self):
        super().__init__("Size")

    def _run(self, x):
        return x.numel()


class DType(Primitive):
    def __init__(self):
        super().__init__("DType")

    def _run(self, x):
        return x.dtype


class Transpose(Primitive):
    def __init__(self):
        super().__init__("Transpose")

    def _run(self, x, perm):
        return x.permute(*_axis(perm))


class ExpandDims(Primitive):
    def __init__(self):
        super().__init__("ExpandDims")

    def _run(self, x, axis):
        return x.unsqueeze(axis)


class Squeeze(Primitive):
    @prim_attr_register
    def __init__(self, axis=()):
        pass

    def _run(self, x):
        if self.axis == () or self.axis is None:
            return x.squeeze()
        ax = self.axis if isinstance(self.axis, (tuple, list)) else (self.axis,)
        for a in sorted((a % x.dim() for a in ax), reverse=True):
            x = x.squeeze(a)
        return x


class Concat(Primitive):
    @prim_attr_register
    def __init__(self, axis=0):
        pass

    def _run(self, xs):
        return torch.cat(list(xs), dim=self.axis)


class Stack(Primitive):
    @prim_attr_register
    def __init__(self, axis=0):
        pass

    def _run(self, xs):
        return torch.stack(list(xs), dim=self.axis)


Pack = Stack


class Unstack(Primitive):
    @prim_attr_register
    def __init__(self, axis=0, num=None):
        pass

    def _run(self, x):
        return tuple(torch.unbind(x, dim=self.axis))


class Split(Primitive):
    @prim_attr_register
    def __init__(self, axis=0, output_num=1):
        pass

    def _run(self, x):
        return tuple(torch.chunk(x, self.output_num, dim=self.axis))


class SplitV(Primitive):
    @prim_attr_register
    def __init__(self, size_splits, split_dim, num_split):
        pass

    def _run(self, x):
        sizes = list(self.size_splits)
        if -1 in sizes:
            sizes[sizes.index(-1)] = x.shape[self.split_dim] - sum(s for s in sizes if s != -1)
        return tuple(torch.split(x, sizes, dim=self.split_dim))


class Slice(Primitive):
    def __init__(self):
        super().__init__("Slice")

    def _run(self, x, begin, size):
        idx = tuple(slice(int(b), None if int(s) == -1 else int(b) + int(s)) for b, s in zip(begin, size))
        return x[idx]


class StridedSlice(Primitive):
    @prim_attr_register
    def __init__(self, begin_mask=0, end_mask=0, ellipsis_mask=0, new_axis_mask=0, shrink_axis_mask=0):
        pass

    def _run(self, x, begin, end, strides):
        idx = []
        for i, (b, e, s) in enumerate(zip(begin, end, strides)):
            b, e, s = int(b), int(e), int(s)
            if (self.shrink_axis_mask >> i) & 1:
                idx.append(b)
                continue
            if (self.new_axis_mask >> i) & 1:
                idx.append(None)
                continue
            if (self.ellipsis_mask >> i) & 1:
                idx.append(Ellipsis)
                continue
            bb = None if (self.begin_mask >> i) & 1 else b
            ee = None if (self.end_mask >> i) & 1 else e
            if s < 0:
                n = x.shape[i]
                sel = torch.arange(n - 1 if bb is None else (bb if bb >= 0 else bb + n),
                                   -1 if ee is None else (ee if ee >= 0 else ee + n), s, device=x.device)
                x = x.index_select(i, sel)
                idx.append(slice(None))
            else:
                idx.append(slice(bb, ee, s))
        return x[tuple(idx)]


class Tile(Primitive):
    def __init__(self):
        super().__init__("Tile")

    def _run(self, x, multiples):
        return x.repeat(*[int(m) for m in multiples]) if len(multiples) >= x.dim() else x.repeat(
            *([1] * (x.dim() - len(multiples)) + [int(m) for m in multiples]))


class BroadcastTo(Primitive):
    @prim_attr_register
    def __init__(self, shape):
        pass

    def _run(self, x):
        shp = [x.shape[i - (len(self.shape) - x.dim())] if s == -1 else s for i, s in enumerate(self.shape)]
        return torch.broadcast_to(x, shp)


class Gather(Primitive):
    @prim_attr_register
    def __init__(self, batch_dims=0):
        pass

    def _run(self, params, indices, axis):
        axis = int(axis)
        if axis == 0 and params.dim() == 2 and self.batch_dims == 0:
            return fused.embedding(params, indices)
        flat = torch.index_select(params, axis, indices.reshape(-1).long())
        return flat.reshape(params.shape[:axis] + tuple(indices.shape) + params.shape[axis + 1:])


GatherV2 = Gather
SparseGatherV2 = Gather


class EmbeddingLookup(Primitive):
    def __init__(self):
        super().__init__("EmbeddingLookup")

    def _run(self, params, indices, offset=0):
        return fused.embedding(params, indices, int(offset))


class GatherD(Primitive):
    def __init__(self):
        super().__init__("GatherD")

    def _run(self, x, dim, index):
        return torch.gather(x, int(dim), index.long())


class GatherNd(Primitive):
    def __init__(self):
        super().__init__("GatherNd")

    def _run(self, x, indices):
        idx = indices.long()
        return x[tuple(idx[..., i] for i in range(idx.shape[-1]))]


class ScatterNd(Primitive):
    def __init__(self):
        super().__init__("ScatterNd")

    def _run(self, indices, updates, shape):
        out = torch.zeros(tuple(shape), dtype=updates.dtype, device=updates.device)
        idx = indices.long()
        out.index_put_(tuple(idx[..., i] for i in range(idx.shape[-1])), updates, accumulate=True)
        return out


class TensorScatterUpdate(Primitive):
    def __init__(self):
        super().__init__("TensorScatterUpdate")

    def _run(self, x, indices, updates):
        out = x.clone()
        idx = indices.long()
        out[tuple(idx[..., i] for i in range(idx.shape[-1]))] = updates
        return out


class TensorScatterAdd(Primitive):
    def __init__(self):
        super().__init__("TensorScatterAdd")

    def _run(self, x, indices, updates):
        out = x.clone()
        idx = indices.long()
        out.index_put_(tuple(idx[..., i] for i in range(idx.shape[-1])), updates, accumulate=True)
        return out


class UnsortedSegmentSum(Primitive):
    def __init__(self):
        super().__init__("UnsortedSegmentSum")

    def _run(self, x, segment_ids, num_segments):
        ids = segment_ids.reshape(-1).long()
        flat = x.reshape((ids.numel(),) + tuple(x.shape[segment_ids.dim():]))
        out = torch.zeros((int(num_segments),) + tuple(flat.shape[1:]), dtype=x.dtype, device=x.device)
        return out.index_add_(0, ids, flat)


class OneHot(Primitive):
    @prim_attr_register
    def __init__(self, axis=-1):
        pass

    def _run(self, indices, depth, on_value, off_value):
        oh = F.one_hot(indices.long(), int(depth))
        on, off = _t(on_value), _t(off_value)
        out = torch.where(oh.bool(), on.to(oh.device), off.to(oh.device))
        if self.axis not in (-1, indices.dim()):
            out = out.movedim(-1, self.axis)
        return out


class Select(Primitive):
    def __init__(self):
        super().__init__("Select")

    def _run(self, cond, x, y):
        return torch.where(cond.bool(), _t(x, y if isinstance(y, torch.Tensor) else None),
                           _t(y, x if isinstance(x, torch.Tensor) else None))


class MaskedFill(Primitive):
    def __init__(self):
        super().__init__("MaskedFill")

    def _run(self, x, mask, value):
        return x.masked_fill(mask.bool(), value.item() if isinstance(value, torch.Tensor) and value.numel() == 1
                             else value)


class Fill(Primitive):
    def __init__(self):
        super().__init__("Fill")

    def _run(self, dtype, shape, value):
        return torch.full(tuple(shape), value, dtype=dtype)


class FillV2(Primitive):
    def __init__(self):
        super().__init__("FillV2")

    def _run(self, shape, value):
        v = _t(value)
        return torch.full(tuple(_axis(shape)), v.item(), dtype=v.dtype)


class Zeros(Primitive):
    def __init__(self):
        super().__init__("Zeros")

    def _run(self, shape, dtype=mstype.float32):
        return torch.zeros(tuple(shape) if not isinstance(shape, int) else (shape,), dtype=dtype)


class Ones(Zeros):
    def __init__(self):
        Primitive.__init__(self, "Ones")

    def _run(self, shape, dtype=mstype.float32):
        return torch.ones(tuple(shape) if not isinstance(shape, int) else (shape,), dtype=dtype)


class ReverseV2(Primitive):
    @prim_attr_register
    def __init__(self, axis):
        pass

    def _run(self, x):
        return torch.flip(x, tuple(self.axis))


class Tril(Primitive):
    @prim_attr_register
    def __init__(self, diagonal=0):
        pass

    def _run(self, x):
        return torch.tril(x, self.diagonal)


class Triu(Tril):
    def _run(self, x):
        return torch.triu(x, self.diagonal)


class Pad(Primitive):
    @prim_attr_register
    def __init__(self, paddings):
        pass

    def _run(self, x):
        flat = []
        for lo, hi in reversed(self.paddings):
            flat += [lo, hi]
        return F.pad(x, flat)


class PadV3(Primitive):
    @prim_attr_register
    def __init__(self, mode="constant", paddings_contiguous=True):
        pass

    def _run(self, x, paddings, value=0):
        return F.pad(x, [int(p) for p in _axis(paddings)], mode=self.mode, value=float(value) if self.mode == "constant" else None)


class Unique(Primitive):
    def __init__(self):
        super().__init__("Unique")

    def _run(self, x):
        vals, inv = torch.unique(x, sorted=False, return_inverse=True)
        return vals, inv.to(torch.int32)


class NonZero(Primitive):
    def __init__(self):
        super().__init__("NonZero")

    def _run(self, x):
        return torch.nonzero(x)


class Assign(Primitive):
    def __init__(self):
        super().__init__("Assign")
        self._update_parameter = True

    def _run(self, var, value):
        with torch.no_grad():
            torch.Tensor.copy_(var, _t(value, var))
        return var


class AssignAdd(Assign):
    def __init__(self):
        Primitive.__init__(self, "AssignAdd")
        self._update_parameter = True

    def _run(self, var, value):
        with torch.no_grad():
            torch.Tensor.add_(var, _t(value, var))
        return var


class AssignSub(Assign):
    def __init__(self):
        Primitive.__init__(self, "AssignSub")
        self._update_parameter = True

    def _run(self, var, value):
        with torch.no_grad():
            torch.Tensor.sub_(var, _t(value, var))
        return var


class Depend(Primitive):
    """value, expr -> value; orders side effects in graph mode (no-op in eager)."""

    def __init__(self):
        super().__init__("Depend")

    def _run(self, value, expr):
        return value


class UpdateState(Primitive):
    def __init__(self):
        super().__init__("UpdateState")

    def _run(self, state, *deps):
        return state


class Load(Primitive):
    def __init__(self):
        super().__init__("Load")

    def _run(self, param, state=None):
        return param


class Print(Primitive):
    def __init__(self):
        super().__init__("Print")

    def _run(self, *args):
        print(*[a.asnumpy() if isinstance(a, Tensor) else a for a in args])
        return None


# ------------------------------------------------------------------------------------ nn ops
class Softmax(Primitive):
    @prim_attr_register
    def __init__(self, axis=-1):
        pass

    def _run(self, x):
        ax = self.axis if isinstance(self.axis, int) else self.axis[0]
        return torch.softmax(x, dim=ax)


class LogSoftmax(Primitive):
    @prim_attr_register
    def __init__(self, axis=-1):
        pass

    def _run(self, x):
        return torch.log_softmax(x, dim=self.axis)


class GeLU(Primitive):
    def __init__(self):
        super().__init__("GeLU")

    def _run(self, x):
        return fused.gelu_tanh(x)


Gelu = GeLU


class Elu(Primitive):
    @prim_attr_register
    def __init__(self, alpha=1.0):
        pass

    def _run(self, x):
        return F.elu(x, self.alpha)


class LeakyReLU(Primitive):
    @prim_attr_register
    def __init__(self, alpha=0.2):
        pass

    def _run(self, x):
        return F.leaky_relu(x, self.alpha)


class PReLU(Primitive):
    def __init__(self):
        super().__init__("PReLU")

    def _run(self, x, w):
        return F.prelu(x, w)


class Dropout(Primitive):
    @prim_attr_register
    def __init__(self, keep_prob=0.5, Seed0=0, Seed1=0):
        pass

    def _run(self, x):
        if self.keep_prob >= 1.0:
            return x, torch.ones_like(x, dtype=torch.bool)
        mask = torch.rand_like(x, dtype=torch.float32) < self.keep_prob
        return x * mask.to(x.dtype) / self.keep_prob, mask


class LayerNorm(Primitive):
    @prim_attr_register
    def __init__(self, begin_norm_axis=1, begin_params_axis=1, epsilon=1e-7):
        pass

    def _run(self, x, gamma, beta):
        ax = self.begin_norm_axis % x.dim()
        if ax == x.dim() - 1:
            y = fused.layer_norm(x, gamma, beta, self.epsilon)
        else:
            y = F.layer_norm(x, tuple(x.shape[ax:]), gamma, beta, self.epsilon)
        xf = x.float()
        dims = tuple(range(ax, x.dim()))
        mean = xf.mean(dims, keepdim=True)
        var = xf.var(dims, unbiased=False, keepdim=True)
        return y, mean, var


class RmsNorm(Primitive):
    @prim_attr_register
    def __init__(self, epsilon=1e-6):
        pass

    def _run(self, x, gamma):
        y, _, rstd = fused.rms_norm(x, gamma, self.epsilon, with_rstd=True)
        return y, rstd


class ApplyRotaryPosEmb(Primitive):
    @prim_attr_register
    def __init__(self, cos_format=0):
        pass

    def _run(self, query, key, cos, sin, position_ids=None):
        # query/key: [B, S, H*D]; cos/sin: [S, D/2] fp32 tables
        S = query.shape[-2]
        D = cos.shape[-1] * 2
        return (fused.rope(query, cos, sin, query.shape[-1] // D, D, S),
                fused.rope(key, cos, sin, key.shape[-1] // D, D, S))


class FlashAttentionScore(Primitive):
    @prim_attr_register
    def __init__(self, head_num, keep_prob=1.0, scale_value=1.0, pre_tokens=2147483647, next_tokens=2147483647,
                 inner_precise=0, input_layout="BSH", sparse_mode=0):
        pass

    def _run(self, query, key, value, real_shift=None, drop_mask=None, padding_mask=None, attn_mask=None,
             prefix=None, actual_seq_qlen=None, actual_seq_kvlen=None):
        causal = self.next_tokens == 0 or self.sparse_mode in (2, 3)
        lay = self.input_layout
        H = self.head_num
        if lay == "BSH":
            B, S, Hd = query.shape
            D = Hd // H
            q = query.reshape(B, S, H, D)
            k = key.reshape(B, key.shape[1], -1, D)
            v = value.reshape(B, value.shape[1], -1, D)
        elif lay == "BNSD":
            q, k, v = (t.permute(0, 2, 1, 3) for t in (query, key, value))
        elif lay == "BSND":
            q, k, v = query, key, value
        elif lay == "SBH":
            S, B, Hd = query.shape
            D = Hd // H
            q = query.reshape(S, B, H, D).permute(1, 0, 2, 3)
            k = key.reshape(key.shape[0], B, -1, D).permute(1, 0, 2, 3)
            v = value.reshape(value.shape[0], B, -1, D).permute(1, 0, 2, 3)
        else:
            raise ValueError("input_layout %s is not supported" % lay)
        if attn_mask is not None and not causal:
            from .attention import reference_attention  # arbitrary mask: evaluate densely
            qt, kt, vt = (t.permute(0, 2, 1, 3) for t in (q, k, v))
            if kt.shape[1] != qt.shape[1]:
                kt = kt.repeat_interleave(qt.shape[1] // kt.shape[1], 1)
                vt = vt.repeat_interleave(qt.shape[1] // vt.shape[1], 1)
            m = attn_mask.bool()
            o = F.scaled_dot_product_attention(qt, kt, vt, attn_mask=~m if m.dim() >= 2 else None,
                                               scale=self.scale_value).permute(0, 2, 1, 3)
        else:
            o = fused.flash_attention(q.contiguous(), k.contiguous(), v.contiguous(), causal, self.scale_value)
        if lay == "BSH":
            out = o.reshape(query.shape)
        elif lay == "BNSD":
            out = o.permute(0, 2, 1, 3)
        elif lay == "SBH":
            out = o.permute(1, 0, 2, 3).reshape(query.shape)
        else:
            out = o
        return None, None, None, out


class SoftmaxCrossEntropyWithLogits(Primitive):
    def __init__(self):
        super().__init__("SoftmaxCrossEntropyWithLogits")

    def _run(self, logits, labels):
        lsm = torch.log_softmax(logits.float(), -1)
        loss = -(labels.float() * lsm).sum(-1)
        return loss, (torch.softmax(logits.float(), -1) - labels.float()).to(logits.dtype)


class SparseSoftmaxCrossEntropyWithLogits(Primitive):
    @prim_attr_register
    def __init__(self, is_grad=False):
        pass

    def _run(self, logits, labels):
        if self.is_grad:
            p = torch.softmax(logits.float(), -1)
            p[torch.arange(p.shape[0]), labels.long()] -= 1
            return (p / logits.shape[0]).to(logits.dtype)
        return fused.softmax_cross_entropy(logits, labels)


class NLLLoss(Primitive):
    @prim_attr_register
    def __init__(self, reduction="mean", ignore_index=-100):
        pass

    def _run(self, logits, labels, weight):
        loss = F.nll_loss(logits, labels.long(), weight, reduction=self.reduction, ignore_index=self.ignore_index)
        tw = weight[labels.long()].sum() if weight is not None else torch.tensor(float(labels.numel()))
        return loss, tw


class SigmoidCrossEntropyWithLogits(Primitive):
    def __init__(self):
        super().__init__("SigmoidCrossEntropyWithLogits")

    def _run(self, logits, labels):
        return F.binary_cross_entropy_with_logits(logits, labels, reduction="none")


class BinaryCrossEntropy(Primitive):
    @prim_attr_register
    def __init__(self, reduction="mean"):
        pass

    def _run(self, x, y, weight=None):
        return F.binary_cross_entropy(x, y, weight, reduction=self.reduction)


class SmoothL1Loss(Primitive):
    @prim_attr_register
    def __init__(self, beta=1.0, reduction="none"):
        pass

    def _run(self, x, y):
        return F.smooth_l1_loss(x, y, beta=self.beta, reduction=self.reduction)


class KLDivLoss(Primitive):
    @prim_attr_register
    def __init__(self, reduction="mean"):
        pass

    def _run(self, x, y):
        return F.kl_div(x, y, reduction=self.reduction)


def _pair(v):
    return (v, v) if isinstance(v, int) else tuple(v)


class Conv2D(Primitive):
    @prim_attr_register
    def __init__(self, out_channel, kernel_size, mode=1, pad_mode="valid", pad=0, stride=1, dilation=1, group=1,
                 data_format="NCHW"):
        pass

    def _run(self, x, w):
        from . import conv as _conv
        stride = _pair(self.stride)[-2:]
        dil = _pair(self.dilation)[-2:]
        return _conv.conv2d(x, w, stride, self.pad_mode, self.pad, dil, self.group)


class Conv2DTranspose(Primitive):
    @prim_attr_register
    def __init__(self, out_channel, kernel_size, pad_mode="valid", pad=0, pad_list=None, mode=1, stride=1,
                 dilation=1, group=1, data_format="NCHW"):
        pass

    def _run(self, dout, w, input_size):
        stride = _pair(self.stride)[-2:]
        pad = _pair(self.pad)[:2] if not isinstance(self.pad, int) else (self.pad, self.pad)
        return torch.nn.grad.conv2d_input(tuple(input_size), w, dout, stride, pad, _pair(self.dilation)[-2:],
                                          self.group)


class MaxPool(Primitive):
    @prim_attr_register
    def __init__(self, kernel_size=1, strides=1, pad_mode="valid", data_format="NCHW"):
        pass

    def _run(self, x):
        k, s = _pair(self.kernel_size)[-2:], _pair(self.strides)[-2:]
        if self.pad_mode.lower() == "same":
            x = _same_pad(x, k, s, float("-inf"))
        return F.max_pool2d(x, k, s)


class AvgPool(MaxPool):
    def _run(self, x):
        k, s = _pair(self.kernel_size)[-2:], _pair(self.strides)[-2:]
        if self.pad_mode.lower() == "same":
            x = _same_pad(x, k, s, 0.0)
        return F.avg_pool2d(x, k, s)


def _same_pad(x, k, s, value):
    h, w = x.shape[-2:]
    ph = max((math.ceil(h / s[0]) - 1) * s[0] + k[0] - h, 0)
    pw = max((math.ceil(w / s[1]) - 1) * s[1] + k[1] - w, 0)
    return F.pad(x, (pw // 2, pw - pw // 2, ph // 2, ph - ph // 2), value=value)


class BatchNorm(Primitive):
    @prim_attr_register
    def __init__(self, is_training=False, epsilon=1e-5, momentum=0.1, data_format="NCHW"):
        pass

    def _run(self, x, scale, bias, mean, variance):
        from . import conv as _conv
        y = _conv.batch_norm(x, scale, bias, mean, variance, self.is_training, self.momentum, self.epsilon)
        return y, mean, variance, mean, variance


class ResizeNearestNeighbor(Primitive):
    @prim_attr_register
    def __init__(self, size, align_corners=False):
        pass

    def _run(self, x):
        return F.interpolate(x, size=tuple(self.size), mode="nearest")


class ResizeBilinearV2(Primitive):
    @prim_attr_register
    def __init__(self, align_corners=False, half_pixel_centers=False):
        pass

    def _run(self, x, size):
        return F.interpolate(x, size=tuple(size), mode="bilinear", align_corners=self.align_corners)


class Flatten(Primitive):
    def __init__(self):
        super().__init__("Flatten")

    def _run(self, x):
        return x.reshape(x.shape[0], -1)


# ------------------------------------------------------------------------------------ optimizer apply ops
class ApplyMomentum(Primitive):
    @prim_attr_register
    def __init__(self, use_nesterov=False, use_locking=False, gradient_scale=1.0):
        self._update_parameter = True

    def _run(self, var, accum, lr, grad, momentum):
        with torch.no_grad():
            lr = float(lr) if not isinstance(lr, torch.Tensor) else lr
            g = grad.to(var.dtype)
            torch.Tensor.mul_(accum, momentum).add_(g)
            if self.use_nesterov:
                torch.Tensor.sub_(var, (g + accum * momentum) * lr)
            else:
                torch.Tensor.sub_(var, accum * lr)
        return var


class SGD(Primitive):
    @prim_attr_register
    def __init__(self, dampening=0.0, weight_decay=0.0, nesterov=False):
        self._update_parameter = True

    def _run(self, var, grad, lr, accum, momentum, stat):
        with torch.no_grad():
            g = grad.to(var.dtype)
            if self.weight_decay:
                g = g + self.weight_decay * var
            if float(momentum) != 0:
                first = bool(stat.any()) if isinstance(stat, torch.Tensor) else False
                if first:
                    torch.Tensor.copy_(accum, g)
                    torch.Tensor.zero_(stat)
                else:
                    torch.Tensor.mul_(accum, momentum).add_(g * (1 - self.dampening))
                g = g + momentum * accum if self.nesterov else accum
            torch.Tensor.sub_(var, lr * g)
        return var


class Adam(Primitive):
    @prim_attr_register
    def __init__(self, use_locking=False, use_nesterov=False):
        self._update_parameter = True

    def _run(self, var, m, v, beta1_power, beta2_power, lr, beta1, beta2, epsilon, grad):
        with torch.no_grad():
            g = grad.to(var.dtype)
            torch.Tensor.mul_(m, beta1).add_(g, alpha=1 - float(beta1))
            torch.Tensor.mul_(v, beta2).addcmul_(g, g, value=1 - float(beta2))
            lr_t = lr * math.sqrt(1 - float(beta2_power)) / (1 - float(beta1_power))
            torch.Tensor.sub_(var, lr_t * m / (torch.sqrt(v) + epsilon))
        return var, m, v


class AdamWeightDecay(Primitive):
    @prim_attr_register
    def __init__(self, use_locking=False):
        self._update_parameter = True

    def _run(self, var, m, v, lr, beta1, beta2, epsilon, decay, grad):
        with torch.no_grad():
            g = grad.to(m.dtype)
            torch.Tensor.mul_(m, beta1).add_(g, alpha=1 - float(beta1))
            torch.Tensor.mul_(v, beta2).addcmul_(g, g, value=1 - float(beta2))
            update = m / (torch.sqrt(v) + epsilon) + float(decay) * var
            torch.Tensor.sub_(var, (float(lr) if not isinstance(lr, torch.Tensor) else lr) * update)
        return var, m, v


# ------------------------------------------------------------------------------------ random
class StandardNormal(Primitive):
    @prim_attr_register
    def __init__(self, seed=0, seed2=0):
        pass

    def _run(self, shape):
        return torch.randn(tuple(shape))


class UniformReal(StandardNormal):
    def _run(self, shape):
        return torch.rand(tuple(shape))


class UniformInt(StandardNormal):
    def _run(self, shape, minval, maxval):
        return torch.randint(int(minval), int(maxval), tuple(shape), dtype=torch.int32)


class Multinomial(Primitive):
    @prim_attr_register
    def __init__(self, seed=0, seed2=0, dtype=mstype.int32):
        pass

    def _run(self, x, num):
        return torch.multinomial(x, int(num), replacement=True).to(self.dtype)


class TopKRouter(Primitive):
    """Token -> expert dispatch bookkeeping (capacity-limited top-k routing)."""

    def __init__(self):
        super().__init__("TopKRouter")

    def _run(self, x, capacity, expert_num, drop_type=0):
        # x: [B, T, k] expert ids per token -> dispatch_idx [B, E, cap], combine_idx [B, T, k]
        B, T, k = x.shape
        E, cap = int(expert_num), int(capacity)
        ids = x.reshape(B, T * k).long()
        oh = F.one_hot(ids, E)
        pos = (oh.cumsum(1) - 1) * oh
        pos_in_e = pos.sum(-1)
        keep = pos_in_e < cap
        dispatch = torch.zeros(B, E, cap, dtype=torch.int32, device=x.device)
        tok = torch.arange(T * k, device=x.device)[None].expand(B, -1) // k + 1
        bidx = torch.arange(B, device=x.device)[:, None].expand(-1, T * k)
        dispatch[bidx[keep], ids[keep], pos_in_e[keep]] = tok[keep].to(torch.int32)
        combine = torch.where(keep, ids * (cap + 1) + pos_in_e + 1, torch.zeros_like(ids)).reshape(B, T, k)
        return dispatch, combine.to(torch.int32)


__all__ = [n for n, v in list(globals().items()) if isinstance(v, type) and issubclass(v, Primitive)]


from .operations_ext import *  # noqa: E402,F401,F403  (second-tier primitives)
from .operations_more import *  # noqa: E402,F401,F403  (third tier: the long tail)
from .operations_tail import *  # noqa: E402,F401,F403  (recurrent cells over packed weights, replay buffer, ...)
from .llm_ops import *  # noqa: E402,F401,F403  (fused decoder primitives)
from . import llm_ops as _llm_ops  # noqa: E402

from . import operations_ext as _ops_ext, operations_more as _ops_more, operations_tail as _ops_tail  # noqa: E402

__all__ = list(dict.fromkeys(__all__ + list(_ops_ext.__all__) + list(_ops_more.__all__) + list(_ops_tail.__all__) +
                             list(_llm_ops.__all__)))



_COMM_NAMES = ("AllGather", "AllReduce", "AlltoAll", "AlltoAllV", "Barrier", "BatchISendIRecv", "Broadcast",
               "CollectiveGather", "CollectiveScatter", "NeighborExchange", "NeighborExchangeV2", "Receive", "Reduce",
               "ReduceOp", "ReduceScatter", "Send", "AShardIdentity", "_AllSwap")


def __getattr__(name):
    # the communication primitives import the communication package, which imports ops: resolved on first use
    if name in _COMM_NAMES:
        import importlib
        return getattr(importlib.import_module(__package__ + ".comm_ops"), name)
    if name == "Partial":
        import importlib
        return importlib.import_module(__package__ + ".composite").Partial
    raise AttributeError("module %r has no attribute %r" % (__name__, name))
