"""Distributed semantics of the array, convolution / normalisation and selection primitives that sit between the
MatMuls of a network: which dims may be split, how shape-like arguments change on a slice, what communication a
split needs.  Each class follows the rule of its reference counterpart:

  StridedSlice / Slice      ops_info/strided_slice_info.cc, slice_info.cc   a dim that is really sliced stays whole
  Split / SplitV / Unstack  ops_info/split_info.cc                          the split axis stays whole
  Concat / Stack            ops_info/concat_info.cc, stack_info.cc          inputs alike, the axis stays whole
  Tile                      ops_info/tile_info.cc                           a split of a tiled dim divides the multiple
  ExpandDims / Squeeze      ops_info/activation_info.cc (ExpandDimsInfo, SqueezeInfo)
  BroadcastTo               ops_info/broadcast_to_info.cc
  BiasAdd / PReLU           ops_info/bias_add_info.cc, prelu_info.cc        per-channel operand follows the channel split
  BatchNorm                 ops_info/batchnorm_info.cc                      batch / spatial splits all-reduce the statistics
  Conv2D                    ops_info/conv2d_info.cc                         batch, in-channel (AllReduce) and out-channel
  MaxPool / AvgPool / resize ops_info/maxpool_info.cc, resizebilinear_info.cc   batch and channel
  TopK / Sort / CumSum / ArgMax(Min)WithValue / L2Normalize / GatherD      the working axis stays whole
  UnsortedSegmentSum        ops_info/unsorted_segment_op_info.cc            split id dims -> AllReduce of the partial sums

A halo exchange for convolutions / pooling split along H or W (conv2d_info.cc:600-1100) is not implemented: those
strategies raise ``StrategyError``."""
from __future__ import annotations

import numpy as np

from .operator_info import ActivationInfo, OperatorInfo, StrategyError, _AxisOpInfo, _divisors, register


def _norm_axis(a, rank):
    a = int(a)
    if a < -rank or a >= rank:
        raise StrategyError("axis %d is out of range for rank %d" % (a, rank))
    return a % rank


class _SingleInputInfo(OperatorInfo):
    """One tensor input; the device matrix is its strategy; other (non-tensor) arguments ride along."""

    def __init__(self, prim, in_shapes, in_strategy, out_strategy=None, stage_devices=1, attrs=None, **extra):
        self.extra = extra
        super().__init__(prim, in_shapes[:1], in_strategy[:1], out_strategy, stage_devices, attrs)

    def base_dev_matrix(self):
        return list(self.in_strategy[0])

    def infer_inputs_tensor_map(self):
        return [[self._k(i) if s > 1 else -1 for i, s in enumerate(self.in_strategy[0])]]

    def out_shapes(self):
        return [self.in_shapes[0]]

    def infer_outputs_tensor_map(self):
        return [list(self.inputs_tensor_map[0])]

    def _whole(self, dims, what):
        for d in dims:
            if self.in_strategy[0][d] != 1:
                raise StrategyError("%s: %s (dim %d) can not be split, got strategy %s"
                                    % (self.prim_name, what, d, self.in_strategy[0]))

    @classmethod
    def generate_strategies(cls, in_shapes, device_num):
        return ActivationInfo.generate_strategies(in_shapes[:1], device_num)


# ------------------------------------------------------------------------------------------------ slicing
@register("StridedSlice")
class StridedSliceInfo(_SingleInputInfo):
    """extra: begin, end, strides (tuples, one entry per leading dim).  A dim whose whole extent is taken with
    stride 1 may be split (its ``end`` is divided on the slice); a dim that is cut, strided or shrunk may not."""

    def _spec(self):
        x = self.in_shapes[0]
        begin, end, strides = (tuple(int(v) for v in self.extra[k]) for k in ("begin", "end", "strides"))
        if not (len(begin) == len(end) == len(strides)) or len(begin) > len(x):
            raise StrategyError("StridedSlice: begin / end / strides must have equal length <= rank")
        a = self.attrs
        if a.get("ellipsis_mask", 0) or a.get("new_axis_mask", 0):
            raise StrategyError("StridedSlice: ellipsis_mask / new_axis_mask are not supported under a shard strategy")
        return begin, end, strides, int(a.get("begin_mask", 0)), int(a.get("end_mask", 0)), int(a.get("shrink_axis_mask", 0))

    def _full(self, i):
        begin, end, strides, bm, em, sm = self._spec()
        if i >= len(begin):
            return True
        if (sm >> i) & 1 or strides[i] != 1:
            return False
        n = self.in_shapes[0][i]
        b = 0 if (bm >> i) & 1 else (begin[i] + n if begin[i] < 0 else begin[i])
        e = n if (em >> i) & 1 else (end[i] + n if end[i] < 0 else min(end[i], n))
        return b == 0 and e == n

    def check_strategy(self):
        OperatorInfo.check_strategy(self)
        self._whole([i for i in range(len(self.in_shapes[0])) if not self._full(i)], "a dim that is sliced")

    def out_shapes(self):
        begin, end, strides, bm, em, sm = self._spec()
        out = []
        for i, n in enumerate(self.in_shapes[0]):
            if i >= len(begin):
                out.append(n)
                continue
            if (sm >> i) & 1:
                continue
            out.append(len(range(*slice(None if (bm >> i) & 1 else begin[i], None if (em >> i) & 1 else end[i],
                                        strides[i]).indices(n))))
        return [tuple(out)]

    def infer_outputs_tensor_map(self):
        _, _, _, _, _, sm = self._spec()
        return [[m for i, m in enumerate(self.inputs_tensor_map[0]) if not (sm >> i) & 1]]

    def localize_args(self, others):
        begin, end, strides, bm, em, sm = self._spec()
        st = self.in_strategy[0]
        x = self.in_shapes[0]
        new_end = tuple((x[i] // st[i]) if (st[i] > 1 and not (em >> i) & 1) else end[i] for i in range(len(end)))
        new_begin = tuple(0 if st[i] > 1 else begin[i] for i in range(len(begin)))
        return [new_begin, new_end, strides] + list(others[3:])


@register("Slice", "SliceExt")
class SliceInfo(_SingleInputInfo):
    """extra: begin, size.  Dims taken whole (begin 0, size = extent or -1) may be split."""

    def _full(self, i):
        begin, size = self.extra["begin"], self.extra["size"]
        return int(begin[i]) == 0 and int(size[i]) in (-1, self.in_shapes[0][i])

    def check_strategy(self):
        OperatorInfo.check_strategy(self)
        self._whole([i for i in range(len(self.in_shapes[0])) if not self._full(i)], "a dim that is sliced")

    def out_shapes(self):
        begin, size = self.extra["begin"], self.extra["size"]
        return [tuple(n - int(b) if int(s) == -1 else int(s) for n, b, s in zip(self.in_shapes[0], begin, size))]

    def localize_args(self, others):
        begin, size = others[0], others[1]
        st = self.in_strategy[0]
        new_size = tuple(int(s) if (st[i] == 1 or int(s) == -1) else int(s) // st[i] for i, s in enumerate(size))
        return [tuple(begin), new_size] + list(others[2:])


@register("Split", "SplitV", "SplitTensor", "SplitWithSize", "Unstack")
class SplitInfo(_SingleInputInfo):
    def _axis_num(self):
        a = self.attrs
        rank = len(self.in_shapes[0])
        if self.prim_name == "SplitV":
            sizes = list(a["size_splits"])
            ax = _norm_axis(a["split_dim"], rank)
            if -1 in sizes:
                sizes[sizes.index(-1)] = self.in_shapes[0][ax] - sum(s for s in sizes if s != -1)
            return ax, sizes
        ax = _norm_axis(a.get("axis", 0), rank)
        n = self.in_shapes[0][ax]
        if self.prim_name == "Unstack":
            return ax, [None] * n
        num = int(a.get("output_num", 1))
        if n % num:
            raise StrategyError("Split: dim %d of size %d is not divisible into %d outputs" % (ax, n, num))
        return ax, [n // num] * num

    def check_strategy(self):
        OperatorInfo.check_strategy(self)
        self._whole([self._axis_num()[0]], "the split axis")

    def out_shapes(self):
        ax, sizes = self._axis_num()
        x = list(self.in_shapes[0])
        if self.prim_name == "Unstack":
            return [tuple(x[:ax] + x[ax + 1:]) for _ in sizes]
        return [tuple(x[:ax] + [s] + x[ax + 1:]) for s in sizes]

    def infer_outputs_tensor_map(self):
        ax, sizes = self._axis_num()
        m = list(self.inputs_tensor_map[0])
        if self.prim_name == "Unstack":
            m = m[:ax] + m[ax + 1:]
        return [list(m) for _ in sizes]


class _ListInputInfo(OperatorInfo):
    """Concat / Stack / AddN style: every input has the same shape class and must be split alike."""

    def __init__(self, prim, in_shapes, in_strategy, out_strategy=None, stage_devices=1, attrs=None, **extra):
        self.extra = extra
        if len(in_strategy) == 1 and len(in_shapes) > 1:
            in_strategy = tuple(in_strategy) * len(in_shapes)      # one strategy given for the whole tuple
        super().__init__(prim, in_shapes, in_strategy, out_strategy, stage_devices, attrs)

    def check_strategy(self):
        OperatorInfo.check_strategy(self)
        if any(st != self.in_strategy[0] for st in self.in_strategy):
            raise StrategyError("%s: every input must use the same strategy, got %s" % (self.prim_name,
                                                                                       self.in_strategy))

    def used_devices(self):
        return int(np.prod(self.in_strategy[0])) if self.in_strategy[0] else 1

    def base_dev_matrix(self):
        return list(self.in_strategy[0])

    def infer_inputs_tensor_map(self):
        m = [self._k(i) if s > 1 else -1 for i, s in enumerate(self.in_strategy[0])]
        return [list(m) for _ in self.in_shapes]


@register("Concat")
class ConcatInfo(_ListInputInfo):
    def _axis(self):
        return _norm_axis(self.attrs.get("axis", 0), len(self.in_shapes[0]))

    def check_strategy(self):
        super().check_strategy()
        if self.in_strategy[0][self._axis()] != 1:
            raise StrategyError("Concat: the concat axis %d can not be split" % self._axis())

    def out_shapes(self):
        ax = self._axis()
        x = list(self.in_shapes[0])
        x[ax] = sum(s[ax] for s in self.in_shapes)
        return [tuple(x)]

    def infer_outputs_tensor_map(self):
        return [list(self.inputs_tensor_map[0])]


@register("Stack", "StackExt", "Pack")
class StackInfo(_ListInputInfo):
    def _axis(self):
        return _norm_axis(self.attrs.get("axis", 0), len(self.in_shapes[0]) + 1)

    def out_shapes(self):
        ax = self._axis()
        x = list(self.in_shapes[0])
        return [tuple(x[:ax] + [len(self.in_shapes)] + x[ax:])]

    def infer_outputs_tensor_map(self):
        ax = self._axis()
        m = list(self.inputs_tensor_map[0])
        return [m[:ax] + [-1] + m[ax:]]


# ------------------------------------------------------------------------------------------------ shape changers
@register("Tile")
class TileInfo(_SingleInputInfo):
    """extra: multiples.  The strategy is written over the *output* dims (rank = len(multiples)): where the
    multiple is 1 it splits the input dim; where the multiple is > 1 the input dim stays whole and the split divides
    the multiple (every rank produces multiple / split copies)."""

    def __init__(self, prim, in_shapes, in_strategy, out_strategy=None, stage_devices=1, attrs=None, **extra):
        self.mult = tuple(int(m) for m in extra["multiples"])
        x = tuple(in_shapes[0])
        self.pad = len(self.mult) - len(x)
        if self.pad < 0:
            self.mult = (1,) * (-self.pad) + self.mult
            self.pad = 0
        self.full_strategy = tuple(in_strategy[0])
        if len(self.full_strategy) != len(self.mult):
            raise StrategyError("Tile: the strategy %s must have one entry per multiple %s" % (self.full_strategy,
                                                                                              self.mult))
        xs = (1,) * self.pad + x
        for s, m, d in zip(self.full_strategy, self.mult, xs):
            if m > 1 and m % s:
                raise StrategyError("Tile: multiple %d is not divisible by the split %d" % (m, s))
            if m == 1 and d % s:
                raise StrategyError("Tile: dim of size %d is not divisible by the split %d" % (d, s))
        in_st = tuple(1 if m > 1 else s for s, m in zip(self.full_strategy, self.mult))[self.pad:]
        super().__init__(prim, in_shapes, (in_st,), out_strategy, stage_devices, attrs, **extra)

    def used_devices(self):
        return int(np.prod(self.full_strategy))

    def base_dev_matrix(self):
        return list(self.full_strategy)

    def infer_inputs_tensor_map(self):
        return [[self._k(self.pad + i) if (self.mult[self.pad + i] == 1 and self.full_strategy[self.pad + i] > 1)
                 else -1 for i in range(len(self.in_shapes[0]))]]

    def out_shapes(self):
        xs = (1,) * self.pad + tuple(self.in_shapes[0])
        return [tuple(d * m for d, m in zip(xs, self.mult))]

    def infer_outputs_tensor_map(self):
        return [[self._k(i) if s > 1 else -1 for i, s in enumerate(self.full_strategy)]]

    def localize_args(self, others):
        return [tuple(m // s if m > 1 else m for m, s in zip(self.mult, self.full_strategy))] + list(others[1:])


@register("ExpandDims")
class ExpandDimsInfo(_SingleInputInfo):
    def _axis(self):
        return _norm_axis(self.extra.get("axis", 0), len(self.in_shapes[0]) + 1)

    def out_shapes(self):
        x = list(self.in_shapes[0])
        ax = self._axis()
        return [tuple(x[:ax] + [1] + x[ax:])]

    def infer_outputs_tensor_map(self):
        m = list(self.inputs_tensor_map[0])
        ax = self._axis()
        return [m[:ax] + [-1] + m[ax:]]


@register("Squeeze")
class SqueezeInfo(_SingleInputInfo):
    def _axes(self):
        ax = self.attrs.get("axis", ())
        x = self.in_shapes[0]
        if ax in ((), None):
            return [i for i, d in enumerate(x) if d == 1]
        ax = [ax] if isinstance(ax, int) else list(ax)
        return sorted(_norm_axis(a, len(x)) for a in ax)

    def check_strategy(self):
        OperatorInfo.check_strategy(self)
        self._whole(self._axes(), "a squeezed dim")

    def out_shapes(self):
        ax = self._axes()
        return [tuple(d for i, d in enumerate(self.in_shapes[0]) if i not in ax)]

    def infer_outputs_tensor_map(self):
        ax = self._axes()
        return [[m for i, m in enumerate(self.inputs_tensor_map[0]) if i not in ax]]


@register("BroadcastTo")
class BroadcastToInfo(_SingleInputInfo):
    """attr shape.  Input dims of size 1 that are expanded stay whole; the other dims keep their split; new leading
    dims are not split."""

    def _target(self):
        x = self.in_shapes[0]
        shp = list(self.attrs.get("shape", self.extra.get("shape", ())))
        off = len(shp) - len(x)
        return [x[i - off] if s == -1 else int(s) for i, s in enumerate(shp)], off

    def check_strategy(self):
        OperatorInfo.check_strategy(self)
        tgt, off = self._target()
        self._whole([i for i, d in enumerate(self.in_shapes[0]) if d == 1 and tgt[off + i] != 1], "an expanded dim")

    def out_shapes(self):
        return [tuple(self._target()[0])]

    def infer_outputs_tensor_map(self):
        _, off = self._target()
        return [[-1] * off + list(self.inputs_tensor_map[0])]

    def local_attrs(self):
        tgt, off = self._target()
        st = self.in_strategy[0]
        return {"shape": tuple(tgt[:off]) + tuple(t // st[i] for i, t in enumerate(tgt[off:]))}


# ------------------------------------------------------------------------------------------------ per-channel operands
class _ChannelOperandInfo(OperatorInfo):
    """x [N, C, ...] with 1-D per-channel operands (bias, PReLU slope, BatchNorm scale / statistics): the operands
    follow the split of the channel dim (dim 1, or the last dim for NHWC)."""

    def _cdim(self):
        fmt = self.attrs.get("data_format", "NCHW")
        return len(self.in_shapes[0]) - 1 if fmt == "NHWC" or len(self.in_shapes[0]) == 2 and fmt != "NCHW" else 1

    def check_strategy(self):
        OperatorInfo.check_strategy(self)
        c = self.in_strategy[0][self._cdim()]
        for st, sh in zip(self.in_strategy[1:], self.in_shapes[1:]):
            if len(sh) == 1 and sh[0] != 1 and st[0] != c:
                raise StrategyError("%s: a per-channel operand must be split like the channel dim (%d), got %s"
                                    % (self.prim_name, c, st))

    def used_devices(self):
        return int(np.prod(self.in_strategy[0]))

    def base_dev_matrix(self):
        return list(self.in_strategy[0])

    def infer_inputs_tensor_map(self):
        m = [self._k(i) if s > 1 else -1 for i, s in enumerate(self.in_strategy[0])]
        maps = [m]
        for sh in self.in_shapes[1:]:
            maps.append([m[self._cdim()] if (len(sh) == 1 and sh[0] != 1) else -1] * len(sh))
        return maps

    def out_shapes(self):
        return [self.in_shapes[0]]

    def infer_outputs_tensor_map(self):
        return [list(self.inputs_tensor_map[0])]


@register("BiasAdd", "PReLU")
class BiasAddInfo(_ChannelOperandInfo):
    pass


@register("BatchNorm")
class BatchNormInfo(_ChannelOperandInfo):
    """x (n, c, h, w) and scale / bias / mean / variance (c,).  A channel split is purely local.  A split of the
    batch (or spatial) dims in training mode makes every rank hold part of each channel's samples: the per-channel
    sums are all-reduced over those device dims before normalising (``needs_sync_stats`` -> the dispatcher runs the
    synchronised formulation), the reference's forward AllReduce of batchnorm_info.cc:276-345."""

    def out_shapes(self):
        x, c = self.in_shapes[0], self.in_shapes[1]
        return [x, c, c, c, c]

    def infer_outputs_tensor_map(self):
        m = list(self.inputs_tensor_map[0])
        cm = [m[self._cdim()]]
        return [m, list(cm), list(cm), list(cm), list(cm)]

    def stat_dev_dims(self):
        """Device dims over which a channel's samples are spread (everything but the channel split)."""
        m = self.inputs_tensor_map[0]
        return [k for i, k in enumerate(m) if i != self._cdim() and k != -1]

    def needs_sync_stats(self):
        return bool(self.attrs.get("is_training", False)) and bool(self.stat_dev_dims())


@register("Conv2D", "Convolution")
class Conv2DInfo(OperatorInfo):
    """x (n, ci, h, w), weight (co, ci / group, kh, kw) -> (n, co, h', w').  Device matrix [n, ci, co]: the batch
    and the output channels split freely; a split of the input channels (both operands alike) yields partial sums
    that are all-reduced.  H / W splits need a halo exchange and are refused."""

    def check_strategy(self):
        OperatorInfo.check_strategy(self)
        sx, sw = self.in_strategy[0], self.in_strategy[1]
        if any(s != 1 for s in sx[2:]) or any(s != 1 for s in sw[2:]):
            raise StrategyError("Conv2D: splitting H / W (halo exchange) or the kernel dims is not supported")
        if sx[1] != sw[1]:
            raise StrategyError("Conv2D: the input channels are split %d ways in x but %d in the weight" % (sx[1], sw[1]))
        g = int(self.attrs.get("group", 1))
        if g > 1 and (sx[1] > 1 or sw[0] > 1) and (sx[1] != sw[0] or g % sw[0]):
            raise StrategyError("Conv2D: with group=%d channels may only be split by whole groups (in and out alike)" % g)

    def used_devices(self):
        sx, sw = self.in_strategy[0], self.in_strategy[1]
        return sx[0] * sx[1] * sw[0] if int(self.attrs.get("group", 1)) == 1 else sx[0] * sw[0]

    def _grouped(self):
        return int(self.attrs.get("group", 1)) > 1 and self.in_strategy[1][0] > 1

    def base_dev_matrix(self):
        sx, sw = self.in_strategy[0], self.in_strategy[1]
        if self._grouped():
            return [sx[0], 1, sw[0]]
        return [sx[0], sx[1], sw[0]]

    def infer_inputs_tensor_map(self):
        sx, sw = self.in_strategy[0], self.in_strategy[1]
        kn = self._k(0) if sx[0] > 1 else -1
        kco = self._k(2) if sw[0] > 1 else -1
        if self._grouped():
            return [[kn, kco, -1, -1], [kco, -1, -1, -1]]
        kci = self._k(1) if sx[1] > 1 else -1
        return [[kn, kci, -1, -1], [kco, kci, -1, -1]]

    def out_shapes(self):
        a = self.attrs
        n, _, h, w = self.in_shapes[0]
        co, _, kh, kw = self.in_shapes[1]

        def pair(v):
            return (v, v) if isinstance(v, int) else tuple(v)[-2:]
        sh, sw_ = pair(a.get("stride", 1))
        dh, dw = pair(a.get("dilation", 1))
        mode = str(a.get("pad_mode", "valid")).lower()
        if mode == "same":
            ho, wo = -(-h // sh), -(-w // sw_)
        else:
            p = a.get("pad", 0)
            pt, pb, pl, pr = (p, p, p, p) if isinstance(p, int) else tuple(p)
            if mode == "valid":
                pt = pb = pl = pr = 0
            ho = (h + pt + pb - dh * (kh - 1) - 1) // sh + 1
            wo = (w + pl + pr - dw * (kw - 1) - 1) // sw_ + 1
        return [(n, co, ho, wo)]

    def infer_outputs_tensor_map(self):
        sx, sw = self.in_strategy[0], self.in_strategy[1]
        return [[self._k(0) if sx[0] > 1 else -1, self._k(2) if sw[0] > 1 else -1, -1, -1]]

    def infer_forward_comm(self):
        sx = self.in_strategy[0]
        self.forward_comm = ("AllReduce", [self._k(1)]) if (sx[1] > 1 and not self._grouped()) else None

    def local_attrs(self):
        out = {"out_channel": int(self.attrs.get("out_channel", self.in_shapes[1][0])) // self.in_strategy[1][0]}
        if self._grouped():
            out["group"] = int(self.attrs["group"]) // self.in_strategy[1][0]
        return out

    @classmethod
    def generate_strategies(cls, in_shapes, device_num):
        x, w = in_shapes
        cands = []
        for dn in _divisors(device_num):
            for dco in _divisors(device_num // dn):
                if x[0] % dn or w[0] % dco:
                    continue
                cands.append(((dn, 1, 1, 1), (dco, 1, 1, 1)))
        return cands


@register("MaxPool", "AvgPool", "ResizeNearestNeighbor", "ResizeBilinearV2", "MaxPool3D", "AvgPool3D", "ROIAlign",
          "CropAndResize", "GridSampler2D")
class SpatialOpInfo(_SingleInputInfo):
    """Pooling / resize on (n, c, spatial...): batch and channel split; spatial dims need a halo exchange."""

    def check_strategy(self):
        OperatorInfo.check_strategy(self)
        self._whole(range(2, len(self.in_shapes[0])), "a spatial dim")

    def out_shapes(self):
        return [None]          # spatial extents follow the op's attributes; only the map matters here

    def infer_outputs_tensor_map(self):
        return [list(self.inputs_tensor_map[0])]


# ------------------------------------------------------------------------------------------------ axis-bound ops
class _WholeAxisInfo(_SingleInputInfo):
    """The working axis (attr ``axis`` / argument) must stay whole; everything else splits freely."""

    n_outputs = 1
    drops_axis = False

    def _axis(self):
        a = self.extra.get("axis", self.attrs.get("axis", -1))
        return _norm_axis(a, len(self.in_shapes[0]))

    def check_strategy(self):
        OperatorInfo.check_strategy(self)
        self._whole([self._axis()], "the working axis")

    def _keep(self):
        return bool(self.attrs.get("keep_dims", False))

    def out_shapes(self):
        x = list(self.in_shapes[0])
        if self.drops_axis:
            ax = self._axis()
            x = x[:ax] + ([1] if self._keep() else []) + x[ax + 1:]
        return [tuple(x)] * self.n_outputs

    def infer_outputs_tensor_map(self):
        m = list(self.inputs_tensor_map[0])
        if self.drops_axis:
            ax = self._axis()
            m = m[:ax] + ([-1] if self._keep() else []) + m[ax + 1:]
        return [list(m) for _ in range(self.n_outputs)]


@register("CumSum", "CumProd", "Cummax", "Cummin", "L2Normalize", "ReverseV2", "Sort", "LogSoftmaxExt")
class CumSumInfo(_WholeAxisInfo):
    def __init__(self, *a, **k):
        super().__init__(*a, **k)

    @property
    def n_outputs(self):          # Sort / Cummax / Cummin return (values, indices)
        return 2 if self.prim_name in ("Sort", "Cummax", "Cummin") else 1


@register("TopK", "TopkExt")
class TopKInfo(_WholeAxisInfo):
    n_outputs = 2

    def _axis(self):
        return len(self.in_shapes[0]) - 1

    def out_shapes(self):
        x = list(self.in_shapes[0])
        x[-1] = int(self.extra.get("k", x[-1]))
        return [tuple(x), tuple(x)]


@register("ArgMaxWithValue", "ArgMinWithValue", "Argmax", "Argmin")
class ArgExtremumInfo(_WholeAxisInfo):
    drops_axis = True

    @property
    def n_outputs(self):
        return 2 if self.prim_name.endswith("WithValue") else 1

    def _axis(self):
        return _norm_axis(self.attrs.get("axis", -1 if self.prim_name in ("Argmax", "Argmin") else 0),
                          len(self.in_shapes[0]))


@register("GatherD")
class GatherDInfo(OperatorInfo):
    """x, index alike in rank; the gather dim stays whole, the others are split alike."""

    def __init__(self, prim, in_shapes, in_strategy, out_strategy=None, stage_devices=1, attrs=None, dim=0, **_):
        self.dim = _norm_axis(dim, len(in_shapes[0]))
        super().__init__(prim, in_shapes[:2], in_strategy[:2], out_strategy, stage_devices, attrs)

    def check_strategy(self):
        OperatorInfo.check_strategy(self)
        if self.in_strategy[0] != self.in_strategy[1] or self.in_strategy[0][self.dim] != 1:
            raise StrategyError("GatherD: x and index must be split alike with the gather dim whole")

    def used_devices(self):
        return int(np.prod(self.in_strategy[0]))

    def base_dev_matrix(self):
        return list(self.in_strategy[0])

    def infer_inputs_tensor_map(self):
        m = [self._k(i) if s > 1 else -1 for i, s in enumerate(self.in_strategy[0])]
        return [m, list(m)]

    def out_shapes(self):
        return [self.in_shapes[1]]

    def infer_outputs_tensor_map(self):
        return [list(self.inputs_tensor_map[1])]


@register("UnsortedSegmentSum", "UnsortedSegmentProd")
class UnsortedSegmentSumInfo(OperatorInfo):
    """x [ids dims..., rest...], segment_ids [ids dims...] -> [num_segments, rest...].  The id dims of both are split
    alike: every rank sums its part of the rows, the partial results are all-reduced; trailing dims split freely."""

    def __init__(self, prim, in_shapes, in_strategy, out_strategy=None, stage_devices=1, attrs=None,
                 num_segments=None, **_):
        self.num_segments = int(num_segments)
        super().__init__(prim, in_shapes[:2], in_strategy[:2], out_strategy, stage_devices, attrs)

    def check_strategy(self):
        OperatorInfo.check_strategy(self)
        sx, si = self.in_strategy
        if tuple(sx[:len(si)]) != tuple(si):
            raise StrategyError("%s: the id dims of x and segment_ids must be split alike" % self.prim_name)
        if self.prim_name.endswith("Prod") and any(s > 1 for s in si):
            raise StrategyError("UnsortedSegmentProd: the id dims can not be split")

    def used_devices(self):
        return int(np.prod(self.in_strategy[0]))

    def base_dev_matrix(self):
        return list(self.in_strategy[0])

    def infer_inputs_tensor_map(self):
        m = [self._k(i) if s > 1 else -1 for i, s in enumerate(self.in_strategy[0])]
        return [m, m[:len(self.in_shapes[1])]]

    def out_shapes(self):
        return [(self.num_segments,) + tuple(self.in_shapes[0][len(self.in_shapes[1]):])]

    def infer_outputs_tensor_map(self):
        return [[-1] + list(self.inputs_tensor_map[0][len(self.in_shapes[1]):])]

    def infer_forward_comm(self):
        dims = [k for k in self.inputs_tensor_map[1] if k != -1]
        self.forward_comm = ("AllReduce", dims) if dims else None


@register("Pad", "PadV3", "MirrorPad")
class PadInfo(_SingleInputInfo):
    """attr paddings ((before, after) per dim): a padded dim stays whole."""

    def _padded(self):
        p = self.attrs.get("paddings", self.extra.get("paddings"))
        x = self.in_shapes[0]
        if p is None:
            return list(range(len(x)))
        p = list(p)
        if p and isinstance(p[0], (tuple, list)):
            return [i for i, (a, b) in enumerate(p) if a or b]
        # flat, last dim first (PadV3)
        out = []
        for j in range(len(p) // 2):
            if p[2 * j] or p[2 * j + 1]:
                out.append(len(x) - 1 - j)
        return out

    def check_strategy(self):
        OperatorInfo.check_strategy(self)
        self._whole(self._padded(), "a padded dim")

    def out_shapes(self):
        return [None]
