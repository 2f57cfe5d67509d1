"""Distributed semantics of primitives (``OperatorInfo``).

Given the shard strategy of a primitive (one tuple of split counts per input) an OperatorInfo derives

* the operator's device matrix (strategy dims, plus a leading "repeat" dim when the strategy uses fewer devices
  than the stage has - repeated calculation),
* the tensor map of every input and output,
* the forward communication (AllReduce over the device dims of a split contraction / reduction axis, or
  ReduceScatter for a row-parallel MatMul whose ``out_strategy`` row-shards the output),
* whether and by how much the loss must be divided when the op is the loss (``as_loss_divisor``),
* candidate strategies for the search.

Infos are registered by primitive name; a primitive without an info behaves as ``BatchParallel`` (split dim 0 of
everything by the device count) when possible, else ``StandAlone``.

Parity: ccsrc/frontend/parallel/ops_info/operator_info.h:119-330, operator_info.cc:425-548,654-749,1297-1557;
matmul_info.cc:290-403,839-910; activation_info.cc, arithmetic_info.cc, reduce_method_info.cc, loss_info.cc,
layer_norm_info.cc, gather_info.cc, onehot_info.cc, transpose_info.cc, reshape_info.cc, batch_parallel_info.cc.
"""
from __future__ import annotations

import itertools

import numpy as np

from .layout import TensorLayout

_REGISTRY = {}


def register(*names):
    def deco(cls):
        for n in names:
            _REGISTRY[n] = cls
        return cls
    return deco


def get_info_class(prim_name):
    return _REGISTRY.get(prim_name)


def registered_names():
    return sorted(_REGISTRY)


class StrategyError(ValueError):
    pass


class OperatorInfo:
    """Base: elementwise semantics over broadcast-compatible inputs."""

    def __init__(self, prim, in_shapes, in_strategy, out_strategy=None, stage_devices=1, attrs=None):
        self.prim_name = prim if isinstance(prim, str) else prim.name
        self.attrs = attrs if attrs is not None else (getattr(prim, "attrs", {}) if not isinstance(prim, str) else {})
        self.in_shapes = [tuple(s) for s in in_shapes]
        self.in_strategy = tuple(tuple(s) for s in in_strategy)
        self.out_strategy = out_strategy
        self.stage_devices = stage_devices
        self.forward_comm = None      # None | ("AllReduce", [dev dims]) | ("ReduceScatter", [dev dims], tensor_dim)
        self.check_strategy()
        self.dev_matrix = self.infer_dev_matrix()
        self._apply_repeat()
        self.inputs_tensor_map = self.infer_inputs_tensor_map()
        self.outputs_tensor_map = self.infer_outputs_tensor_map()
        self.infer_forward_comm()

    # ---- checks
    def check_strategy(self):
        if len(self.in_strategy) != len(self.in_shapes):
            raise StrategyError("%s: strategy has %d entries for %d inputs" % (self.prim_name, len(self.in_strategy),
                                                                              len(self.in_shapes)))
        for st, sh in zip(self.in_strategy, self.in_shapes):
            if len(st) != len(sh):
                raise StrategyError("%s: strategy %s does not match input rank %d" % (self.prim_name, st, len(sh)))
            for s, d in zip(st, sh):
                if s < 1 or d % s:
                    raise StrategyError("%s: dim of size %d can not be split %d ways" % (self.prim_name, d, s))
        prod = self.used_devices()
        if prod > self.stage_devices or self.stage_devices % prod:
            raise StrategyError("%s: strategy %s uses %d devices, the stage has %d" % (self.prim_name,
                                                                                      self.in_strategy, prod,
                                                                                      self.stage_devices))

    def used_devices(self):
        return int(np.prod(self.base_dev_matrix())) if self.base_dev_matrix() else 1

    # ---- device matrix
    def base_dev_matrix(self):
        """Elementwise: per output dim, the (common) split count of the inputs."""
        rank = max((len(s) for s in self.in_shapes), default=0)
        dm = [1] * rank
        for st, sh in zip(self.in_strategy, self.in_shapes):
            off = rank - len(sh)
            for i, (s, d) in enumerate(zip(st, sh)):
                if d == 1 and s == 1:
                    continue
                if dm[off + i] not in (1, s) and s != 1:
                    raise StrategyError("%s: inputs disagree on the split of dim %d" % (self.prim_name, off + i))
                dm[off + i] = max(dm[off + i], s)
        return dm

    def infer_dev_matrix(self):
        return list(self.base_dev_matrix())

    def _apply_repeat(self):
        prod = int(np.prod(self.dev_matrix)) if self.dev_matrix else 1
        self.repeat = self.stage_devices // max(prod, 1)
        self.repeat_left = True
        if self.repeat > 1:
            # the reference appends the repeat factor on the right by default; we put it on the left so that the
            # ranks of one replica group are strided and the maps below stay valid (repeated_num_in_dev_matrix_right
            # = False in the reference's terms)
            self.dev_matrix = [self.repeat] + self.dev_matrix

    def _k(self, base_index):
        """tensor-map value of base device-matrix position ``base_index`` (counted from the left)."""
        n = len(self.dev_matrix)
        off = 1 if self.repeat > 1 else 0
        return n - 1 - (base_index + off)

    # ---- tensor maps
    def infer_inputs_tensor_map(self):
        rank = max((len(s) for s in self.in_shapes), default=0)
        maps = []
        for st, sh in zip(self.in_strategy, self.in_shapes):
            off = rank - len(sh)
            maps.append([self._k(off + i) if s > 1 else -1 for i, s in enumerate(st)])
        return maps

    def out_shapes(self):
        rank = max((len(s) for s in self.in_shapes), default=0)
        out = [1] * rank
        for sh in self.in_shapes:
            off = rank - len(sh)
            for i, d in enumerate(sh):
                out[off + i] = max(out[off + i], d)
        return [tuple(out)]

    def infer_outputs_tensor_map(self):
        base = self.base_dev_matrix()
        return [[self._k(i) if s > 1 else -1 for i, s in enumerate(base)]]

    def infer_forward_comm(self):
        self.forward_comm = None

    # ---- results
    def input_layouts(self):
        return [TensorLayout(self.dev_matrix, m, s) for m, s in zip(self.inputs_tensor_map, self.in_shapes)]

    def output_layouts(self, local_shapes=None):
        """Layouts of the outputs.  An operator that can not tell an output's extents from its attributes returns
        None for that shape; the layout is then rebuilt from the shape of the local result (``local_shapes``)."""
        lays = []
        for i, (m, s) in enumerate(zip(self.outputs_tensor_map, self.out_shapes())):
            if s is None:
                if local_shapes is None or i >= len(local_shapes):
                    raise StrategyError("%s: the output shape is only known after running the local operator"
                                        % self.prim_name)
                dm = self.dev_matrix
                s = tuple(int(d) * (dm[len(dm) - 1 - k] if k != -1 else 1) for d, k in zip(local_shapes[i], m))
            lays.append(TensorLayout(self.dev_matrix, m, s))
        return lays

    def as_loss_divisor(self):
        """Number of ranks holding the same output slice: the loss gradient is divided by it (_VirtualDiv)."""
        return self.output_layouts()[0].repeat_num()

    def local_attrs(self):
        """Attribute / argument adjustments needed when the op runs on slices (e.g. Reshape target shape)."""
        return {}

    def localize_args(self, others):
        """Non-tensor call arguments as the local operator must see them (slice ends, tile multiples ...)."""
        return list(others)

    # ---- search
    @classmethod
    def generate_strategies(cls, in_shapes, device_num):
        """Default candidates: replicate, or split the batch dim of every input."""
        cands = [tuple(tuple(1 for _ in s) for s in in_shapes)]
        if in_shapes and all(len(s) > 0 and s[0] % device_num == 0 for s in in_shapes):
            cands.append(tuple(tuple([device_num] + [1] * (len(s) - 1)) for s in in_shapes))
        return cands


def _elementwise_strategies(shape, device_num, limit=64):
    """Every way to split the dims of ``shape`` by divisors of ``device_num`` (product dividing ``device_num``)."""
    out = []

    def rec(i, cur, prod):
        if len(out) >= limit:
            return
        if i == len(shape):
            out.append(tuple(cur))
            return
        for d in _divisors(device_num):
            if prod * d > device_num or device_num % (prod * d) or shape[i] % d:
                continue
            rec(i + 1, cur + [d], prod * d)
    rec(0, [], 1)
    return out


@register("Add", "Sub", "Mul", "Div", "RealDiv", "Pow", "Maximum", "Minimum", "Equal", "NotEqual", "Greater",
          "GreaterEqual", "Less", "LessEqual", "LogicalAnd", "LogicalOr", "FloorDiv", "FloorMod", "Mod", "Atan2",
          "SquaredDifference", "Xdivy", "Xlogy", "BitwiseAnd", "BitwiseOr", "BitwiseXor", "Select", "MaskedFill",
          "AddN", "Lerp", "Addcmul", "Addcdiv", "TruncateDiv", "TruncateMod", "DivNoNan", "MulNoNan",
          "Hypot", "ApproximateEqual", "AddExt", "SubExt", "DivMod", "Gcd", "Igamma", "Igammac", "NextAfter",
          "LeftShift", "RightShift", "Betainc", "Assign", "AssignAdd", "AssignSub", "DropoutDoMask", "KLDivLoss",
          "SigmoidCrossEntropyWithLogits", "BinaryCrossEntropy", "SmoothL1Loss", "FakeQuantPerLayer",
          "InplaceAdd", "InplaceSub", "InplaceUpdate", "Zeta")
class ArithmeticInfo(OperatorInfo):
    @classmethod
    def generate_strategies(cls, in_shapes, device_num):
        if in_shapes and all(tuple(s) == tuple(in_shapes[0]) for s in in_shapes):
            return [tuple(st for _ in in_shapes) for st in _elementwise_strategies(in_shapes[0], device_num)]
        return super().generate_strategies(in_shapes, device_num)


@register("ReLU", "ReLU6", "Sigmoid", "Tanh", "GeLU", "FastGeLU", "SiLU", "Mish", "Softplus", "Softsign", "Abs",
          "Neg", "Exp", "Expm1", "Log", "Log1p", "Sqrt", "Rsqrt", "Square", "Sign", "Sin", "Cos", "Tan", "Asin", "ACos",
          "Atan", "Sinh", "Cosh", "Asinh", "Acosh", "Atanh", "Erf", "Erfc", "Erfinv", "Floor", "Ceil", "Round",
          "Trunc", "Rint", "Reciprocal", "Inv", "Invert", "LogicalNot", "IsFinite", "IsNan", "IsInf", "Cast",
          "OnesLike", "ZerosLike", "Identity", "StopGradient", "Elu", "LeakyReLU", "HSigmoid", "HSwish", "SeLU",
          "Dropout", "Lgamma", "Digamma", "BesselI0", "BesselI0e", "BesselI1", "BesselI1e", "Sinc", "Logit",
          "_VirtualDiv", "_VirtualOutput", "_MirrorOperator", "AShardIdentity", "Activation", "BesselJ0", "BesselJ1",
          "HShrink", "SoftShrink", "ClampScalar", "PopulationCount", "Quant", "QuantV2", "Dequant", "AntiQuant",
          "L2Loss", "FillV2", "VirtualOutput", "SelfDefineShard", "LinSpace", "LinSpaceExt", "Gamma")
class ActivationInfo(OperatorInfo):
    @classmethod
    def generate_strategies(cls, in_shapes, device_num):
        if len(in_shapes) == 1:
            return [(st,) for st in _elementwise_strategies(in_shapes[0], device_num)]
        return super().generate_strategies(in_shapes, device_num)


@register("MatMul", "BatchMatMul")
class MatMulInfo(OperatorInfo):
    """A [.., M, K] x B [.., K, N] (with transpose flags).  Device matrix [batch.., M, K, N]; a split K needs
    AllReduce of the partial products, or ReduceScatter when out_strategy row-shards the output."""

    def _flags(self):
        return bool(self.attrs.get("transpose_a", False)), bool(self.attrs.get("transpose_b", False))

    def _mkn(self):
        ta, tb = self._flags()
        sa, sb = self.in_strategy
        m, k = (sa[-1], sa[-2]) if ta else (sa[-2], sa[-1])
        kb, n = (sb[-1], sb[-2]) if tb else (sb[-2], sb[-1])
        if k != kb:
            raise StrategyError("%s: the contraction dim is split %d ways in A but %d in B" % (self.prim_name, k, kb))
        return m, k, n

    def base_dev_matrix(self):
        sa, sb = self.in_strategy
        batch = list(sa[:-2])
        if len(sb) > 2 and list(sb[:-2])[-len(batch):] != batch[-(len(sb) - 2):] and any(x > 1 for x in sb[:-2]):
            raise StrategyError("%s: batch dims of A and B are split differently" % self.prim_name)
        m, k, n = self._mkn()
        return batch + [m, k, n]

    def infer_inputs_tensor_map(self):
        ta, tb = self._flags()
        sa, sb = self.in_strategy
        nb = len(sa) - 2
        bm = [self._k(i) if sa[i] > 1 else -1 for i in range(nb)]
        m, k, n = self._mkn()
        km, kk, kn = (self._k(nb) if m > 1 else -1), (self._k(nb + 1) if k > 1 else -1), (self._k(nb + 2) if n > 1 else -1)
        a_map = bm + ([kk, km] if ta else [km, kk])
        nbb = len(sb) - 2
        bmb = [(self._k(nb - nbb + i) if sb[i] > 1 else -1) for i in range(nbb)]
        b_map = bmb + ([kn, kk] if tb else [kk, kn])
        return [a_map, b_map]

    def out_shapes(self):
        ta, tb = self._flags()
        a, b = self.in_shapes
        m = a[-1] if ta else a[-2]
        n = b[-2] if tb else b[-1]
        return [tuple(a[:-2]) + (m, n)]

    def infer_outputs_tensor_map(self):
        sa, _ = self.in_strategy
        nb = len(sa) - 2
        m, k, n = self._mkn()
        out = [self._k(i) if sa[i] > 1 else -1 for i in range(nb)]
        km, kn = (self._k(nb) if m > 1 else -1), (self._k(nb + 2) if n > 1 else -1)
        if self._reduce_scatter():
            # rows additionally sharded over the contraction devices: (M axis, K axis) both map to the row dim
            kk = self._k(nb + 1)
            return [out + [(km, kk) if km != -1 else kk, kn]]
        return [out + [km, kn]]

    def _reduce_scatter(self):
        m, k, n = self._mkn()
        if k == 1 or not self.out_strategy:
            return False
        os_ = tuple(self.out_strategy[0])
        return os_[-2] == m * k and os_[-1] == n

    def infer_forward_comm(self):
        m, k, n = self._mkn()
        if k == 1:
            self.forward_comm = None
            return
        nb = len(self.in_strategy[0]) - 2
        kk = self._k(nb + 1)
        if self._reduce_scatter():
            self.forward_comm = ("ReduceScatter", [kk], len(self.out_shapes()[0]) - 2)
        else:
            if self.out_strategy:
                os_ = tuple(self.out_strategy[0])
                if os_[-2] != m or os_[-1] != n:
                    raise StrategyError("%s: out_strategy %s is neither the AllReduce layout (%d, %d) nor the "
                                        "ReduceScatter layout (%d, %d)" % (self.prim_name, os_, m, n, m * k, n))
            self.forward_comm = ("AllReduce", [kk])

    @classmethod
    def generate_strategies(cls, in_shapes, device_num, transpose_b=False):
        a, b = in_shapes
        cands = []
        m, k = a[-2], a[-1]
        n = b[-2] if transpose_b else b[-1]
        for dm, dk, dn in itertools.product(_divisors(device_num), repeat=3):
            if dm * dk * dn > device_num or device_num % (dm * dk * dn):
                continue
            if m % dm or k % dk or n % dn:
                continue
            sa = tuple([1] * (len(a) - 2) + [dm, dk])
            sb = tuple([1] * (len(b) - 2) + ([dn, dk] if transpose_b else [dk, dn]))
            cands.append((sa, sb))
        return cands


def _divisors(n):
    return [d for d in range(1, n + 1) if n % d == 0]


class _AxisOpInfo(OperatorInfo):
    """Single-input ops with a special axis that must stay unsplit (or triggers a reduction)."""

    def axis(self):
        raise NotImplementedError

    def base_dev_matrix(self):
        return list(self.in_strategy[0])

    def infer_inputs_tensor_map(self):
        maps = [[self._k(i) if s > 1 else -1 for i, s in enumerate(self.in_strategy[0])]]
        for st in self.in_strategy[1:]:
            maps.append([-1] * len(st))
        return maps

    def out_shapes(self):
        return [self.in_shapes[0]]

    def infer_outputs_tensor_map(self):
        return [list(self.inputs_tensor_map[0])]


@register("Softmax", "LogSoftmax")
class SoftmaxInfo(_AxisOpInfo):
    def check_strategy(self):
        super().check_strategy()
        ax = self.attrs.get("axis", -1)
        ax = ax[0] if isinstance(ax, (tuple, list)) else ax
        if self.in_strategy[0][ax] != 1:
            raise StrategyError("%s: the softmax axis can not be split" % self.prim_name)


@register("LayerNorm", "RmsNorm")
class NormInfo(_AxisOpInfo):
    def check_strategy(self):
        OperatorInfo.check_strategy(self)
        begin = self.attrs.get("begin_norm_axis", -1) % len(self.in_shapes[0])
        if any(s != 1 for s in self.in_strategy[0][begin:]):
            raise StrategyError("%s: normalised dims can not be split" % self.prim_name)
        for st in self.in_strategy[1:]:
            if any(s != 1 for s in st):
                raise StrategyError("%s: gamma / beta can not be split" % self.prim_name)

    def used_devices(self):
        return int(np.prod(self.in_strategy[0]))

    def out_shapes(self):
        x = self.in_shapes[0]
        if self.prim_name == "LayerNorm":
            begin = self.attrs.get("begin_norm_axis", -1) % len(x)
            stat = tuple(x[:begin]) + (1,) * (len(x) - begin)
            return [x, stat, stat]
        return [x, tuple(x[:-1]) + (1,)]

    def infer_outputs_tensor_map(self):
        m = list(self.inputs_tensor_map[0])
        outs = [m]
        for sh in self.out_shapes()[1:]:
            outs.append([m[i] if sh[i] != 1 else -1 for i in range(len(sh))])
        return outs


@register("AddRmsNorm")
class AddRmsNormInfo(OperatorInfo):
    """(x, residual, gamma) -> (y, x + residual): x and the residual share one strategy whose normalised (last) dim
    is whole; gamma is replicated, so under sequence parallelism its gradient is a partial sum per rank (mirror)."""

    def check_strategy(self):
        OperatorInfo.check_strategy(self)
        if self.in_strategy[0] != self.in_strategy[1]:
            raise StrategyError("AddRmsNorm: x and the residual must be split alike, got %s / %s"
                                % (self.in_strategy[0], self.in_strategy[1]))
        if self.in_strategy[0][-1] != 1 or any(s != 1 for s in self.in_strategy[2]):
            raise StrategyError("AddRmsNorm: the normalised dim and gamma can not be split")

    def used_devices(self):
        return int(np.prod(self.in_strategy[0]))

    def base_dev_matrix(self):
        return list(self.in_strategy[0])

    def infer_inputs_tensor_map(self):
        m = [self._k(i) if s > 1 else -1 for i, s in enumerate(self.in_strategy[0])]
        return [m, list(m), [-1] * len(self.in_shapes[2])]

    def out_shapes(self):
        return [self.in_shapes[0], self.in_shapes[0]]

    def infer_outputs_tensor_map(self):
        m = list(self.inputs_tensor_map[0])
        return [m, list(m)]


class _PackedLastDimInfo(OperatorInfo):
    """Ops on a last dim packed in ``groups`` blocks (``ops/llm_ops.py``): that dim may be split by a divisor of
    ``groups``; each rank then runs the op with ``groups / split`` blocks."""

    def _groups(self):
        return int(self.attrs.get("groups", 1))

    def check_strategy(self):
        OperatorInfo.check_strategy(self)
        s = self.in_strategy[0][-1]
        if self._groups() % s:
            raise StrategyError("%s: the packed dim holds %d groups and can not be split %d ways"
                                % (self.prim_name, self._groups(), s))
        for st in self.in_strategy[1:]:
            if any(x != 1 for x in st):
                raise StrategyError("%s: only the first input can be split" % self.prim_name)

    def used_devices(self):
        return int(np.prod(self.in_strategy[0]))

    def base_dev_matrix(self):
        return list(self.in_strategy[0])

    def infer_inputs_tensor_map(self):
        maps = [[self._k(i) if s > 1 else -1 for i, s in enumerate(self.in_strategy[0])]]
        for sh in self.in_shapes[1:]:
            maps.append([-1] * len(sh))
        return maps

    def infer_outputs_tensor_map(self):
        return [list(self.inputs_tensor_map[0])]

    def local_attrs(self):
        return {"groups": self._groups() // self.in_strategy[0][-1]}


@register("SwiGLU")
class SwiGLUInfo(_PackedLastDimInfo):
    def out_shapes(self):
        x = self.in_shapes[0]
        return [tuple(x[:-1]) + (x[-1] // 2,)]


@register("RotaryFlashAttention")
class RotaryFlashAttentionInfo(_PackedLastDimInfo):
    """qkv [tokens, (H + 2 Hk) * D] split (t, g): heads over ``g`` ranks (g divides ``groups``); a split token dim
    must keep whole sequences on a rank (batch split), i.e. tokens / t is a multiple of ``seq_length``."""

    def check_strategy(self):
        super().check_strategy()
        t = self.in_strategy[0][0]
        seq = int(self.in_shapes[1][0]) if len(self.in_shapes) > 1 else 1
        if t > 1 and (self.in_shapes[0][0] // t) % seq:
            raise StrategyError("RotaryFlashAttention: a token split of %d would cut sequences of %d tokens" % (t, seq))

    def out_shapes(self):
        a = self.attrs
        return [(self.in_shapes[0][0], int(a["head_num"]) * int(a["head_dim"]))]

    def local_attrs(self):
        g = self.in_strategy[0][-1]
        a = self.attrs
        return {"groups": self._groups() // g, "head_num": int(a["head_num"]) // g,
                "kv_head_num": int(a["kv_head_num"]) // g}


@register("ReduceSum", "ReduceMean", "ReduceMax", "ReduceMin", "ReduceAll", "ReduceAny", "ReduceProd")
class ReduceInfo(_AxisOpInfo):
    def __init__(self, prim, in_shapes, in_strategy, out_strategy=None, stage_devices=1, attrs=None, axis=()):
        self._axis = axis
        super().__init__(prim, in_shapes[:1], in_strategy[:1], out_strategy, stage_devices, attrs)

    def _axes(self):
        ax = self._axis
        rank = len(self.in_shapes[0])
        if ax is None or ax == ():
            return list(range(rank))
        ax = [ax] if isinstance(ax, int) else list(ax)
        return [a % rank for a in ax]

    def out_shapes(self):
        keep = bool(self.attrs.get("keep_dims", False))
        axes = self._axes()
        out = []
        for i, d in enumerate(self.in_shapes[0]):
            if i in axes:
                if keep:
                    out.append(1)
            else:
                out.append(d)
        return [tuple(out)]

    def infer_outputs_tensor_map(self):
        keep = bool(self.attrs.get("keep_dims", False))
        axes = self._axes()
        out = []
        for i, m in enumerate(self.inputs_tensor_map[0]):
            if i in axes:
                if keep:
                    out.append(-1)
            else:
                out.append(m)
        return [out]

    def infer_forward_comm(self):
        dims = [self.inputs_tensor_map[0][a] for a in self._axes() if self.inputs_tensor_map[0][a] != -1]
        if not dims:
            self.forward_comm = None
        elif self.prim_name in ("ReduceSum", "ReduceMean"):
            self.forward_comm = ("AllReduce", dims) if self.prim_name == "ReduceSum" else ("AllReduceMean", dims)
        elif self.prim_name in ("ReduceMax", "ReduceMin"):
            self.forward_comm = ("AllReduce" + self.prim_name[6:], dims)
        else:
            raise StrategyError("%s: the reduced axis can not be split" % self.prim_name)


@register("Transpose")
class TransposeInfo(_AxisOpInfo):
    def __init__(self, prim, in_shapes, in_strategy, out_strategy=None, stage_devices=1, attrs=None, perm=None):
        self.perm = tuple(perm) if perm is not None else tuple(reversed(range(len(in_shapes[0]))))
        super().__init__(prim, in_shapes[:1], in_strategy[:1], out_strategy, stage_devices, attrs)

    def out_shapes(self):
        return [tuple(self.in_shapes[0][p] for p in self.perm)]

    def infer_outputs_tensor_map(self):
        return [[self.inputs_tensor_map[0][p] for p in self.perm]]


@register("Reshape")
class ReshapeInfo(_AxisOpInfo):
    """Reshape keeps a split only on a leading dim that survives in the target shape; the local target shape is
    the global one divided by the same factor."""

    def __init__(self, prim, in_shapes, in_strategy, out_strategy=None, stage_devices=1, attrs=None, shape=None):
        self.target = tuple(int(s) for s in shape)
        total = int(np.prod(in_shapes[0]))
        if -1 in self.target:
            known = -int(np.prod(self.target))
            self.target = tuple(total // known if s == -1 else s for s in self.target)
        super().__init__(prim, in_shapes[:1], in_strategy[:1], out_strategy, stage_devices, attrs)

    def check_strategy(self):
        OperatorInfo.check_strategy(self)
        st = self.in_strategy[0]
        if any(s != 1 for s in st[1:]):
            raise StrategyError("Reshape: only the first dim may be split (got %s); redistribute first" % (st,))
        if st and st[0] > 1 and self.target[0] % st[0]:
            raise StrategyError("Reshape: target dim 0 (%d) is not divisible by the split %d" % (self.target[0], st[0]))

    def out_shapes(self):
        return [self.target]

    def infer_outputs_tensor_map(self):
        m0 = self.inputs_tensor_map[0][0] if self.inputs_tensor_map[0] else -1
        return [[m0] + [-1] * (len(self.target) - 1)]

    def local_attrs(self):
        s = self.in_strategy[0][0] if self.in_strategy[0] else 1
        return {"shape": (self.target[0] // s,) + tuple(self.target[1:])}


@register("Gather", "EmbeddingLookup", "SparseGatherV2")
class GatherInfo(OperatorInfo):
    """params [V, H] with strategy (v, h), indices replicated or batch-split: a split vocabulary needs a range mask
    and AllReduce of the partial lookups."""

    def __init__(self, prim, in_shapes, in_strategy, out_strategy=None, stage_devices=1, attrs=None, axis=0):
        self.axis_ = int(axis)
        super().__init__(prim, in_shapes[:2], in_strategy[:2], out_strategy, stage_devices, attrs)

    def check_strategy(self):
        if self.axis_ != 0:
            for s in self.in_strategy[0]:
                if s != 1:
                    raise StrategyError("Gather: only axis 0 tables can be split")
        for st, sh in zip(self.in_strategy, self.in_shapes):
            for s, d in zip(st, sh):
                if d % s:
                    raise StrategyError("Gather: dim %d not divisible by %d" % (d, s))

    def base_dev_matrix(self):
        p, i = self.in_strategy
        return list(i) + list(p)           # [index dims..., vocab, hidden...]

    def infer_inputs_tensor_map(self):
        p, i = self.in_strategy
        ni = len(i)
        return [[self._k(ni + t) if s > 1 else -1 for t, s in enumerate(p)],
                [self._k(t) if s > 1 else -1 for t, s in enumerate(i)]]

    def out_shapes(self):
        p, i = self.in_shapes
        return [tuple(i) + tuple(p[1:])]

    def _reduce_scatter(self):
        """out_strategy whose dim 0 is split by the vocabulary split: the partial lookups are reduce-scattered over
        the index rows instead of all-reduced (sequence parallelism starts at the embedding)."""
        p, i = self.in_strategy
        if p[0] == 1 or not self.out_strategy or len(i) != 1 or i[0] != 1:
            return False
        os_ = tuple(self.out_strategy[0])
        return os_[0] == p[0] and all(x == 1 for x in os_[1:]) and self.in_shapes[1][0] % p[0] == 0

    def infer_outputs_tensor_map(self):
        p, i = self.in_strategy
        ni = len(i)
        if self._reduce_scatter():
            return [[self._k(ni)] + [-1] * (len(p) - 1)]
        return [[self._k(t) if s > 1 else -1 for t, s in enumerate(i)] +
                [self._k(ni + 1 + t) if s > 1 else -1 for t, s in enumerate(p[1:])]]

    def infer_forward_comm(self):
        p, i = self.in_strategy
        if p[0] == 1:
            self.forward_comm = None
        elif self._reduce_scatter():
            self.forward_comm = ("ReduceScatter", [self._k(len(i))], 0)
        else:
            self.forward_comm = ("AllReduce", [self._k(len(i))])

    def vocab_split(self):
        return self.in_strategy[0][0]


@register("OneHot")
class OneHotInfo(OperatorInfo):
    def __init__(self, prim, in_shapes, in_strategy, out_strategy=None, stage_devices=1, attrs=None, depth=None):
        self.depth = depth
        idx_st = tuple(in_strategy[0][:len(in_shapes[0])]) if in_strategy else ()
        self.class_split = in_strategy[0][len(in_shapes[0])] if len(in_strategy[0]) > len(in_shapes[0]) else 1
        super().__init__(prim, in_shapes[:1], (idx_st,), out_strategy, stage_devices, attrs)

    def base_dev_matrix(self):
        return list(self.in_strategy[0]) + [self.class_split]

    def infer_inputs_tensor_map(self):
        return [[self._k(i) if s > 1 else -1 for i, s in enumerate(self.in_strategy[0])]]

    def out_shapes(self):
        return [tuple(self.in_shapes[0]) + (int(self.depth),)]

    def infer_outputs_tensor_map(self):
        n = len(self.in_strategy[0])
        return [list(self.inputs_tensor_map[0]) + [self._k(n) if self.class_split > 1 else -1]]


@register("SoftmaxCrossEntropyWithLogits", "SparseSoftmaxCrossEntropyWithLogits")
class LossInfo(OperatorInfo):
    """logits [B, C] split (b, c).  b > 1: batch-parallel loss, the mean is all-reduced.  c > 1 (sparse variant
    only): vocabulary-parallel loss - every rank reduces its class shard to (max, sum-exp, target logit), the three
    numbers per row are combined over the class group and each rank writes the gradient of its own shard; the
    scalar result is identical on the ranks of that group and its backward does not all-reduce, so those ranks do
    not count as repeats for the loss divisor."""

    def check_strategy(self):
        st = self.in_strategy[0]
        if st[-1] != 1 and not self.prim_name.startswith("Sparse"):
            raise StrategyError("%s: the class dim can not be split" % self.prim_name)
        if self.in_shapes[0][0] % st[0] or self.in_shapes[0][-1] % st[-1]:
            raise StrategyError("%s: logits %s are not divisible by %s" % (self.prim_name, self.in_shapes[0], st))
        if st[0] * st[-1] > self.stage_devices or self.stage_devices % (st[0] * st[-1]):
            raise StrategyError("%s: strategy %s does not fit %d devices" % (self.prim_name, st, self.stage_devices))

    def class_split(self):
        return int(self.in_strategy[0][-1])

    def used_devices(self):
        return int(self.in_strategy[0][0]) * self.class_split()

    def base_dev_matrix(self):
        return [self.in_strategy[0][0], self.class_split()]

    def infer_inputs_tensor_map(self):
        b = self._k(0) if self.in_strategy[0][0] > 1 else -1
        c = self._k(1) if self.class_split() > 1 else -1
        maps = [[b, c]]
        for sh in self.in_shapes[1:]:
            maps.append([b] + [-1] * (len(sh) - 1))
        return maps

    def out_shapes(self):
        if self.prim_name.startswith("Sparse"):
            return [()]
        return [(self.in_shapes[0][0],), self.in_shapes[0]]

    def infer_outputs_tensor_map(self):
        b = self.inputs_tensor_map[0][0]
        if self.prim_name.startswith("Sparse"):
            return [[]]
        return [[b], [b, -1]]

    def infer_forward_comm(self):
        if self.prim_name.startswith("Sparse") and self.in_strategy[0][0] > 1:
            self.forward_comm = ("AllReduceMean", [self._k(0)])

    def as_loss_divisor(self):
        return max(1, self.output_layouts()[0].repeat_num() // self.class_split())


@register("FlashAttentionScore")
class FlashAttentionInfo(OperatorInfo):
    """query/key/value in BSH: strategy (b, s, h) - batch and heads may be split; a split sequence needs the
    ring / context-parallel expansion (``parallel.context_parallel``)."""

    def __init__(self, prim, in_shapes, in_strategy, out_strategy=None, stage_devices=1, attrs=None):
        super().__init__(prim, in_shapes[:3], in_strategy[:3], out_strategy, stage_devices, attrs)

    def check_strategy(self):
        q, k, v = self.in_strategy
        if k != v or q[0] != k[0] or q[-1] != k[-1]:
            raise StrategyError("FlashAttentionScore: q/k/v strategies must agree on batch and hidden splits")
        head_num = self.attrs.get("head_num", 1)
        if head_num % q[-1]:
            raise StrategyError("FlashAttentionScore: head_num %d not divisible by %d" % (head_num, q[-1]))
        if len(q) == 3 and k[1] != 1 and not self.attrs.get("enable_ring_attention", False):
            raise StrategyError("FlashAttentionScore: key/value sequence split needs enable_ring_attention")

    def base_dev_matrix(self):
        return list(self.in_strategy[0])

    def infer_inputs_tensor_map(self):
        m = [self._k(i) if s > 1 else -1 for i, s in enumerate(self.in_strategy[0])]
        mk = [self._k(i) if s > 1 else -1 for i, s in enumerate(self.in_strategy[1])]
        return [m, mk, list(mk)]

    def out_shapes(self):
        return [self.in_shapes[0]]

    def infer_outputs_tensor_map(self):
        return [list(self.inputs_tensor_map[0])]

    def local_attrs(self):
        return {"head_num": self.attrs.get("head_num", 1) // self.in_strategy[0][-1]}


@register("BatchParallel", "_VirtualDataset", "GetNext", "Unique", "ApplyRotaryPosEmb", "VirtualDataset",
          "Conv3D", "Conv2DBackpropInput", "Conv2DTranspose", "GroupNorm",
          "LayerNormV3", "BatchMatMulExt", "MatMulExt", "BoundingBoxEncode", "BoundingBoxDecode", "CheckValid", "IOU",
          "Cdist", "Cholesky", "Custom", "DecoderKVCache",
          "PromptKVCache", "KVCacheMgr", "KVCacheScatterUpdate", "ReshapeAndCache", "PagedAttention",
          "PagedAttentionMask", "IncreFlashAttention", "PromptFlashAttention", "FusedInferAttentionScore",
          "DynamicQuantExt", "FFN", "FFNExt", "FakeQuantPerChannel", "MinMaxUpdatePerChannel", "MinMaxUpdatePerLayer",
          "GatherNd", "GenerateEodMask", "GroupedMatmul", "IndexSelect", "MoeFinalizeRouting", "OneHotExt", "QuantBatchMatmul", "WeightQuantBatchMatmul",
          "RandomChoiceWithMask", "RepeatElements", "ScatterAdd", "ScatterDiv", "ScatterMax", "ScatterMin",
          "ScatterMul", "ScatterSub", "ScatterUpdate", "ScatterNdAdd", "ScatterNdSub", "ScatterNdUpdate",
          "TensorScatterAdd", "TensorScatterDiv", "TensorScatterMax", "TensorScatterMin", "TensorScatterMul",
          "TensorScatterSub", "TensorScatterUpdate", "UnsortedSegmentMax", "UnsortedSegmentMin",
          "SumExt", "TensorDot", "UniformCandidateSampler", "WKV", "Range", "SquareSumAll", "TopKRouter", "Tril", "Triu", "UniformReal", "StandardNormal")
class BatchParallelInfo(OperatorInfo):
    """Dim 0 of every input and output is split by the strategy's first entry; other dims stay whole."""

    def check_strategy(self):
        OperatorInfo.check_strategy(self)
        for st in self.in_strategy:
            if any(s != 1 for s in st[1:]):
                raise StrategyError("%s: only the batch dim may be split (got %s)" % (self.prim_name, st))

    def used_devices(self):
        return max((st[0] for st in self.in_strategy if st), default=1)

    def base_dev_matrix(self):
        return [self.used_devices()]

    def infer_inputs_tensor_map(self):
        return [[(self._k(0) if st[0] > 1 else -1)] + [-1] * (len(st) - 1) if st else [] for st in self.in_strategy]

    def out_shapes(self):
        return [self.in_shapes[0]]

    def infer_outputs_tensor_map(self):
        return [list(self.inputs_tensor_map[0])]


@register("StandAlone")
class StandAloneInfo(OperatorInfo):
    def check_strategy(self):
        for st in self.in_strategy:
            if any(s != 1 for s in st):
                raise StrategyError("StandAlone ops can not be split")

    def used_devices(self):
        return 1

    def base_dev_matrix(self):
        return []

    def infer_inputs_tensor_map(self):
        return [[-1] * len(s) for s in self.in_shapes]

    def out_shapes(self):
        return [self.in_shapes[0]] if self.in_shapes else [()]

    def infer_outputs_tensor_map(self):
        return [[-1] * len(self.out_shapes()[0])]


def make_info(prim, in_shapes, in_strategy, out_strategy=None, stage_devices=1, **extra):
    cls = get_info_class(prim.name if not isinstance(prim, str) else prim)
    if cls is None:
        cls = BatchParallelInfo if all(all(s == 1 for s in st[1:]) for st in in_strategy) else None
        if cls is None:
            raise StrategyError("primitive %s has no distributed OperatorInfo and its strategy %s is not batch-parallel"
                                % (prim if isinstance(prim, str) else prim.name, in_strategy))
    return cls(prim, in_shapes, in_strategy, out_strategy, stage_devices, **extra)


from . import operator_info_ext  # noqa: E402,F401  (array / convolution / selection operators register themselves)
