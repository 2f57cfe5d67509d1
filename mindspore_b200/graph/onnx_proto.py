"""ONNX export: a traced forward graph as an ONNX ``ModelProto`` (opset 17).

The exporter works from the same primitive-level description that the MindIR writer produces (torch-level calls of
``nn`` layers already restated as primitives, weights as named tensors), so one lowering serves both formats: the
MindIR model is built in memory and every primitive node is then restated with ONNX operators.  Constants that a
primitive takes as operands (the target shape of ``Reshape``, the axes of a reduction, the permutation of
``Transpose``) become ONNX attributes or int64 initializers, whichever the ONNX operator wants; weights become
initializers; tuples (``MakeTuple`` / ``TupleGetItem``) are resolved at export time and never reach the file.

Parity: mindspore/ccsrc/transform/express_ir/onnx_exporter.cc (OpNameInfo table + the hand-written exporters for
Reshape / Reduce / Transpose / BatchNorm / MatMul with transposes / Conv pads ...), ``export(..., file_format="ONNX")``
in mindspore/python/mindspore/train/serialization.py.

The message classes are built at import time from a description of the public ONNX schema (onnx.proto: field names and
numbers), so neither the ``onnx`` package nor ``protoc`` is needed.
"""
from __future__ import annotations

import numpy as np
import torch

from .mindir import MindIRError

OPSET = 17

_SCHEMA = {
    "AttributeProto": [
        ("name", 1, "string"), ("f", 2, "float"), ("i", 3, "int64"), ("s", 4, "bytes"), ("t", 5, "TensorProto"),
        ("g", 6, "GraphProto"), ("floats", 7, "float*"), ("ints", 8, "int64*"), ("strings", 9, "bytes*"),
        ("tensors", 10, "TensorProto*"), ("graphs", 11, "GraphProto*"), ("doc_string", 13, "string"),
        ("type", 20, "enum"), ("ref_attr_name", 21, "string")],
    "ValueInfoProto": [("name", 1, "string"), ("type", 2, "TypeProto"), ("doc_string", 3, "string")],
    "NodeProto": [
        ("input", 1, "string*"), ("output", 2, "string*"), ("name", 3, "string"), ("op_type", 4, "string"),
        ("attribute", 5, "AttributeProto*"), ("doc_string", 6, "string"), ("domain", 7, "string")],
    "ModelProto": [
        ("ir_version", 1, "int64"), ("producer_name", 2, "string"), ("producer_version", 3, "string"),
        ("domain", 4, "string"), ("model_version", 5, "int64"), ("doc_string", 6, "string"),
        ("graph", 7, "GraphProto"), ("opset_import", 8, "OperatorSetIdProto*")],
    "OperatorSetIdProto": [("domain", 1, "string"), ("version", 2, "int64")],
    "GraphProto": [
        ("node", 1, "NodeProto*"), ("name", 2, "string"), ("initializer", 5, "TensorProto*"),
        ("doc_string", 10, "string"), ("input", 11, "ValueInfoProto*"), ("output", 12, "ValueInfoProto*"),
        ("value_info", 13, "ValueInfoProto*")],
    "TensorProto": [
        ("dims", 1, "int64*"), ("data_type", 2, "int32"), ("float_data", 4, "float*"), ("int32_data", 5, "int32*"),
        ("string_data", 6, "bytes*"), ("int64_data", 7, "int64*"), ("name", 8, "string"), ("raw_data", 9, "bytes"),
        ("double_data", 10, "double*"), ("uint64_data", 11, "uint64*"), ("doc_string", 12, "string")],
    "TypeProto": [("tensor_type", 1, "TypeProtoTensor"), ("denotation", 6, "string")],
    "TypeProtoTensor": [("elem_type", 1, "int32"), ("shape", 2, "TensorShapeProto")],
    "TensorShapeProto": [("dim", 1, "Dimension*")],
    "Dimension": [("dim_value", 1, "int64"), ("dim_param", 2, "string"), ("denotation", 3, "string")],
}

# AttributeProto.AttributeType
AT_FLOAT, AT_INT, AT_STRING, AT_TENSOR, AT_FLOATS, AT_INTS, AT_STRINGS = 1, 2, 3, 4, 6, 7, 8
# TensorProto.DataType
DT = {torch.float32: 1, torch.uint8: 2, torch.int8: 3, torch.int16: 5, torch.int32: 6, torch.int64: 7, torch.bool: 9,
      torch.float16: 10, torch.float64: 11, torch.bfloat16: 16}
DT_REV = {v: k for k, v in DT.items()}

_messages = None


def messages():
    """{message name: class} of the ONNX schema (package ``onnx``)."""
    global _messages
    if _messages is None:
        from .mindir_proto import build_messages
        _messages = build_messages(_SCHEMA, "onnx", "mindspore_b200/onnx.proto")
    return _messages


def _tensor_proto(tp, t, name):
    plain = t.detach().to("cpu").contiguous() if isinstance(t, torch.Tensor) else torch.as_tensor(np.asarray(t))
    if plain.dtype not in DT:
        raise MindIRError("tensor %s has dtype %s, which ONNX files do not carry" % (name, plain.dtype))
    tp.name = name
    tp.data_type = DT[plain.dtype]
    tp.dims.extend(int(d) for d in plain.shape)
    if plain.dtype == torch.bfloat16:
        tp.raw_data = plain.view(torch.int16).numpy().tobytes()
    else:
        tp.raw_data = plain.numpy().tobytes()


def read_tensor(tp):
    """An initializer / constant back as a torch tensor (``raw_data`` or the typed repeated fields)."""
    dtype = DT_REV[tp.data_type]
    shape = tuple(tp.dims)
    if tp.raw_data:
        if dtype == torch.bfloat16:
            return torch.from_numpy(np.frombuffer(tp.raw_data, np.int16).copy()).view(torch.bfloat16).reshape(shape)
        npdt = torch.empty(0, dtype=dtype).numpy().dtype
        return torch.from_numpy(np.frombuffer(tp.raw_data, npdt).copy()).reshape(shape)
    if tp.float_data:
        return torch.tensor(list(tp.float_data), dtype=dtype).reshape(shape)
    if tp.int64_data:
        return torch.tensor(list(tp.int64_data), dtype=dtype).reshape(shape)
    if tp.int32_data:
        return torch.tensor(list(tp.int32_data), dtype=dtype).reshape(shape)
    return torch.zeros(shape, dtype=dtype)


class _Tuple:
    """A MakeTuple result during export: the names of its elements."""

    def __init__(self, items):
        self.items = list(items)


class _Emitter:
    def __init__(self, graph):
        self.g = graph
        self.n = 0
        self.consts = {}          # MindIR name -> python value / tensor of a Constant node
        self.alias = {}           # MindIR name -> ONNX name (or _Tuple)
        self.shapes = {}          # ONNX name -> (shape, dtype) where the exporter knows it
        self._const_cache = {}

    def fresh(self, hint):
        self.n += 1
        return "%s_%d" % (hint, self.n)

    def node(self, op_type, inputs, n_out=1, **attrs):
        nd = self.g.node.add()
        nd.op_type = op_type
        nd.name = self.fresh(op_type)
        nd.input.extend(inputs)
        outs = [nd.name + ("" if k == 0 else "_o%d" % k) for k in range(n_out)]
        nd.output.extend(outs)
        for k, v in attrs.items():
            if v is None:
                continue
            ap = nd.attribute.add()
            ap.name = k
            if isinstance(v, bool):
                ap.type, ap.i = AT_INT, int(v)
            elif isinstance(v, int):
                ap.type, ap.i = AT_INT, v
            elif isinstance(v, float):
                ap.type, ap.f = AT_FLOAT, v
            elif isinstance(v, str):
                ap.type, ap.s = AT_STRING, v.encode()
            elif isinstance(v, torch.Tensor):
                ap.type = AT_TENSOR
                _tensor_proto(ap.t, v, "value")
            elif isinstance(v, (tuple, list)) and all(isinstance(x, int) and not isinstance(x, bool) for x in v):
                ap.type = AT_INTS
                ap.ints.extend(int(x) for x in v)
            elif isinstance(v, (tuple, list)) and all(isinstance(x, (int, float)) for x in v):
                ap.type = AT_FLOATS
                ap.floats.extend(float(x) for x in v)
            else:
                raise MindIRError("attribute %s=%r of %s has no ONNX form" % (k, v, op_type))
        return outs[0] if n_out == 1 else outs

    def initializer(self, value, hint="const"):
        t = value if isinstance(value, torch.Tensor) else torch.as_tensor(np.asarray(value))
        key = (str(t.dtype), tuple(t.shape), t.detach().cpu().numpy().tobytes()) if t.numel() <= 64 and \
            t.dtype != torch.bfloat16 else None
        if key is not None and key in self._const_cache:
            return self._const_cache[key]
        name = self.fresh(hint)
        _tensor_proto(self.g.initializer.add(), t, name)
        if key is not None:
            self._const_cache[key] = name
        return name

    def ints(self, values):
        return self.initializer(torch.tensor([int(v) for v in values], dtype=torch.int64), "ints")

    # -- operands of a MindIR node --
    def value(self, name):
        """The Python value of a constant operand, or None when the operand is computed at run time."""
        return self.consts.get(name)

    def is_const(self, name):
        return name in self.consts

    def tensor(self, name, like=None):
        """The ONNX name that holds a MindIR operand; constants are written as initializers (a Python scalar takes
        the dtype of ``like``, the ONNX name of the other operand, when that is known)."""
        if name in self.alias:
            out = self.alias[name]
            if isinstance(out, _Tuple):
                raise MindIRError("a tuple is used where a tensor is expected (%s)" % name)
            return out
        if name in self.consts:
            v = self.consts[name]
            if isinstance(v, torch.Tensor):
                t = v
            else:
                dtype = self.shapes.get(like, (None, None))[1] if like else None
                if dtype is None:
                    dtype = torch.float32 if isinstance(v, float) else torch.bool if isinstance(v, bool) else \
                        torch.int64
                t = torch.tensor(v, dtype=dtype)
            out = self.initializer(t)
            self.shapes[out] = (tuple(t.shape), t.dtype)
            return out
        raise MindIRError("operand %r is not defined" % name)


def _auto_pad(pad_mode):
    mode = str(pad_mode).lower()
    return {"same": "SAME_UPPER", "valid": "VALID"}.get(mode)


def _handlers():
    H = {}

    def reg(*names):
        def deco(fn):
            for n in names:
                H[n] = fn
            return fn
        return deco

    def simple(onnx_op):
        def h(e, ins, attrs):
            return e.node(onnx_op, [e.tensor(i) for i in ins])
        return h

    for ms_name, onnx_op in (("ReLU", "Relu"), ("Sigmoid", "Sigmoid"), ("Tanh", "Tanh"), ("Exp", "Exp"),
                             ("Log", "Log"), ("Sqrt", "Sqrt"), ("Neg", "Neg"), ("Abs", "Abs"), ("Erf", "Erf"),
                             ("Floor", "Floor"), ("Ceil", "Ceil"), ("Sin", "Sin"), ("Cos", "Cos"),
                             ("Reciprocal", "Reciprocal"), ("Identity", "Identity"), ("StopGradient", "Identity"),
                             ("Softplus", "Softplus"), ("Softsign", "Softsign"), ("Sign", "Sign"),
                             ("LogicalNot", "Not")):
        H[ms_name] = simple(onnx_op)

    def binary(onnx_op):
        def h(e, ins, attrs):
            # a Python scalar operand takes the dtype of the tensor operand
            if e.is_const(ins[0]) and not isinstance(e.value(ins[0]), torch.Tensor):
                b = e.tensor(ins[1])
                a = e.tensor(ins[0], like=b)
            else:
                a = e.tensor(ins[0])
                b = e.tensor(ins[1], like=a)
            return e.node(onnx_op, [a, b])
        return h

    for ms_name, onnx_op in (("Add", "Add"), ("Sub", "Sub"), ("Mul", "Mul"), ("RealDiv", "Div"), ("Div", "Div"),
                             ("Pow", "Pow"), ("Maximum", "Max"), ("Minimum", "Min"), ("Greater", "Greater"),
                             ("Less", "Less"), ("GreaterEqual", "GreaterOrEqual"), ("LessEqual", "LessOrEqual"),
                             ("Equal", "Equal"), ("LogicalAnd", "And"), ("LogicalOr", "Or")):
        H[ms_name] = binary(onnx_op)

    @reg("NotEqual")
    def not_equal(e, ins, attrs):
        return e.node("Not", [H["Equal"](e, ins, attrs)])

    @reg("SiLU")
    def silu(e, ins, attrs):
        x = e.tensor(ins[0])
        return e.node("Mul", [x, e.node("Sigmoid", [x])])

    @reg("GeLU")
    def gelu(e, ins, attrs):
        # 0.5 * x * (1 + erf(x / sqrt(2))): the Gelu operator itself arrives with opset 20
        x = e.tensor(ins[0])
        inv = e.initializer(torch.tensor(0.7071067811865476), "rsqrt2")
        half = e.initializer(torch.tensor(0.5), "half")
        one = e.initializer(torch.tensor(1.0), "one")
        erf = e.node("Erf", [e.node("Mul", [x, inv])])
        return e.node("Mul", [e.node("Mul", [x, half]), e.node("Add", [erf, one])])

    @reg("Softmax", "LogSoftmax")
    def softmax(e, ins, attrs):
        axis = attrs.get("axis", -1)
        axis = axis[0] if isinstance(axis, (tuple, list)) else axis
        return e.node(attrs["__op__"], [e.tensor(ins[0])], axis=int(axis))          # same names in ONNX

    @reg("Flatten")
    def flatten(e, ins, attrs):
        return e.node("Flatten", [e.tensor(ins[0])], axis=1)

    @reg("Reshape")
    def reshape(e, ins, attrs):
        shape = e.value(ins[1])
        target = e.ints(shape) if shape is not None else e.tensor(ins[1])
        return e.node("Reshape", [e.tensor(ins[0]), target])

    @reg("Transpose")
    def transpose(e, ins, attrs):
        perm = e.value(ins[1])
        if perm is None:
            raise MindIRError("Transpose needs a constant permutation")
        return e.node("Transpose", [e.tensor(ins[0])], perm=[int(p) for p in perm])

    @reg("MatMul", "BatchMatMul")
    def matmul(e, ins, attrs):
        a, b = e.tensor(ins[0]), e.tensor(ins[1])
        if attrs["__op__"] == "MatMul":
            ta, tb = bool(attrs.get("transpose_a", False)), bool(attrs.get("transpose_b", False))
            if ta or tb:
                return e.node("Gemm", [a, b], transA=int(ta), transB=int(tb))
            return e.node("MatMul", [a, b])
        for flag, which in (("transpose_a", 0), ("transpose_b", 1)):
            if attrs.get(flag, False) or attrs.get(flag.replace("transpose", "adj"), False):
                raise MindIRError("BatchMatMul with a transposed operand is not exported")
        return e.node("MatMul", [a, b])

    @reg("BiasAdd")
    def bias_add(e, ins, attrs):
        x, b = e.tensor(ins[0]), e.tensor(ins[1])
        rank = len(e.shapes[x][0]) if x in e.shapes else None
        if rank is not None and rank > 2:              # NCHW: the bias runs along axis 1
            b = e.node("Reshape", [b, e.ints([1, -1] + [1] * (rank - 2))])
        elif rank is None:
            raise MindIRError("BiasAdd on an operand of unknown rank is not exported")
        return e.node("Add", [x, b])

    @reg("Conv2D")
    def conv2d(e, ins, attrs):
        pad_mode = str(attrs.get("pad_mode", "valid")).lower()
        kw = {"kernel_shape": [int(k) for k in attrs["kernel_size"]], "group": int(attrs.get("group", 1)),
              "strides": [int(s) for s in tuple(attrs.get("stride", (1, 1, 1, 1)))[-2:]],
              "dilations": [int(s) for s in tuple(attrs.get("dilation", (1, 1, 1, 1)))[-2:]]}
        if pad_mode == "pad":
            t, b, l, r = [int(p) for p in attrs.get("pad", (0, 0, 0, 0))]
            kw["pads"] = [t, l, b, r]                  # ONNX order: begins of every axis, then ends
        else:
            kw["auto_pad"] = _auto_pad(pad_mode)
        return e.node("Conv", [e.tensor(i) for i in ins[:3]], **kw)

    def pooling(onnx_op):
        def h(e, ins, attrs):
            kw = {"kernel_shape": [int(k) for k in tuple(attrs["kernel_size"])[-2:]],
                  "strides": [int(s) for s in tuple(attrs["strides"])[-2:]],
                  "auto_pad": _auto_pad(attrs.get("pad_mode", "valid"))}
            return e.node(onnx_op, [e.tensor(ins[0])], **kw)
        return h
    H["MaxPool"] = pooling("MaxPool")
    H["AvgPool"] = pooling("AveragePool")

    @reg("BatchNorm")
    def batch_norm(e, ins, attrs):
        if attrs.get("is_training", False):
            raise MindIRError("training-mode BatchNorm is not exported")
        y = e.node("BatchNormalization", [e.tensor(i) for i in ins[:5]], epsilon=float(attrs.get("epsilon", 1e-5)))
        return _Tuple([y])

    @reg("LayerNorm")
    def layer_norm(e, ins, attrs):
        y = e.node("LayerNormalization", [e.tensor(i) for i in ins[:3]], axis=int(attrs.get("begin_norm_axis", -1)),
                   epsilon=float(attrs.get("epsilon", 1e-7)))
        return _Tuple([y])

    def reduction(onnx_op, axes_as_input):
        def h(e, ins, attrs):
            axes = e.value(ins[1]) if len(ins) > 1 else ()
            if axes is None and len(ins) > 1 and not e.is_const(ins[1]):
                raise MindIRError("%s needs constant axes" % onnx_op)
            axes = [int(axes)] if isinstance(axes, int) else [int(a) for a in (axes or ())]
            keep = int(bool(attrs.get("keep_dims", False)))
            x = e.tensor(ins[0])
            if axes_as_input:
                return e.node(onnx_op, [x] + ([e.ints(axes)] if axes else []), keepdims=keep)
            return e.node(onnx_op, [x], keepdims=keep, axes=axes or None)
        return h
    H["ReduceSum"] = reduction("ReduceSum", True)          # axes moved to an input in opset 13
    H["ReduceMean"] = reduction("ReduceMean", False)       # ... and only in opset 18 for the others
    H["ReduceMax"] = reduction("ReduceMax", False)
    H["ReduceMin"] = reduction("ReduceMin", False)
    H["ReduceProd"] = reduction("ReduceProd", False)

    @reg("Concat")
    def concat(e, ins, attrs):
        src = e.alias.get(ins[0])
        items = src.items if isinstance(src, _Tuple) else [e.tensor(i) for i in ins]
        return e.node("Concat", items, axis=int(attrs.get("axis", 0)))

    @reg("Gather")
    def gather(e, ins, attrs):
        axis = e.value(ins[2]) if len(ins) > 2 else 0
        return e.node("Gather", [e.tensor(ins[0]), e.tensor(ins[1])], axis=int(axis or 0))

    @reg("Cast")
    def cast(e, ins, attrs):
        dtype = e.value(ins[1]) if len(ins) > 1 else attrs.get("dst_type")
        if dtype not in DT:
            raise MindIRError("Cast to %r is not exported" % (dtype,))
        return e.node("Cast", [e.tensor(ins[0])], to=DT[dtype])

    @reg("ExpandDims")
    def expand_dims(e, ins, attrs):
        return e.node("Unsqueeze", [e.tensor(ins[0]), e.ints([e.value(ins[1])])])

    @reg("Squeeze")
    def squeeze(e, ins, attrs):
        axis = attrs.get("axis", ())
        axis = [axis] if isinstance(axis, int) else list(axis or ())
        return e.node("Squeeze", [e.tensor(ins[0])] + ([e.ints(axis)] if axis else []))

    @reg("Tile")
    def tile(e, ins, attrs):
        return e.node("Tile", [e.tensor(ins[0]), e.ints(e.value(ins[1]))])

    @reg("ZerosLike", "OnesLike")
    def fill_like(e, ins, attrs):
        x = e.tensor(ins[0])
        zero = e.node("Sub", [x, x])
        if attrs["__op__"] == "ZerosLike":
            return zero
        dtype = e.shapes.get(x, (None, torch.float32))[1]
        return e.node("Add", [zero, e.initializer(torch.tensor(1, dtype=dtype), "one")])

    @reg("StridedSlice")
    def strided_slice(e, ins, attrs):
        begin, end, strides = (e.value(i) for i in ins[1:4])
        if begin is None or end is None or strides is None:
            raise MindIRError("StridedSlice needs constant bounds")
        for mask in ("begin_mask", "end_mask", "ellipsis_mask", "new_axis_mask"):
            if attrs.get(mask, 0):
                raise MindIRError("StridedSlice with %s is not exported" % mask)
        axes = list(range(len(begin)))
        y = e.node("Slice", [e.tensor(ins[0]), e.ints(begin), e.ints(end), e.ints(axes), e.ints(strides)])
        shrink = [a for a in axes if (int(attrs.get("shrink_axis_mask", 0)) >> a) & 1]
        return e.node("Squeeze", [y, e.ints(shrink)]) if shrink else y

    @reg("Select")
    def select(e, ins, attrs):
        return e.node("Where", [e.tensor(i) for i in ins[:3]])

    @reg("ArgMaxWithValue", "Argmax")
    def argmax(e, ins, attrs):
        axis = int(attrs.get("axis", -1))
        idx = e.node("ArgMax", [e.tensor(ins[0])], axis=axis, keepdims=int(bool(attrs.get("keep_dims", False))))
        if attrs["__op__"] == "Argmax":
            return idx
        val = e.node("ReduceMax", [e.tensor(ins[0])], axes=[axis], keepdims=int(bool(attrs.get("keep_dims", False))))
        return _Tuple([idx, val])

    @reg("Dropout")
    def dropout(e, ins, attrs):
        x = e.tensor(ins[0])
        return _Tuple([e.node("Identity", [x]), x])

    return H


_HANDLERS = None

_RESULT_DTYPE_BOOL = {"Greater", "Less", "GreaterEqual", "LessEqual", "Equal", "NotEqual", "LogicalNot",
                      "LogicalAnd", "LogicalOr"}


def build_onnx_model(fg, producer_version="2.4.0"):
    """The ONNX ModelProto of a traced forward graph."""
    from . import mindir_proto
    from .mindir_proto import _read_attr, _read_tensor
    global _HANDLERS
    if _HANDLERS is None:
        _HANDLERS = _handlers()
    src = mindir_proto.build_model_proto(fg, producer_version)
    if src.functions:
        raise MindIRError("control flow (Switch / While nodes) is not exported to ONNX")
    M = messages()
    model = M["ModelProto"]()
    model.ir_version = 8
    model.producer_name = "MindSpore"
    model.producer_version = producer_version
    op = model.opset_import.add()
    op.version = OPSET                                  # the default operator set: no domain
    g = model.graph
    g.name = src.graph.name
    e = _Emitter(g)
    prims = {p.name: p for p in src.primitives}

    def value_info(vi, name, shape, dtype):
        vi.name = name
        tt = vi.type.tensor_type
        tt.elem_type = DT[dtype]
        tt.shape.SetInParent()
        for d in shape:
            tt.shape.dim.add().dim_value = int(d)

    for vi in src.graph.input:
        e.alias[vi.name] = vi.name
        if not vi.tensor:
            raise MindIRError("input %s has no recorded shape" % vi.name)
        dtype = mindir_proto._DT_REV[vi.tensor[0].data_type]
        shape = tuple(int(d) for d in vi.tensor[0].dims)
        value_info(g.input.add(), vi.name, shape, dtype)
        e.shapes[vi.name] = (shape, dtype)
    for tp in src.graph.parameter:
        t = _read_tensor(tp)
        _tensor_proto(g.initializer.add(), t, tp.name)
        e.alias[tp.name] = tp.name
        e.shapes[tp.name] = (tuple(t.shape), t.dtype)

    # `e.shapes` follows ranks and dtypes along the nodes: BiasAdd needs the rank of its operand, a scalar constant
    # takes the dtype of the tensor it meets
    for nd in src.graph.node:
        out_name = nd.output[0]
        if nd.op_type == "Constant":
            e.consts[out_name] = _read_attr(nd.attribute[0]) if nd.attribute else None
            continue
        pp = prims[nd.op_type[5:]]
        attrs = {a.name: _read_attr(a) for a in pp.attribute}
        attrs["__op__"] = pp.op_type
        ins = list(nd.input)
        if pp.op_type == "MakeTuple":
            e.alias[out_name] = _Tuple([e.tensor(i) for i in ins])
            continue
        if pp.op_type == "TupleGetItem":
            src_tuple = e.alias.get(ins[0])
            if not isinstance(src_tuple, _Tuple):
                raise MindIRError("TupleGetItem of a value that is not a tuple")
            e.alias[out_name] = src_tuple.items[int(e.value(ins[1]))]
            continue
        if pp.op_type in ("Depend", "Load", "Return"):
            e.alias[out_name] = e.tensor(ins[0])
            continue
        h = _HANDLERS.get(pp.op_type)
        if h is None:
            raise MindIRError("primitive %s has no ONNX counterpart in this exporter" % pp.op_type)
        res = h(e, ins, attrs)
        e.alias[out_name] = res
        _note_shape(e, pp.op_type, res, ins, attrs)
    outs = [o.name for o in src.graph.output]
    final = e.alias.get(outs[0]) if outs else None
    names = final.items if isinstance(final, _Tuple) else [e.tensor(outs[0])]
    examples = fg.example_outputs
    examples = list(examples) if isinstance(examples, (tuple, list)) else [examples]
    for k, name in enumerate(names):
        vi = g.output.add()
        ex = examples[k] if k < len(examples) else None
        if isinstance(ex, torch.Tensor) and ex.dtype in DT:
            value_info(vi, name, tuple(ex.shape), ex.dtype)
        else:
            vi.name = name
    return model


def _note_shape(e, op_type, res, ins, attrs):
    """Rank / dtype bookkeeping for the few places that need it (BiasAdd's reshape, dtypes of scalar constants)."""
    if isinstance(res, _Tuple) or not isinstance(res, str):
        if isinstance(res, _Tuple) and res.items and ins and e.alias.get(ins[0]) in e.shapes:
            e.shapes[res.items[0]] = e.shapes[e.alias[ins[0]]]
        return
    operands = [e.alias.get(i) for i in ins]
    known = next((e.shapes[o] for o in operands if isinstance(o, str) and o in e.shapes), None)
    if op_type in ("MatMul", "Conv2D"):              # results of fixed rank, whatever is known of the operands
        e.shapes[res] = ((None,) * (2 if op_type == "MatMul" else 4), known[1] if known else torch.float32)
        return
    first = operands[0] if operands else None
    known = e.shapes.get(first) if isinstance(first, str) else None
    if known is None:
        return
    shape, dtype = known
    if op_type in _RESULT_DTYPE_BOOL:
        dtype = torch.bool
    if op_type == "Cast":
        dtype = e.value(ins[1]) if len(ins) > 1 and e.value(ins[1]) in DT else attrs.get("dst_type", dtype)
    same_rank = {"ReLU", "Sigmoid", "Tanh", "Exp", "Log", "Sqrt", "Neg", "Abs", "Erf", "SiLU", "GeLU", "Softmax",
                 "LogSoftmax", "Add", "Sub", "Mul", "RealDiv", "Div", "Pow", "BiasAdd", "Conv2D", "MaxPool", "AvgPool",
                 "Identity", "StopGradient", "Cast", "Transpose", "ZerosLike", "OnesLike", "Maximum", "Minimum"} | \
        _RESULT_DTYPE_BOOL
    if op_type in same_rank:
        e.shapes[res] = ((None,) * len(shape), dtype)
    elif op_type == "Reshape" and e.value(ins[1]) is not None:
        e.shapes[res] = ((None,) * len(e.value(ins[1])), dtype)
    elif op_type == "Flatten":
        e.shapes[res] = ((None, None), dtype)
    elif op_type in ("MatMul", "BatchMatMul"):
        e.shapes[res] = ((None,) * len(shape), dtype)


def save_onnx(fg, path):
    data = build_onnx_model(fg).SerializeToString()
    with open(path, "wb") as f:
        f.write(data)
    return path
