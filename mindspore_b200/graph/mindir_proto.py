"""MindIR in the reference's protobuf wire format (``mind_ir.proto``: ModelProto / GraphProto / NodeProto /
PrimitiveProto / AttributeProto / TensorProto), so that graph files travel between the two frameworks.

Writer: ``save_model_proto(fg, path)`` stores a traced forward graph the way the reference's exporter lays one out
(ccsrc/common/debug/mindir_exporter.cc):

* weights are ``GraphProto.parameter`` tensors (name, dims, data_type, raw little-endian bytes), network inputs are
  ``GraphProto.input`` value infos;
* every primitive call is a ``NodeProto`` whose ``op_type`` is ``REF::<Prim>:<id>`` and names an entry of
  ``ModelProto.primitives`` carrying the primitive's attributes; node outputs are named ``<graph>:<n>``;
* values that are not nodes (scalars, tuples, dtypes, small tensors) become ``Constant`` nodes with one attribute
  ``value``; tuple indexing is the primitive ``TupleGetItem``, a tuple result ``MakeTuple``;
* attribute values carry their ``AttributeType``: INT64 / BOOL in ``i``, FLOAT in ``f``, DOUBLE in ``d``, STRING in
  ``s``, TUPLE / LIST in ``values``, a tensor or a dtype as one ``tensors`` entry (TENSORS), None as NONE.

Reader: ``load_model_proto(bytes)`` accepts that layout and the older one in which a node's ``op_type`` is the
primitive name itself and the attributes sit on the node (core/load_mindir/load_model.cc:1770-1780 distinguishes the
two by the ``REF::`` prefix).  Primitives are looked up by name in ``mindspore_b200.ops``; an operator this build does
not define is reported by name.  A model with sub-graphs (``functions``: the branches of an ``if``, the recursion of
a ``while``, closures) loads as one node run by an interpreter of the file's nodes (``_Program``).

The message classes are built at import time from a description of the schema (field names, numbers and types are
the file format), so no generated ``_pb2`` module and no ``protoc`` are needed."""
from __future__ import annotations

import inspect
import operator

import numpy as np
import torch

from .ir import FuncGraph
from .mindir import LoadedGraph, MindIRError

# ---------------------------------------------------------------------------------------------------- schema
_OPT, _REP, _REQ = 1, 3, 2
_T = {"string": 9, "bytes": 12, "int64": 3, "int32": 5, "uint64": 4, "float": 2, "double": 1, "bool": 8, "msg": 11,
      "enum": 5}        # enums travel as int32 here: unknown values of a newer writer must not fail the parse

_SCHEMA = {
    "AttributeProto": [
        ("name", 1, "string"), ("f", 2, "float"), ("i", 3, "int64"), ("d", 4, "double"), ("s", 5, "bytes"),
        ("t", 6, "TensorProto"), ("g", 7, "GraphProto"), ("floats", 8, "float*"), ("doubles", 9, "double*"),
        ("ints", 10, "int64*"), ("strings", 11, "bytes*"), ("tensors", 12, "TensorProto*"),
        ("graphs", 13, "GraphProto*"), ("doc_string", 14, "string"), ("ref_attr_name", 15, "string"),
        ("type", 16, "enum"), ("values", 17, "AttributeProto*")],
    "ValueInfoProto": [
        ("name", 1, "string"), ("tensor", 2, "TensorProto*"), ("doc_string", 3, "string"),
        ("denotation", 4, "string"), ("attr_info", 5, "AttributeProto")],
    "NodeProto": [
        ("input", 1, "string*"), ("output", 2, "string*"), ("name", 3, "string"), ("op_type", 4, "string"),
        ("attribute", 5, "AttributeProto*"), ("doc_string", 6, "string"), ("domain", 7, "string"),
        ("node_attr", 8, "AttributeProto*"), ("primal_attr", 9, "AttributeProto*")],
    "ModelProto": [
        ("ir_version", 1, "string"), ("producer_name", 2, "string"), ("producer_version", 3, "string"),
        ("domain", 4, "string"), ("model_version", 5, "string"), ("doc_string", 6, "string"),
        ("graph", 7, "GraphProto"), ("functions", 8, "GraphProto*"), ("little_endian", 10, "bool"),
        ("parallel", 11, "ParallelProto"), ("primitives", 12, "PrimitiveProto*"), ("mind_ir_version", 13, "int64")],
    "GraphProto": [
        ("node", 1, "NodeProto*"), ("name", 2, "string"), ("parameter", 3, "TensorProto*"),
        ("doc_string", 4, "string"), ("input", 5, "ValueInfoProto*"), ("output", 6, "ValueInfoProto*"),
        ("bprop_hash", 7, "string"), ("attribute", 8, "AttributeProto*"), ("bprop_filepath", 9, "string")],
    "TensorProto": [
        ("dims", 1, "int64*"), ("data_type", 2, "int32"), ("float_data", 3, "float*"), ("int32_data", 4, "int32*"),
        ("string_data", 5, "bytes*"), ("int64_data", 6, "int64*"), ("name", 7, "string"), ("doc_string", 8, "string"),
        ("raw_data", 9, "bytes"), ("double_data", 10, "double*"), ("uint64_data", 11, "uint64*"),
        ("ref_key", 13, "string"), ("min_dims", 14, "int64*"), ("max_dims", 15, "int64*"),
        ("compression_type", 16, "enum")],
    "ParallelProto": [("layout", 1, "LayoutProto*")],
    "LayoutProto": [
        ("name", 1, "string"), ("device_arrangement_int", 2, "int64*"), ("tensor_map_int", 3, "int64*"),
        ("slice_shape_int", 4, "int64*"), ("field_size", 5, "int64"), ("uniform_split", 6, "bool"),
        ("opt_shard_group", 7, "string")],
    "PrimitiveProto": [
        ("name", 1, "string"), ("op_type", 2, "string"), ("attribute", 3, "AttributeProto*"),
        ("instance_name", 4, "string"), ("prim_type", 5, "enum")],
}

_messages = None


def build_messages(schema, package, file_name):
    """{message name: class} for a schema given as {message: [(field, number, kind)]}; ``kind`` is a scalar type, the
    name of another message of the schema, or either followed by ``*`` for a repeated field."""
    from google.protobuf import descriptor_pb2, descriptor_pool, message_factory
    fdp = descriptor_pb2.FileDescriptorProto()
    fdp.name = file_name
    fdp.package = package
    fdp.syntax = "proto2"
    for mname, fields in schema.items():
        m = fdp.message_type.add()
        m.name = mname
        for fname, number, kind in fields:
            f = m.field.add()
            f.name, f.number = fname, number
            rep = kind.endswith("*")
            kind = kind.rstrip("*")
            f.label = _REP if rep else _OPT
            if kind in _T:
                f.type = _T[kind]
            else:
                f.type = _T["msg"]
                f.type_name = ".%s.%s" % (package, kind)
    pool = descriptor_pool.DescriptorPool()
    if hasattr(pool, "AddSerializedFile"):
        pool.AddSerializedFile(fdp.SerializeToString())
    else:
        pool.Add(fdp)
    get = getattr(message_factory, "GetMessageClass", None)
    out = {}
    for mname in schema:
        desc = pool.FindMessageTypeByName("%s.%s" % (package, mname))
        out[mname] = get(desc) if get else message_factory.MessageFactory(pool).GetPrototype(desc)
    return out


def messages():
    """{message name: class} built from ``_SCHEMA`` (package ``mind_ir``)."""
    global _messages
    if _messages is None:
        _messages = build_messages(_SCHEMA, "mind_ir", "mindspore_b200/mind_ir.proto")
    return _messages


# AttributeProto.AttributeType / TensorProto.DataType values used here
A_FLOAT, A_INT8, A_INT16, A_INT32, A_INT64, A_STRING, A_BOOL, A_DOUBLE = 1, 3, 5, 6, 7, 8, 9, 11
A_UINT8, A_UINT16, A_UINT32, A_UINT64 = 2, 4, 12, 13
A_TENSOR, A_TENSORS, A_TUPLE, A_LIST, A_DICT, A_UMONAD, A_IOMONAD, A_NONE = 17, 19, 20, 21, 22, 23, 24, 25
_INT_ATTR = (A_INT8, A_INT16, A_INT32, A_INT64, A_UINT8, A_UINT16, A_UINT32, A_UINT64)

_DT = {torch.float32: 1, torch.uint8: 2, torch.int8: 3, torch.int16: 5, torch.int32: 6, torch.int64: 7, torch.bool: 9,
       torch.float16: 10, torch.float64: 11, torch.complex64: 14, torch.complex128: 15, torch.bfloat16: 16}
_DT_REV = {v: k for k, v in _DT.items()}
_DT_REV[17] = torch.float64          # FLOAT64 is a second code for double
_DT_REV[4] = torch.int32             # uint16 / uint32 / uint64 have no torch counterpart everywhere: widened on load
_DT_REV[12] = torch.int64
_DT_REV[13] = torch.int64
_DT_NP = {4: np.uint16, 12: np.uint32, 13: np.uint64}

_BUILTIN_PRIMS = {operator.add: "Add", operator.sub: "Sub", operator.mul: "Mul", operator.truediv: "RealDiv",
                  operator.neg: "Neg", operator.matmul: "MatMul", operator.pow: "Pow"}


# ---------------------------------------------------------------------------------------------------- tensors
def _fill_tensor(tp, t, name=None):
    plain = t.detach().to("cpu").contiguous()
    if plain.dtype not in _DT:
        raise MindIRError("tensors of type %s have no MindIR data type" % plain.dtype)
    if name is not None:
        tp.name = name
    tp.data_type = _DT[plain.dtype]
    tp.dims.extend(int(d) for d in plain.shape)
    tp.raw_data = plain.view(torch.uint8).numpy().tobytes() if plain.dtype == torch.bfloat16 \
        else plain.numpy().tobytes()


def _read_tensor(tp):
    code = tp.data_type
    if code not in _DT_REV:
        raise MindIRError("tensor %r has MindIR data type %d, which is not supported" % (tp.name, code))
    dt = _DT_REV[code]
    shape = [int(d) for d in tp.dims]
    n = int(np.prod(shape)) if shape else 1
    if tp.raw_data:
        raw = bytearray(tp.raw_data)
        if code in _DT_NP:
            return torch.from_numpy(np.frombuffer(raw, dtype=_DT_NP[code]).astype(np.int64)).to(dt).reshape(shape)
        if dt == torch.bfloat16:
            return torch.frombuffer(raw, dtype=torch.uint8).view(torch.bfloat16).reshape(shape).clone()
        return torch.frombuffer(raw, dtype=dt).reshape(shape).clone()
    for field in ("float_data", "int32_data", "int64_data", "double_data", "uint64_data"):
        vals = list(getattr(tp, field))
        if vals:
            return torch.tensor(vals).to(dt).reshape(shape)
    if n == 0:
        return torch.empty(shape, dtype=dt)
    return None                                   # a type-only tensor (no data): the caller decides what it means


# ---------------------------------------------------------------------------------------------------- attributes
def _fill_attr(ap, v, in_sequence=False):
    """Python value -> AttributeProto (type tag + payload).  A scalar that is an element of a tuple / list goes
    into the repeated field of its kind (``ints`` / ``floats`` / ``doubles`` / ``strings``, one entry), a top-level
    scalar into ``i`` / ``f`` / ``d`` / ``s``: the two forms the reference's exporter writes
    (ccsrc/transform/express_ir/mindir_exporter.cc SetScalarToAttributeProto_irs / _ir)."""
    if v is None:
        ap.type = A_NONE
    elif isinstance(v, (bool, np.bool_)):
        ap.type = A_BOOL
        if in_sequence:
            ap.ints.append(int(bool(v)))
        else:
            ap.i = int(bool(v))
    elif isinstance(v, (int, np.integer)):
        ap.type = A_INT64
        if in_sequence:
            ap.ints.append(int(v))
        else:
            ap.i = int(v)
    elif isinstance(v, (float, np.floating)):
        f32 = float(np.float32(v))
        single = f32 == float(v) or v != v
        ap.type = A_FLOAT if single else A_DOUBLE
        if in_sequence:
            (ap.floats if single else ap.doubles).append(float(v))
        elif single:
            ap.f = float(v)
        else:
            ap.d = float(v)
    elif isinstance(v, str):
        ap.type = A_STRING
        if in_sequence:
            ap.strings.append(v.encode())
        else:
            ap.s = v.encode()
    elif isinstance(v, (tuple, list, torch.Size)):
        ap.type = A_LIST if isinstance(v, list) else A_TUPLE
        for item in v:
            _fill_attr(ap.values.add(), item, True)
    elif isinstance(v, dict):
        ap.type = A_DICT
        for k, item in v.items():
            sub = ap.values.add()
            sub.name = str(k)
            _fill_attr(sub, item, True)
    elif isinstance(v, torch.dtype):
        ap.type = A_TENSORS                       # a type value: one tensor entry that carries only a data type
        tp = ap.tensors.add()
        tp.name = "value0"
        if v not in _DT:
            raise MindIRError("dtype %s has no MindIR data type" % v)
        tp.data_type = _DT[v]
    elif isinstance(v, torch.Tensor):
        ap.type = A_TENSORS
        _fill_tensor(ap.tensors.add(), v, "value0")
    elif isinstance(v, np.ndarray):
        ap.type = A_TENSORS
        _fill_tensor(ap.tensors.add(), torch.from_numpy(np.ascontiguousarray(v)), "value0")
    else:
        raise MindIRError("value of type %s cannot be stored as a MindIR attribute" % type(v).__name__)


def _read_attr(ap):
    t = ap.type
    if t == A_NONE:
        return None
    # scalars: the single-value field, or (elements of sequences) one entry of the repeated field of their kind
    if t == A_BOOL:
        return bool(ap.ints[0]) if len(ap.ints) and not ap.HasField("i") else bool(ap.i)
    if t in _INT_ATTR:
        return int(ap.ints[0]) if len(ap.ints) and not ap.HasField("i") else int(ap.i)
    if t == A_FLOAT:
        return float(ap.floats[0]) if len(ap.floats) and not ap.HasField("f") else float(ap.f)
    if t == A_DOUBLE:
        return float(ap.doubles[0]) if len(ap.doubles) and not ap.HasField("d") else float(ap.d)
    if t == A_STRING:
        return (ap.strings[0] if len(ap.strings) and not ap.HasField("s") else ap.s).decode()
    if t in (A_TUPLE, A_LIST):
        vals = [_read_attr(x) for x in ap.values]
        return vals if t == A_LIST else tuple(vals)
    if t == A_DICT:
        return {x.name: _read_attr(x) for x in ap.values}
    if t in (A_TENSORS, A_TENSOR):
        tps = list(ap.tensors) if t == A_TENSORS else [ap.t]
        out = []
        for tp in tps:
            ten = _read_tensor(tp)
            out.append(ten if ten is not None else _DT_REV[tp.data_type])
        return out[0] if len(out) == 1 else tuple(out)
    if t in (A_UMONAD, A_IOMONAD):
        return _MONAD
    if t == 0:                                    # older writers: untyped, the payload field says what it is
        if ap.ints:
            return tuple(int(x) for x in ap.ints)
        if ap.floats:
            return tuple(float(x) for x in ap.floats)
        if ap.strings:
            return tuple(s.decode() for s in ap.strings)
        if ap.tensors:
            tens = [_read_tensor(tp) for tp in ap.tensors]
            return tens[0] if len(tens) == 1 else tuple(tens)
        for field, conv in (("s", lambda s: s.decode()), ("i", int), ("f", float), ("d", float)):
            if ap.HasField(field):
                return conv(getattr(ap, field))
        return None
    raise MindIRError("attribute %r has type %d, which this reader does not handle" % (ap.name, t))


class _Monad:
    def __repr__(self):
        return "U"


_MONAD = _Monad()


# ---------------------------------------------------------------------------------------------------- lowering
def _pair(v):
    return (int(v), int(v)) if isinstance(v, int) else tuple(int(x) for x in v)


def _lowerings():
    """{torch function: rule}.  A rule receives (emit, args, kwargs, node) and returns the name of its result;
    ``emit(primitive name, attributes, inputs)`` writes one primitive node.  Layers of ``nn`` call these torch
    functions directly, so a traced network is a mix of primitives and of them; the rules restate each call with the
    primitives a MindIR consumer knows."""
    import torch.nn.functional as F

    def arg(args, kwargs, i, name, default=None):
        if len(args) > i:
            return args[i]
        return kwargs.get(name, default)

    def conv2d(emit, a, k, n):
        x, w, b = a[0], a[1], arg(a, k, 2, "bias")
        stride, pad = _pair(arg(a, k, 3, "stride", 1)), arg(a, k, 4, "padding", 0)
        dil, groups = _pair(arg(a, k, 5, "dilation", 1)), int(arg(a, k, 6, "groups", 1))
        wshape = tuple(w.meta["shape"])
        if isinstance(pad, str):
            raise MindIRError("string padding of conv2d is not lowered")
        ph, pw = _pair(pad)
        attrs = {"out_channel": int(wshape[0]), "kernel_size": (int(wshape[2]), int(wshape[3])), "mode": 1,
                 "pad_mode": "pad" if (ph or pw) else "valid", "pad": (ph, ph, pw, pw),
                 "stride": (1, 1) + stride, "dilation": (1, 1) + dil, "group": groups, "format": "NCHW"}
        y = emit("Conv2D", attrs, [x, w])
        return emit("BiasAdd", {"format": "NCHW"}, [_Ref(y), b]) if b is not None else y

    def linear(emit, a, k, n):
        x, w, b = a[0], a[1], arg(a, k, 2, "bias")
        rank = len(x.meta.get("shape", (0, 0)))
        if rank != 2:
            shp = tuple(int(d) for d in x.meta["shape"])
            x2 = emit("Reshape", {}, [x, (-1, shp[-1])])
            y = emit("MatMul", {"transpose_a": False, "transpose_b": True}, [_Ref(x2), w])
            if b is not None:
                y = emit("BiasAdd", {"format": "NCHW"}, [_Ref(y), b])
            return emit("Reshape", {}, [_Ref(y), shp[:-1] + (int(w.meta["shape"][0]),)])
        y = emit("MatMul", {"transpose_a": False, "transpose_b": True}, [x, w])
        return emit("BiasAdd", {"format": "NCHW"}, [_Ref(y), b]) if b is not None else y

    def pool(name):
        def rule(emit, a, k, n):
            ks = _pair(arg(a, k, 1, "kernel_size"))
            st = arg(a, k, 2, "stride")
            st = ks if st in (None, ()) else _pair(st)
            if _pair(arg(a, k, 3, "padding", 0)) != (0, 0) or arg(a, k, 5 if name == "MaxPool" else 4, "ceil_mode", False):
                raise MindIRError("padded / ceil-mode pooling is not lowered")
            return emit(name, {"kernel_size": (1, 1) + ks, "strides": (1, 1) + st, "pad_mode": "VALID",
                               "format": "NCHW"}, [a[0]])
        return rule

    def unary(name, **attrs):
        return lambda emit, a, k, n: emit(name, dict(attrs), [a[0]])

    def binary(name):
        def rule(emit, a, k, n):
            if k.get("alpha", 1) != 1:
                raise MindIRError("alpha of torch.add / torch.sub is not lowered")
            return emit(name, {}, [a[0], a[1]])
        return rule

    def softmax(name):
        def rule(emit, a, k, n):
            return emit(name, {"axis": int(arg(a, k, 1, "dim", -1))}, [a[0]])
        return rule

    def flatten(emit, a, k, n):
        start, end = int(arg(a, k, 1, "start_dim", 0)), int(arg(a, k, 2, "end_dim", -1))
        shp = tuple(int(d) for d in a[0].meta["shape"])
        if start == 1 and end in (-1, len(shp) - 1):
            return emit("Flatten", {}, [a[0]])
        end = end % len(shp)
        mid = 1
        for d in shp[start:end + 1]:
            mid *= d
        return emit("Reshape", {}, [a[0], shp[:start] + (mid,) + shp[end + 1:]])

    def layer_norm(emit, a, k, n):
        x, nshape = a[0], tuple(arg(a, k, 1, "normalized_shape"))
        w, b, eps = arg(a, k, 2, "weight"), arg(a, k, 3, "bias"), float(arg(a, k, 4, "eps", 1e-5))
        if w is None or b is None:
            raise MindIRError("layer_norm without affine parameters is not lowered")
        axis = len(x.meta["shape"]) - len(nshape)
        y = emit("LayerNorm", {"begin_norm_axis": axis, "begin_params_axis": axis, "epsilon": eps}, [x, w, b])
        return emit("TupleGetItem", {}, [_Ref(y), 0])

    def batch_norm(emit, a, k, n):
        x, mean, var = a[0], arg(a, k, 1, "running_mean"), arg(a, k, 2, "running_var")
        w, b = arg(a, k, 3, "weight"), arg(a, k, 4, "bias")
        if arg(a, k, 5, "training", False) or mean is None or w is None:
            raise MindIRError("only inference-mode batch_norm with affine parameters is lowered")
        y = emit("BatchNorm", {"is_training": False, "epsilon": float(arg(a, k, 7, "eps", 1e-5)), "momentum": 0.1,
                               "format": "NCHW"}, [x, w, b, mean, var])
        return emit("TupleGetItem", {}, [_Ref(y), 0])

    def reshape(emit, a, k, n):
        shape = a[1] if len(a) == 2 and isinstance(a[1], (tuple, list, torch.Size)) else tuple(a[1:])
        return emit("Reshape", {}, [a[0], tuple(int(d) for d in shape)])

    def permute(emit, a, k, n):
        perm = a[1] if len(a) == 2 and isinstance(a[1], (tuple, list)) else tuple(a[1:])
        return emit("Transpose", {}, [a[0], tuple(int(d) for d in perm)])

    def transpose(emit, a, k, n):
        rank = len(a[0].meta["shape"])
        perm = list(range(rank))
        d0, d1 = int(a[1]) % rank, int(a[2]) % rank
        perm[d0], perm[d1] = perm[d1], perm[d0]
        return emit("Transpose", {}, [a[0], tuple(perm)])

    def matmul(emit, a, k, n):
        rank = len(a[0].meta.get("shape", (0, 0)))
        return emit("MatMul" if rank == 2 else "BatchMatMul", {"transpose_a": False, "transpose_b": False},
                    [a[0], a[1]])

    def dropout(emit, a, k, n):
        if arg(a, k, 2, "training", True):
            raise MindIRError("training-mode dropout is not lowered")
        return emit("Identity", {}, [a[0]])

    def gelu(emit, a, k, n):
        return emit("GeLU", {}, [a[0]])

    def cat(emit, a, k, n):
        xs = list(a[0])
        t = emit("MakeTuple", {}, xs)
        return emit("Concat", {"axis": int(arg(a, k, 1, "dim", 0))}, [_Ref(t)])

    def reduce(name):
        def rule(emit, a, k, n):
            dim = arg(a, k, 1, "dim", ())
            dim = (int(dim),) if isinstance(dim, int) else tuple(int(d) for d in (dim or ()))
            return emit(name, {"keep_dims": bool(arg(a, k, 2, "keepdim", False))}, [a[0], dim])
        return rule

    def embedding(emit, a, k, n):
        return emit("Gather", {"batch_dims": 0}, [a[1], a[0], 0])

    T = torch.Tensor
    table = {
        torch.conv2d: conv2d, F.conv2d: conv2d, F.linear: linear, torch._C._nn.linear: linear,
        F.max_pool2d: pool("MaxPool"), F.avg_pool2d: pool("AvgPool"), torch._C._nn.avg_pool2d: pool("AvgPool"),
        torch.relu: unary("ReLU"), F.relu: unary("ReLU"), T.relu: unary("ReLU"),
        torch.sigmoid: unary("Sigmoid"), T.sigmoid: unary("Sigmoid"), torch.tanh: unary("Tanh"), T.tanh: unary("Tanh"),
        F.silu: unary("SiLU"), F.gelu: gelu, torch.exp: unary("Exp"), torch.sqrt: unary("Sqrt"),
        torch.neg: unary("Neg"), T.neg: unary("Neg"),
        torch.add: binary("Add"), T.add: binary("Add"), torch.sub: binary("Sub"), T.sub: binary("Sub"),
        torch.mul: binary("Mul"), T.mul: binary("Mul"), torch.div: binary("RealDiv"), T.div: binary("RealDiv"),
        torch.true_divide: binary("RealDiv"), torch.pow: binary("Pow"), T.pow: binary("Pow"),
        T.__add__: binary("Add"), T.__sub__: binary("Sub"), T.__mul__: binary("Mul"), T.__truediv__: binary("RealDiv"),
        T.__radd__: binary("Add"), T.__rmul__: binary("Mul"),
        torch.softmax: softmax("Softmax"), F.softmax: softmax("Softmax"), T.softmax: softmax("Softmax"),
        torch.log_softmax: softmax("LogSoftmax"), F.log_softmax: softmax("LogSoftmax"),
        torch.flatten: flatten, T.flatten: flatten, F.layer_norm: layer_norm, torch.layer_norm: layer_norm,
        F.batch_norm: batch_norm, torch.batch_norm: batch_norm,
        torch.reshape: reshape, T.reshape: reshape, T.view: reshape, torch.permute: permute, T.permute: permute,
        torch.transpose: transpose, T.transpose: transpose, torch.matmul: matmul, T.matmul: matmul,
        torch.bmm: matmul, torch.mm: matmul, F.dropout: dropout, torch.dropout: dropout, torch.cat: cat,
        torch.mean: reduce("ReduceMean"), T.mean: reduce("ReduceMean"), torch.sum: reduce("ReduceSum"),
        T.sum: reduce("ReduceSum"), F.embedding: embedding, torch.embedding: embedding,
    }
    table[T.detach] = table[torch.detach] = unary("StopGradient")

    def getitem(emit, a, k, n):
        """``x[i, 2:5, ::2]`` with ints and slices of positive step -> StridedSlice (shrink mask for the ints)."""
        index = a[1] if isinstance(a[1], tuple) else (a[1],)
        shape = tuple(int(d) for d in a[0].meta["shape"])
        if len(index) > len(shape) or not all(isinstance(i, (int, slice)) for i in index):
            raise MindIRError("node %s indexes a tensor with %r; ints and slices are lowered" % (n.name, a[1]))
        begin, end, strides, shrink = [], [], [], 0
        for axis, i in enumerate(index):
            if isinstance(i, int):
                i = i % shape[axis]
                begin.append(i)
                end.append(i + 1)
                strides.append(1)
                shrink |= 1 << axis
                continue
            if not all(isinstance(v, (int, type(None))) for v in (i.start, i.stop, i.step)) or (i.step or 1) <= 0:
                raise MindIRError("node %s slices with %r; constant slices of positive step are lowered"
                                  % (n.name, i))
            lo, hi, st = i.indices(shape[axis])
            begin.append(lo)
            end.append(hi)
            strides.append(st)
        attrs = {"begin_mask": 0, "end_mask": 0, "ellipsis_mask": 0, "new_axis_mask": 0, "shrink_axis_mask": shrink}
        return emit("StridedSlice", attrs, [a[0], tuple(begin), tuple(end), tuple(strides)])
    table[T.__getitem__] = getitem
    for short, dunder, prim_name in (("gt", "__gt__", "Greater"), ("lt", "__lt__", "Less"),
                                     ("ge", "__ge__", "GreaterEqual"), ("le", "__le__", "LessEqual"),
                                     ("eq", "__eq__", "Equal"), ("ne", "__ne__", "NotEqual")):
        for fn in (getattr(torch, short), getattr(T, short), getattr(T, dunder)):
            table[fn] = binary(prim_name)
    return table


class _Ref:
    """The result of a node that this export has just written (by its MindIR name)."""

    def __init__(self, name):
        self.name = name


_LOWER = None


# ---------------------------------------------------------------------------------------------------- writer
def build_model_proto(fg, producer_version="2.4.0"):
    """One ModelProto for a traced graph.  A ``Switch`` node becomes two entries of ``functions`` (its branches),
    two ``Partial`` nodes that bind the operands, a ``Switch`` primitive that picks one and a call of its result; a
    ``While`` node becomes the recursive header / body / exit functions that the reference's parser makes of a
    ``while`` statement (ccsrc/pipeline/jit/ps/parse/parse.cc: ParseWhile)."""
    import torch.fx as fx
    from . import autodiff
    from .control_flow import Switch, While
    M = messages()
    model = M["ModelProto"]()
    model.ir_version = "0.1.1"
    model.producer_name = "MindSpore"
    model.producer_version = producer_version
    model.model_version = "1"
    model.little_endian = True
    model.mind_ir_version = 2
    main = model.graph
    counter = [0]
    written_params = set()
    graph_names = set()

    def unique_graph_name(base):
        name, k = base, 0
        while name in graph_names:
            k += 1
            name = "%s_%d" % (base, k)
        graph_names.add(name)
        return name

    def write_graph(fg, gp, gname):
        gp.name = gname
        names = {}

        def fresh():
            counter[0] += 1
            return "%s:%d" % (gname, counter[0])

        def constant(value):
            node = gp.node.add()
            node.name = fresh()
            node.output.append(node.name)
            node.op_type = "Constant"
            ap = node.attribute.add()
            ap.name = "value"
            _fill_attr(ap, value)
            return node.name

        def operand(a):
            if isinstance(a, fx.Node):
                return names[a]
            if isinstance(a, _Ref):
                return a.name
            return constant(a)

        def raw_node(op_type, ins, scope=""):
            node = gp.node.add()
            node.name = fresh()
            node.output.append(node.name)
            node.op_type = op_type
            node.domain = scope
            node.input.extend(ins)
            return node.name

        def call(prim_name, attrs, inputs, scope=""):
            pp = model.primitives.add()
            pp.name = "%s:%d" % (prim_name, len(model.primitives))
            pp.op_type = prim_name
            pp.prim_type = 1
            for k, v in attrs.items():
                ap = pp.attribute.add()
                ap.name = k
                try:
                    _fill_attr(ap, v)
                except MindIRError:
                    del pp.attribute[-1]          # callables and the like are not part of a primitive's record
            ins = [operand(a) for a in inputs]    # constants are written before the node that reads them
            return raw_node("REF::" + pp.name, ins, scope)

        def function(sub, base):
            """Writes a traced sub-graph as an entry of ``functions`` and returns its name (a node input that is a
            function's name refers to the function itself)."""
            name = unique_graph_name(base)
            write_graph(sub, model.functions.add(), name)
            return name

        def synthetic(name, n_inputs, body):
            """A function that this exporter composes itself under a name reserved by the caller:
            ``body(node, prim, const, input names)`` returns the name of the output."""
            sub = model.functions.add()
            sub.name = name
            ins = []
            for k in range(n_inputs):
                vi = sub.input.add()
                vi.name = "%s:x%d" % (name, k)
                ins.append(vi.name)

            def sub_node(op_type, inputs):
                counter[0] += 1
                node = sub.node.add()
                node.name = "%s:%d" % (name, counter[0])
                node.output.append(node.name)
                node.op_type = op_type
                node.input.extend(inputs)
                return node.name

            def sub_call(prim_name, inputs):
                pp = model.primitives.add()
                pp.name = "%s:%d" % (prim_name, len(model.primitives))
                pp.op_type = prim_name
                pp.prim_type = 1
                return sub_node("REF::" + pp.name, inputs)

            def sub_const(value):
                counter[0] += 1
                node = sub.node.add()
                node.name = "%s:%d" % (name, counter[0])
                node.output.append(node.name)
                node.op_type = "Constant"
                ap = node.attribute.add()
                ap.name = "value"
                _fill_attr(ap, value)
                return node.name

            sub.output.add().name = body(sub_node, sub_call, sub_const, ins)

        def switch(n):
            sw = n.target
            pred, vals = n.args[0], [operand(a) for a in n.args[1:]]
            ops_ = vals[:sw.n_operands]
            caps = (vals[sw.n_operands:sw.n_operands + sw.n_true_caps], vals[sw.n_operands + sw.n_true_caps:])
            partials = []
            for branch, label in ((0, "cond_true"), (1, "cond_false")):
                sub = sw.graphs[branch]
                fname = function(sub, "%s_%s" % (gname, label))
                ins = [ops_[i] for i in sub.operand_positions] + caps[branch]
                partials.append(call("Partial", {}, [_Ref(fname)] + [_Ref(i) for i in ins]))
            chosen = call("Switch", {}, [pred, _Ref(partials[0]), _Ref(partials[1])])
            return raw_node("REF::" + chosen, [])

        def loop(n):
            wl = n.target
            if wl.max_iterations is not None:
                raise MindIRError("a While node with max_iterations has no MindIR form")
            cg, bg = wl.graphs
            vals = [operand(a) for a in n.args]
            ns, nc, nb = wl.n_state, wl.n_cond_caps, wl.n_body_caps
            cond_name = function(cg, gname + "_while_cond")
            body_name = function(bg, gname + "_while_body")
            header_name = unique_graph_name(gname + "_while_header")
            step_name = unique_graph_name(gname + "_while_step")
            exit_name = unique_graph_name(gname + "_while_exit")
            total = ns + nc + nb

            def exit_body(node, prim, const, ins):
                return prim("MakeTuple", ins)
            synthetic(exit_name, ns, exit_body)

            def step_body(node, prim, const, ins):
                state, b_caps = ins[:ns], ins[ns + nc:]
                out = node("REF::" + body_name, [state[i] for i in bg.operand_positions] + b_caps)
                if isinstance(bg.example_outputs, (tuple, list)):
                    nxt = [prim("TupleGetItem", [out, const(k)]) for k in range(ns)]
                else:
                    nxt = [out]
                return node("REF::" + header_name, nxt + ins[ns:])

            def header_body(node, prim, const, ins):
                state, c_caps = ins[:ns], ins[ns:ns + nc]
                c = node("REF::" + cond_name, [state[i] for i in cg.operand_positions] + c_caps)
                again = prim("Partial", [step_name] + ins)
                leave = prim("Partial", [exit_name] + state)
                chosen = prim("Switch", [c, again, leave])
                return node("REF::" + chosen, [])
            synthetic(header_name, total, header_body)
            synthetic(step_name, total, step_body)
            return raw_node("REF::" + header_name, vals)

        for n in fg.graph.nodes:
            if n.op == "placeholder":
                vi = gp.input.add()
                vi.name = n.name if gp is main else "%s:%s" % (gname, n.name)
                names[n] = vi.name
                shape, dtype = n.meta.get("shape"), n.meta.get("dtype")
                if shape is None and isinstance(n.meta.get("example"), tuple) and len(n.meta["example"]) == 2:
                    shape, dtype = n.meta["example"]
                if shape is not None and dtype in _DT:
                    tp = vi.tensor.add()
                    tp.dims.extend(int(d) for d in shape)
                    tp.data_type = _DT[dtype]
            elif n.op == "get_attr":
                if "param" in n.meta:
                    pname = n.target.split("::", 1)[1]
                    if pname not in written_params:           # weights live in the main graph; functions name them
                        written_params.add(pname)
                        _fill_tensor(main.parameter.add(), n.meta["param"], pname)
                    names[n] = pname
                else:
                    names[n] = constant(n.meta["const"])
            elif n.op == "call_function":
                if n.target is autodiff.vjp:
                    raise MindIRError("only forward graphs can be exported (found a gradient node)")
                if isinstance(n.target, Switch):
                    names[n] = switch(n)
                    continue
                if isinstance(n.target, While):
                    names[n] = loop(n)
                    continue
                is_prim = hasattr(n.target, "name") and hasattr(n.target, "attrs")
                if n.kwargs and (is_prim or n.target in _BUILTIN_PRIMS or n.target is operator.getitem):
                    raise MindIRError("node %s passes keyword arguments, which MindIR nodes cannot carry" % n.name)
                if n.target is operator.getitem:
                    if not isinstance(n.args[1], int):
                        raise MindIRError("node %s slices a tensor; only tuple indexing is stored" % n.name)
                    names[n] = call("TupleGetItem", {}, [n.args[0], int(n.args[1])])
                elif n.target in _BUILTIN_PRIMS:
                    names[n] = call(_BUILTIN_PRIMS[n.target], {}, list(n.args))
                elif is_prim:
                    attrs = dict(n.target.attrs)
                    if getattr(n.target, "in_strategy", None) is not None:
                        attrs["in_strategy"] = n.target.in_strategy
                    if getattr(n.target, "out_strategy", None) is not None:
                        attrs["out_strategy"] = n.target.out_strategy
                    names[n] = call(n.target.name, attrs, list(n.args), str(n.meta.get("scope", "")))
                else:
                    global _LOWER
                    if _LOWER is None:
                        _LOWER = _lowerings()
                    rule = _LOWER.get(n.target)
                    if rule is None:
                        raise MindIRError("node %s calls %r, which is neither a primitive nor a function with a "
                                          "lowering to primitives" % (n.name, n.target))
                    names[n] = rule(call, tuple(n.args), dict(n.kwargs), n)
            elif n.op == "output":
                res = n.args[0]
                if isinstance(res, (tuple, list)):
                    out_name = call("MakeTuple", {}, list(res))
                else:
                    out_name = operand(res)
                gp.output.add().name = out_name
            else:
                raise MindIRError("node kind %s is not supported in graph files" % n.op)

    write_graph(fg, main, unique_graph_name(fg.name or "graph"))
    return model


def save_model_proto(fg, path):
    data = build_model_proto(fg).SerializeToString()
    with open(path, "wb") as f:
        f.write(data)
    return path


# ---------------------------------------------------------------------------------------------------- reader
def looks_like_model_proto(data):
    """A ModelProto starts with field 1 (ir_version, a short string): tag 0x0A."""
    return len(data) > 2 and data[0] == 0x0A and data[1] < 32


def _make_primitive(op_type, attrs):
    from .. import ops
    cls = getattr(ops, op_type, None)
    if cls is None or not inspect.isclass(cls):
        raise MindIRError("the graph uses operator %s, which this build does not define" % op_type)
    init = getattr(cls.__init__, "decorated_func", cls.__init__)
    params = [p for p in list(inspect.signature(init).parameters.values())[1:]
              if p.kind in (p.POSITIONAL_OR_KEYWORD, p.KEYWORD_ONLY)]
    kwargs = {p.name: attrs[p.name] for p in params if p.name in attrs}
    prim = cls(**kwargs)
    for k, v in attrs.items():
        if k in ("in_strategy", "out_strategy") or k in kwargs:
            continue
        if hasattr(prim, "add_prim_attr"):
            try:
                prim.add_prim_attr(k, v)
            except Exception:  # noqa: BLE001  (bookkeeping attributes of the writer: not needed to run)
                pass
    if attrs.get("in_strategy") is not None and hasattr(prim, "shard"):
        prim.shard(attrs["in_strategy"], attrs.get("out_strategy"))
    return prim


def _make_tuple(*items):
    return tuple(items)


class _TailCall:
    """A call in tail position, handed back to the caller's loop: a ``while`` written as recursion between the header
    and the step function runs in constant Python stack depth."""

    def __init__(self, callee, args):
        self.callee, self.args = callee, args


class _Closure:
    """A function of the model together with the frame in which its name was read (its free variables)."""

    def __init__(self, program, gp, frame):
        self.program, self.gp, self.frame = program, gp, frame

    def __call__(self, *args):
        return _resolve(self.program.run(self.gp, args, self.frame))


class _BoundCall:
    """``Partial(fn, a, b)``: the callee and its leading arguments."""

    def __init__(self, callee, bound):
        self.callee, self.bound = callee, tuple(bound)

    def __call__(self, *args):
        return _resolve(_TailCall(self.callee, self.bound + tuple(args)))


def _resolve(res):
    while isinstance(res, _TailCall):
        callee, args = res.callee, res.args
        while isinstance(callee, _BoundCall):
            callee, args = callee.callee, callee.bound + tuple(args)
        if isinstance(callee, _Closure):
            res = callee.program.run(callee.gp, args, callee.frame)
        else:
            res = callee(*args)
    return res


class _Program:
    """Interpreter for a model with ``functions``: nodes run in file order; a node input that names a function is
    that function as a value (with the current frame, so nodes of enclosing graphs stay readable by name); a node
    whose ``op_type`` names a function or an earlier node calls it.  ``Switch`` reads its condition on the host and
    returns one of its two operands, ``Partial`` binds leading arguments.  Parity (role): the ANF graphs that
    core/load_mindir/anf_model_parser.cc rebuilds and the VM that runs Switch / Partial / calls of them."""

    def __init__(self, model, weight_names):
        self.primitives = {p.name: p for p in model.primitives}
        self.functions = {f.name: f for f in model.functions}
        self.main = model.graph
        self.weight_names = list(weight_names)
        self._prim_cache = {}
        self._constants = {}
        self.__name__ = "MindIRProgram"

    def __call__(self, *values):
        n_in = len(values) - len(self.weight_names)
        globals_frame = ({name: v for name, v in zip(self.weight_names, values[n_in:])}, None)
        return _resolve(self.run(self.main, values[:n_in], globals_frame))

    def primitive(self, key):
        hit = self._prim_cache.get(key)
        if hit is None:
            pp = self.primitives[key]
            attrs = {a.name: _read_attr(a) for a in pp.attribute}
            special = pp.op_type in ("TupleGetItem", "MakeTuple", "MakeList", "Depend", "UpdateState", "Load",
                                     "Return", "Switch", "Partial", "SwitchLayer")
            hit = self._prim_cache[key] = (pp.op_type, None if special else _make_primitive(pp.op_type, attrs))
        return hit

    def lookup(self, name, frame):
        f = frame
        while f is not None:
            if name in f[0]:
                return f[0][name]
            f = f[1]
        if name in self.functions:
            return _Closure(self, self.functions[name], frame)
        raise MindIRError("node input %r is not defined before its use" % name)

    def run(self, gp, args, outer):
        values = {}
        frame = (values, outer)
        declared = [vi.name for vi in gp.input if vi.name not in self.weight_names]
        if len(declared) != len(args):
            raise MindIRError("graph %s takes %d inputs, but %d were given" % (gp.name, len(declared), len(args)))
        values.update(zip(declared, args))
        out_name = gp.output[0].name if gp.output else None
        for nd in gp.node:
            name = nd.output[0] if nd.output else nd.name
            if nd.op_type == "Constant":
                key = (gp.name, name)
                if key not in self._constants:
                    self._constants[key] = _read_attr(nd.attribute[0]) if nd.attribute else None
                values[name] = self._constants[key]
                continue
            ins = [self.lookup(i, frame) for i in nd.input]
            ins = [a for a in ins if a is not _MONAD]
            key = nd.op_type[5:] if nd.op_type.startswith("REF::") else None
            if key is None or key in self.primitives:
                if key is None:
                    op_type, prim = nd.op_type, None
                    if op_type not in ("TupleGetItem", "MakeTuple", "MakeList", "Depend", "UpdateState", "Load",
                                       "Return", "Switch", "Partial", "SwitchLayer"):
                        ck = ("node", gp.name, name)
                        if ck not in self._prim_cache:
                            self._prim_cache[ck] = _make_primitive(op_type,
                                                                   {a.name: _read_attr(a) for a in nd.attribute})
                        prim = self._prim_cache[ck]
                else:
                    op_type, prim = self.primitive(key)
                if op_type == "TupleGetItem":
                    values[name] = ins[0][int(ins[1])]
                elif op_type == "MakeTuple":
                    values[name] = tuple(ins)
                elif op_type == "MakeList":
                    values[name] = list(ins)
                elif op_type in ("Depend", "UpdateState", "Load"):
                    values[name] = ins[0] if ins else _MONAD
                elif op_type == "Return":
                    values[name] = ins[0]
                elif op_type == "Switch":
                    cond = ins[0]
                    if isinstance(cond, torch.Tensor):
                        cond = bool(cond.detach().as_subclass(torch.Tensor).reshape(-1)[0].item())
                    values[name] = ins[1] if cond else ins[2]
                elif op_type == "SwitchLayer":
                    index = ins[0]
                    if isinstance(index, torch.Tensor):
                        index = int(index.detach().as_subclass(torch.Tensor).reshape(-1)[0].item())
                    values[name] = ins[1][index]
                elif op_type == "Partial":
                    values[name] = _BoundCall(ins[0], ins[1:])
                else:
                    values[name] = prim(*ins)
                continue
            callee = self.lookup(key, frame)
            if not callable(callee):
                raise MindIRError("node %s calls %s, which is not a function of the model" % (nd.name, key))
            if name == out_name:
                return _TailCall(callee, tuple(ins))
            values[name] = _resolve(_TailCall(callee, tuple(ins)))
        if out_name is None:
            raise MindIRError("graph %s has no output" % gp.name)
        outs = [self.lookup(o.name, frame) for o in gp.output]
        return outs[0] if len(outs) == 1 else tuple(outs)


def load_model_proto(data):
    from ..common.parameter import Parameter
    from ..common.tensor import Tensor
    M = messages()
    model = M["ModelProto"]()
    try:
        model.ParseFromString(bytes(data))
    except Exception as e:  # noqa: BLE001
        raise MindIRError("not a MindIR protobuf file: %s" % e)
    gp = model.graph
    prims = {p.name: p for p in model.primitives}
    fg = FuncGraph(gp.name or "graph")
    g = fg.graph
    env = {}
    param_names = {tp.name for tp in gp.parameter}
    n_in = 0
    for vi in gp.input:
        if vi.name in param_names:
            continue                              # older writers list the weights among the inputs too
        node = g.placeholder("x%d" % n_in if not vi.name.isidentifier() else vi.name)
        if vi.tensor:
            node.meta["shape"] = tuple(int(d) for d in vi.tensor[0].dims)
            if vi.tensor[0].data_type in _DT_REV:
                node.meta["dtype"] = _DT_REV[vi.tensor[0].data_type]
        env[vi.name] = node
        n_in += 1
    for tp in gp.parameter:
        ten = _read_tensor(tp)
        if ten is None:
            raise MindIRError("parameter %r has no data (stored outside the file?)" % tp.name)
        p = Parameter(Tensor(ten), name=tp.name, requires_grad=ten.is_floating_point())
        node = g.create_node("get_attr", "param::" + tp.name)
        node.meta["param"] = p
        fg.params[tp.name] = p
        env[tp.name] = node

    def value_of(name):
        if name not in env:
            raise MindIRError("node input %r is not defined before its use" % name)
        return env[name]

    if model.functions:
        # control flow: the whole model is ONE node of the graph, run by the interpreter; the weights stay
        # parameters of the loaded graph (they are the node's trailing operands)
        weights = [tp.name for tp in gp.parameter]
        operands = [env[vi.name] for vi in gp.input if vi.name not in param_names] + [env[w] for w in weights]
        node = g.create_node("call_function", _Program(model, weights), tuple(operands), {})
        node.meta["primitive"] = "MindIRProgram"
        fg.output_node = g.output(node)
        fg.input_positions = list(range(n_in))
        return LoadedGraph(fg)

    for nd in gp.node:
        out_name = nd.output[0] if nd.output else nd.name
        if nd.op_type == "Constant":
            val = _read_attr(nd.attribute[0]) if nd.attribute else None
            if isinstance(val, torch.Tensor):
                cn = g.create_node("get_attr", "const::%d" % len(env))
                cn.meta["const"] = val
                val = cn
            env[out_name] = val
            continue
        if nd.op_type.startswith("REF::"):
            key = nd.op_type[5:]
            if key not in prims:
                raise MindIRError("node %s refers to %s, which is not a primitive of the model (a sub-graph or a "
                                  "closure?)" % (nd.name, key))
            op_type = prims[key].op_type
            attrs = {a.name: _read_attr(a) for a in prims[key].attribute}
        else:
            op_type = nd.op_type
            attrs = {a.name: _read_attr(a) for a in nd.attribute}
        args = [value_of(i) for i in nd.input]
        args = [a for a in args if a is not _MONAD]          # side-effect tokens order nodes: the list order does
        if op_type == "TupleGetItem":
            node = g.create_node("call_function", operator.getitem, (args[0], int(args[1])), {})
        elif op_type == "MakeTuple":
            node = g.create_node("call_function", _make_tuple, tuple(args), {})
        elif op_type in ("Depend", "UpdateState", "Load"):
            env[out_name] = args[0] if args else _MONAD
            continue
        elif op_type == "Return":
            env[out_name] = args[0]
            continue
        else:
            node = g.create_node("call_function", _make_primitive(op_type, attrs), tuple(args), {})
            node.meta["primitive"] = op_type
        if nd.domain:
            node.meta["scope"] = nd.domain
        env[out_name] = node
    if not gp.output:
        raise MindIRError("the graph has no output")
    outs = [value_of(o.name) for o in gp.output]
    fg.output_node = g.output(outs[0] if len(outs) == 1 else tuple(outs))
    fg.input_positions = list(range(n_in))
    return LoadedGraph(fg)
