"""Serialised graphs ("MindIR" role): ``export(net, *inputs, file_name=..., file_format="MINDIR")`` writes the traced
forward graph with its weights into one file; ``load(file)`` gives back an executable graph for ``nn.GraphCell``.

File layout: magic ``MSB200IR`` | u32 version | u64 header length | JSON header | tensor blobs (64-byte aligned).
The header lists the nodes in execution order - placeholders, parameters / constants (by blob index), primitive
calls (class name + constructor attributes + encoded arguments), ``getitem`` and the output structure.  Loading
rebuilds a ``FuncGraph`` (torch.fx graph of ``Primitive`` nodes) and runs it with the ordinary ``GraphExecutor``, so
a loaded graph behaves like a compiled one, CUDA-graph replay included.

The reference stores the same information as protobuf (``mind_ir.proto``: ModelProto / GraphProto / NodeProto /
TensorProto; writer ccsrc/transform/express_ir/mindir_exporter.cc, reader core/load_mindir/load_model.cc,
``nn.GraphCell`` python/mindspore/nn/cell.py:2554)."""
from __future__ import annotations

import inspect
import json
import operator
import struct

import numpy as np
import torch

from .ir import FuncGraph

MAGIC = b"MSB200IR"
VERSION = 1
_ALIGN = 64

_DTYPES = {str(d).replace("torch.", ""): d for d in (
    torch.float32, torch.float64, torch.float16, torch.bfloat16, torch.int8, torch.int16, torch.int32, torch.int64,
    torch.uint8, torch.bool, torch.complex64)}
_BUILTINS = {"getitem": operator.getitem, "add": operator.add, "sub": operator.sub, "mul": operator.mul,
             "truediv": operator.truediv, "neg": operator.neg, "matmul": operator.matmul, "pow": operator.pow}
_BUILTIN_NAMES = {v: k for k, v in _BUILTINS.items()}


class MindIRError(ValueError):
    pass


_SEARCH = ("torch.nn.functional", "torch", "torch.special", "torch.linalg", "torch.fft", "operator", "math")
_ALLOWED_ROOTS = ("torch", "operator", "math", "mindspore_b200")


def _callable_record(fn):
    """Names a function of torch / operator / this package so that loading can find it again."""
    objclass = getattr(fn, "__objclass__", None)
    name = getattr(fn, "__name__", None)
    if objclass is not None and name and hasattr(torch.Tensor, name):
        return {"method": name}
    mod = getattr(fn, "__module__", None) or ""
    qual = getattr(fn, "__qualname__", None) or name
    if not name:
        raise MindIRError("%r has no name and cannot be stored" % (fn,))
    rec = {"fn": qual, "module": mod}
    if _resolve_callable(rec) is not fn:
        # builtins report private modules (torch._C._nn.linear): store the public alias instead
        for cand in _SEARCH:
            import importlib
            if getattr(importlib.import_module(cand), name, None) is fn:
                return {"fn": name, "module": cand}
        raise MindIRError("function %s.%s cannot be found again by name" % (mod, qual))
    return rec


def _resolve_callable(rec):
    import importlib
    if "method" in rec:
        return getattr(torch.Tensor, rec["method"])
    mod = rec.get("module") or ""
    if mod.split(".")[0] not in _ALLOWED_ROOTS:
        return None
    try:
        obj = importlib.import_module(mod)
    except ImportError:
        return None
    for part in rec["fn"].split("."):
        obj = getattr(obj, part, None)
        if obj is None:
            return None
    return obj


# ------------------------------------------------------------------------------------------------ value coding
class _Blobs:
    def __init__(self):
        self.items, self.index = [], {}

    def add(self, t):
        key = id(t)
        if key not in self.index:
            self.index[key] = len(self.items)
            self.items.append(t)
        return self.index[key]


def _enc(v, node_ids, blobs):
    import torch.fx as fx
    if isinstance(v, fx.Node):
        return {"n": node_ids[v]}
    if isinstance(v, torch.Tensor):
        return {"t": blobs.add(v)}
    if isinstance(v, (bool, int, float, str)) or v is None:
        return v
    if isinstance(v, (np.integer, np.floating, np.bool_)):
        return v.item()
    if isinstance(v, tuple):
        return {"tuple": [_enc(x, node_ids, blobs) for x in v]}
    if isinstance(v, list):
        return {"list": [_enc(x, node_ids, blobs) for x in v]}
    if isinstance(v, dict):
        return {"dict": [[_enc(k, node_ids, blobs), _enc(x, node_ids, blobs)] for k, x in v.items()]}
    if isinstance(v, slice):
        return {"slice": [_enc(v.start, node_ids, blobs), _enc(v.stop, node_ids, blobs), _enc(v.step, node_ids, blobs)]}
    if v is Ellipsis:
        return {"ellipsis": 1}
    if isinstance(v, torch.dtype):
        return {"dtype": str(v).replace("torch.", "")}
    if isinstance(v, torch.Size):
        return {"tuple": [int(x) for x in v]}
    if isinstance(v, np.ndarray):
        return {"t": blobs.add(torch.from_numpy(np.ascontiguousarray(v)))}
    raise MindIRError("value of type %s cannot be stored in a graph file" % type(v).__name__)


def _dec(v, nodes, tensors):
    if not isinstance(v, dict):
        return v
    if "n" in v:
        return nodes[v["n"]]
    if "t" in v:
        return tensors[v["t"]]
    if "tuple" in v:
        return tuple(_dec(x, nodes, tensors) for x in v["tuple"])
    if "list" in v:
        return [_dec(x, nodes, tensors) for x in v["list"]]
    if "dict" in v:
        return {_dec(k, nodes, tensors): _dec(x, nodes, tensors) for k, x in v["dict"]}
    if "slice" in v:
        return slice(*[_dec(x, nodes, tensors) for x in v["slice"]])
    if "ellipsis" in v:
        return Ellipsis
    if "dtype" in v:
        return _DTYPES[v["dtype"]]
    raise MindIRError("unknown value record %r" % (v,))


def _prim_record(prim, node_ids, blobs):
    cls = type(prim)
    attrs = {}
    for k, val in getattr(prim, "attrs", {}).items():
        try:
            attrs[k] = _enc(val, node_ids, blobs)
        except MindIRError:
            continue                                  # callables and the like are not part of the constructor record
    rec = {"cls": cls.__name__, "module": cls.__module__, "attrs": attrs}
    for extra in ("in_strategy", "out_strategy"):
        if getattr(prim, extra, None) is not None:
            rec[extra] = _enc(getattr(prim, extra), node_ids, blobs)
    return rec


def _make_prim(rec, tensors):
    import importlib
    try:
        if not rec["module"].startswith("mindspore_b200."):
            raise ImportError(rec["module"])            # a graph file may only name this package's primitives
        mod = importlib.import_module(rec["module"])
        cls = getattr(mod, rec["cls"])
    except (ImportError, AttributeError):
        from ..ops import operations as P
        cls = getattr(P, rec["cls"], None)
        if cls is None:
            raise MindIRError("the graph uses primitive %s, which this build does not define" % rec["cls"])
    attrs = {k: _dec(v, None, tensors) for k, v in rec["attrs"].items()}
    init = getattr(cls.__init__, "decorated_func", cls.__init__)
    params = [p for p in list(inspect.signature(init).parameters.values())[1:]
              if p.kind in (p.POSITIONAL_OR_KEYWORD, p.KEYWORD_ONLY)]
    kwargs = {p.name: attrs[p.name] for p in params if p.name in attrs}
    prim = cls(**kwargs)
    for k, v in attrs.items():
        if k not in kwargs and hasattr(prim, "add_prim_attr"):
            prim.add_prim_attr(k, v)
    if rec.get("in_strategy") is not None and hasattr(prim, "shard"):
        prim.shard(_dec(rec["in_strategy"], None, tensors),
                   _dec(rec["out_strategy"], None, tensors) if rec.get("out_strategy") is not None else None)
    return prim


# ------------------------------------------------------------------------------------------------ save
def save_mindir(fg, path, producer="mindspore_b200"):
    from . import autodiff
    nodes = list(fg.graph.nodes)
    node_ids = {n: i for i, n in enumerate(nodes)}
    blobs = _Blobs()
    recs = []
    for n in nodes:
        r = {"op": n.op, "name": n.name}
        for key in ("shape", "dtype", "stage", "strategy"):
            if key in n.meta:
                try:
                    r.setdefault("meta", {})[key] = _enc(n.meta[key], node_ids, blobs)
                except MindIRError:
                    pass
        if n.op == "placeholder":
            pass
        elif n.op == "get_attr":
            if "param" in n.meta:
                p = n.meta["param"]
                r.update(kind="param", pname=n.target.split("::", 1)[1], blob=blobs.add(p),
                         requires_grad=bool(getattr(p, "requires_grad", False)))
            else:
                r.update(kind="const", blob=blobs.add(n.meta["const"]))
        elif n.op == "call_function":
            if n.target is autodiff.vjp:
                raise MindIRError("only forward graphs can be exported (found a gradient node)")
            if n.target in _BUILTIN_NAMES:
                r["builtin"] = _BUILTIN_NAMES[n.target]
            elif hasattr(n.target, "name") and hasattr(n.target, "attrs"):
                r["prim"] = _prim_record(n.target, node_ids, blobs)
            elif callable(n.target):
                r["callable"] = _callable_record(n.target)
            else:
                raise MindIRError("node %s calls %r, which cannot be stored" % (n.name, n.target))
            r["args"] = _enc(tuple(n.args), node_ids, blobs)
            r["kwargs"] = _enc(dict(n.kwargs), node_ids, blobs)
        elif n.op == "output":
            r["args"] = _enc(n.args[0], node_ids, blobs)
        else:
            raise MindIRError("node kind %s is not supported in graph files" % n.op)
        recs.append(r)
    tensors, offset = [], 0
    payload = []
    for t in blobs.items:
        plain = t.detach().to("cpu").contiguous()
        raw = plain.view(torch.uint8).numpy().tobytes() if plain.dtype == torch.bfloat16 else plain.numpy().tobytes()
        pad = (-offset) % _ALIGN
        offset += pad
        payload.append(b"\0" * pad)
        tensors.append({"dtype": str(plain.dtype).replace("torch.", ""), "shape": list(plain.shape), "offset": offset,
                        "nbytes": len(raw)})
        payload.append(raw)
        offset += len(raw)
    header = json.dumps({"producer": producer, "name": fg.name, "nodes": recs, "tensors": tensors,
                         "input_positions": list(fg.input_positions)}).encode()
    with open(path, "wb") as f:
        f.write(MAGIC)
        f.write(struct.pack("<IQ", VERSION, len(header)))
        f.write(header)
        f.write(b"\0" * ((-(len(MAGIC) + 12 + len(header))) % _ALIGN))
        for chunk in payload:
            f.write(chunk)
    return path


# ------------------------------------------------------------------------------------------------ load
class LoadedGraph:
    """Executable graph read from a file: call it with the network inputs; ``params`` maps names to tensors."""

    def __init__(self, fg):
        from ..common.parameter import Parameter
        from .executor import GraphExecutor
        self.fg = fg
        self.name = fg.name
        self.params = fg.params
        self._exec = GraphExecutor(fg)
        self._Parameter = Parameter

    def __call__(self, *inputs):
        positions = self.fg.input_positions or list(range(len(inputs)))
        tensors = [inputs[i] for i in positions] if len(positions) <= len(inputs) else list(inputs)
        out = self._exec.run(tensors)
        from .executor import _wrap
        return _wrap(out)

    def set_param(self, name, value):
        if name not in self.params:
            raise KeyError("the graph has no parameter named %r" % name)
        with torch.no_grad():
            self.params[name].copy_(torch.as_tensor(value))

    def get_parameters(self):
        return list(self.params.values())

    def to_text(self):
        return self.fg.to_text()


def load_mindir(path):
    from ..common.parameter import Parameter
    from ..common.tensor import Tensor
    with open(path, "rb") as f:
        data = f.read()
    if data[:8] != MAGIC:
        raise MindIRError("%s is not a graph file of this framework (bad magic)" % path)
    version, hlen = struct.unpack_from("<IQ", data, 8)
    if version != VERSION:
        raise MindIRError("graph file version %d is not supported (expected %d)" % (version, VERSION))
    header = json.loads(data[20:20 + hlen].decode())
    base = 20 + hlen
    base += (-base) % _ALIGN
    tensors = []
    for t in header["tensors"]:
        dt = _DTYPES[t["dtype"]]
        raw = bytearray(data[base + t["offset"]:base + t["offset"] + t["nbytes"]])
        if dt == torch.bfloat16:
            ten = torch.frombuffer(raw, dtype=torch.uint8).view(torch.bfloat16).reshape(t["shape"]) if raw else \
                torch.empty(t["shape"], dtype=dt)
        else:
            ten = torch.frombuffer(raw, dtype=dt).reshape(t["shape"]) if raw else torch.empty(t["shape"], dtype=dt)
        tensors.append(ten.clone())
    fg = FuncGraph(header.get("name", "graph"))
    g = fg.graph
    nodes = []
    for r in header["nodes"]:
        op = r["op"]
        if op == "placeholder":
            n = g.placeholder(r["name"])
        elif op == "get_attr":
            if r["kind"] == "param":
                p = Parameter(Tensor(tensors[r["blob"]]), name=r["pname"].split("#")[0],
                              requires_grad=r.get("requires_grad", True))
                n = g.create_node("get_attr", "param::" + r["pname"])
                n.meta["param"] = p
                fg.params[r["pname"]] = p
            else:
                n = g.create_node("get_attr", "const::%d" % len(nodes))
                n.meta["const"] = tensors[r["blob"]]
        elif op == "call_function":
            if "builtin" in r:
                target = _BUILTINS[r["builtin"]]
            elif "callable" in r:
                target = _resolve_callable(r["callable"])
                if target is None:
                    raise MindIRError("the graph calls %r, which is not available here" % (r["callable"],))
            else:
                target = _make_prim(r["prim"], tensors)
            n = g.create_node("call_function", target, _dec(r["args"], nodes, tensors), _dec(r["kwargs"], nodes, tensors))
        elif op == "output":
            n = g.output(_dec(r["args"], nodes, tensors))
            fg.output_node = n
        else:
            raise MindIRError("unknown node kind %r" % op)
        for k, v in r.get("meta", {}).items():
            n.meta[k] = _dec(v, nodes, tensors)
        nodes.append(n)
    fg.input_positions = header.get("input_positions", [])
    return LoadedGraph(fg)
