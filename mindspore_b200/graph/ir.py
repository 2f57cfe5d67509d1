"""Graph IR: a ``torch.fx.Graph`` in execution (ANF) order plus the side tables the passes need.

Node kinds: ``placeholder`` (graph input), ``get_attr`` (Parameter or constant tensor, ``meta['param']`` /
``meta['const']``), ``call_function`` (target is a Primitive instance, a fused-op function, a torch function,
or the ``vjp`` / ``accumulate`` markers of the autodiff pass) and ``output``.  Per-node metadata carries the
parallel annotations: ``strategy``, ``layout``, ``stage``, ``micro``, ``fusion``, ``forward_comm``.
Parity (role): mindspore/core/ir/anf.h (CNode/Parameter/ValueNode), func_graph.h, manager.h.
"""
import torch
import torch.fx as fx


class FuncGraph:
    def __init__(self, name="graph"):
        self.name = name
        self.graph = fx.Graph()
        self.params = {}
        self._param_nodes = {}
        self._n_const = 0
        self.input_positions = []
        self.example_outputs = None
        self.output_node = None
        self.text = None

    def param_node(self, p):
        n = self._param_nodes.get(id(p))
        if n is None:
            key = p.name
            if key in self.params and self.params[key] is not p:
                key = "%s#%d" % (p.name, len(self.params))
            n = self.graph.create_node("get_attr", "param::" + key)
            n.meta["param"] = p
            self.params[key] = p
            self._param_nodes[id(p)] = n
        return n

    def const_node(self, t):
        self._n_const += 1
        n = self.graph.create_node("get_attr", "const::%d" % self._n_const)
        n.meta["const"] = t
        return n

    def set_output(self, structure, example):
        self.output_node = self.graph.output(structure)

    def nodes(self):
        return list(self.graph.nodes)

    def users(self, node):
        return list(node.users)

    def primitive_nodes(self, name=None):
        out = []
        for n in self.graph.nodes:
            if n.op == "call_function" and hasattr(n.target, "name") and hasattr(n.target, "attrs"):
                if name is None or n.target.name == name:
                    out.append(n)
        return out

    def count(self, name):
        return len(self.primitive_nodes(name))

    def to_text(self):
        return graph_to_text(self)


def _target_name(t):
    if hasattr(t, "name") and hasattr(t, "attrs"):
        attrs = {k: v for k, v in t.attrs.items() if k not in ("input_names", "output_names")}
        return "Prim::%s%s" % (t.name, attrs if attrs else "")
    mod = getattr(t, "__module__", "") or ""
    return "%s.%s" % (mod, getattr(t, "__qualname__", getattr(t, "__name__", repr(t))))


def _fmt(a):
    if isinstance(a, fx.Node):
        return "%" + a.name
    if isinstance(a, (tuple, list)):
        return "(" + ", ".join(_fmt(x) for x in a) + ")"
    if isinstance(a, dict):
        return "{" + ", ".join("%s=%s" % (k, _fmt(v)) for k, v in a.items()) + "}"
    if isinstance(a, torch.dtype):
        return str(a)
    r = repr(a)
    return r if len(r) < 60 else r[:57] + "..."


def graph_to_text(fg):
    lines = ["# graph %s" % fg.name]
    for n in fg.graph.nodes:
        meta = {k: v for k, v in n.meta.items() if k in ("strategy", "layout", "stage", "micro", "fusion",
                                                        "forward_comm", "primitive", "vjp_of", "requires_vjp")}
        ann = ("  # " + ", ".join("%s=%s" % kv for kv in meta.items())) if meta else ""
        if "abstract" in n.meta:
            ann = "  : %r%s" % (n.meta["abstract"], ann)
        if n.op == "placeholder":
            lines.append("%%%s = Input %s%s" % (n.name, n.meta.get("example", ""), ann))
        elif n.op == "get_attr":
            p = n.meta.get("param")
            desc = "Param[%s %s %s]" % (p.name, tuple(p.shape), p.dtype) if p is not None else \
                "Const[%s]" % (tuple(n.meta["const"].shape),)
            lines.append("%%%s = %s%s" % (n.name, desc, ann))
        elif n.op == "call_function":
            lines.append("%%%s = %s(%s%s)%s" % (n.name, _target_name(n.target), ", ".join(_fmt(a) for a in n.args),
                                                 (", " + _fmt(n.kwargs)) if n.kwargs else "", ann))
        elif n.op == "output":
            lines.append("return %s" % _fmt(n.args[0]))
    return "\n".join(lines) + "\n"


def dump_graph(fg, path):
    import os
    os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
    with open(path, "w") as f:
        f.write(graph_to_text(fg))
