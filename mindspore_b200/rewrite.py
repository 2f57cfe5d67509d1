"""``rewrite``: edit a network as a list of call nodes and get a new network back.

    stree = SymbolTree.create(net)
    for node in stree.nodes():
        if node.get_instance_type() is nn.ReLU:
            new = Node.create_call_cell(nn.GELU(), targets=node.get_targets(), args=node.get_args(), name="gelu")
            stree.replace(node, [new])
    new_net = stree.get_network()

The tree is built from the source of ``construct`` with Python's ``ast``: every top-level statement becomes a
``Node`` - a call of a sub-cell (``x = self.conv(x)``), of a primitive / function, a plain Python statement, the
inputs, or the return.  Edits (``insert`` / ``replace`` / ``erase`` / ``set_arg``) work on that list;
``get_network`` regenerates ``construct`` from the nodes, compiles it and returns an instance of a new ``Cell``
subclass that shares the original sub-cells and parameters plus whatever cells the edit added; ``get_code``
returns the generated source.  Nested calls inside one statement are flattened into temporaries first
(``flatten=True``) so that each cell call is its own node.

Parity: python/mindspore/rewrite/api/{symbol_tree,node,scoped_value,node_type}.py and rewrite/parsers/* (the
reference keeps a full symbol table per module and also rewrites sub-trees; here a sub-cell's own construct can be
opened with ``SymbolTree.create(subcell)`` and put back with ``Node.create_call_cell``)."""
from __future__ import annotations

import ast
import inspect
import itertools
import textwrap
from enum import Enum

from .nn.cell import Cell

__all__ = ["SymbolTree", "Node", "NodeType", "ScopedValue", "ValueType"]


class NodeType(Enum):
    Unknown = 0
    CallCell = 1
    CallPrimitive = 2
    CallFunction = 3
    CallMethod = 4
    Python = 5
    Input = 6
    Output = 7
    Tree = 8
    CellContainer = 9
    MathOps = 10
    ControlFlow = 11


class ValueType(Enum):
    NamingValue = 0
    ConstantValue = 1


class ScopedValue:
    """An argument of a node: a variable name (optionally ``scope.name`` such as ``self.x``) or a constant."""

    def __init__(self, arg_type, scope="", value=None):
        self.type, self.scope, self.value = arg_type, scope, value

    @classmethod
    def create_naming_value(cls, name, scope=""):
        return cls(ValueType.NamingValue, scope, name)

    @classmethod
    def create_variable_value(cls, value):
        return cls(ValueType.ConstantValue, "", value)

    @staticmethod
    def create_name_values(names, scopes=None):
        scopes = scopes or [""] * len(names)
        return [ScopedValue.create_naming_value(n, s) for n, s in zip(names, scopes)]

    def code(self):
        if self.type is ValueType.NamingValue:
            return "%s.%s" % (self.scope, self.value) if self.scope else str(self.value)
        return repr(self.value)

    def __eq__(self, other):
        return isinstance(other, ScopedValue) and (self.type, self.scope, self.value) == (other.type, other.scope, other.value)

    def __hash__(self):
        return hash((self.type, self.scope, repr(self.value)))

    def __repr__(self):
        return "ScopedValue(%s)" % self.code()


def _to_scoped(v):
    if isinstance(v, ScopedValue):
        return v
    if isinstance(v, str):
        scope, _, name = v.rpartition(".")
        return ScopedValue.create_naming_value(name, scope)
    return ScopedValue.create_variable_value(v)


class Node:
    def __init__(self, node_type, name, targets=None, func=None, args=None, kwargs=None, instance=None, source=None):
        self._type, self._name = node_type, name
        self._targets = [_to_scoped(t) for t in (targets or [])]
        self._func = func                          # ScopedValue naming what is called (self.conv / ops.add / ...)
        self._args = [_to_scoped(a) for a in (args or [])]
        self._kwargs = {k: _to_scoped(v) for k, v in (kwargs or {}).items()}
        self._instance = instance
        self._source = source                      # verbatim statement for Python / control-flow nodes
        self._tree = None

    # ------------------------------------------------------------------ construction
    @staticmethod
    def create_call_cell(cell, targets, args=None, kwargs=None, name="", is_sub_net=False):
        if not isinstance(cell, Cell):
            raise TypeError("create_call_cell needs a Cell, got %s" % type(cell).__name__)
        name = name or type(cell).__name__.lower()
        return Node(NodeType.CallCell, name, targets, ScopedValue.create_naming_value(name, "self"), args, kwargs, cell)

    @staticmethod
    def create_call_function(function, targets, args=None, kwargs=None):
        name = getattr(function, "__name__", "fn")
        n = Node(NodeType.CallFunction, name, targets, ScopedValue.create_naming_value(name, "self"), args, kwargs,
                 function)
        return n

    # ------------------------------------------------------------------ queries
    def get_name(self):
        return self._name

    def get_node_type(self):
        return self._type

    def get_instance(self):
        return self._instance

    def get_instance_type(self):
        return type(self._instance) if self._instance is not None else None

    def get_targets(self):
        return list(self._targets)

    def get_args(self):
        return list(self._args)

    def get_kwargs(self):
        return dict(self._kwargs)

    def get_inputs(self):
        """Nodes whose targets this node reads."""
        if self._tree is None:
            return []
        names = {a.code() for a in list(self._args) + list(self._kwargs.values()) if a.type is ValueType.NamingValue}
        out = []
        for n in self._tree._nodes:
            if n is self:
                break
            if any(t.code() in names for t in n._targets):
                out.append(n)
        return out

    def get_users(self):
        if self._tree is None:
            return []
        mine = {t.code() for t in self._targets}
        seen, out = False, []
        for n in self._tree._nodes:
            if n is self:
                seen = True
                continue
            if seen and any(a.code() in mine for a in list(n._args) + list(n._kwargs.values())):
                out.append(n)
        return out

    def set_arg(self, index, arg):
        self._args[index] = _to_scoped(arg)

    def set_arg_by_node(self, arg_idx, src_node, out_idx=0):
        self._args[arg_idx] = src_node._targets[out_idx]

    def get_symbol_tree(self):
        return self._tree

    # ------------------------------------------------------------------ code
    def code(self):
        if self._type in (NodeType.Python, NodeType.ControlFlow, NodeType.Input, NodeType.MathOps):
            return self._source or ""
        if self._type is NodeType.Output:
            return "return " + ", ".join(a.code() for a in self._args)
        call = "%s(%s)" % (self._func.code(), ", ".join(
            [a.code() for a in self._args] + ["%s=%s" % (k, v.code()) for k, v in self._kwargs.items()]))
        if self._targets:
            return "%s = %s" % (", ".join(t.code() for t in self._targets), call)
        return call

    def __repr__(self):
        return "Node(%s, %s: %s)" % (self._type.name, self._name, self.code())


class _Flatten(ast.NodeTransformer):
    """Hoists nested ``self.<attr>(...)`` calls out of a statement into temporaries, innermost first."""

    def __init__(self, counter):
        self.pre, self.counter = [], counter

    def visit_Call(self, node):
        self.generic_visit(node)
        return node

    def hoist(self, stmt):
        self.pre = []
        value = stmt.value

        def rec(expr, top):
            for field, child in ast.iter_fields(expr):
                if isinstance(child, ast.AST):
                    setattr(expr, field, rec(child, False))
                elif isinstance(child, list):
                    setattr(expr, field, [rec(c, False) if isinstance(c, ast.AST) else c for c in child])
            if not top and isinstance(expr, ast.Call) and _is_self_attr(expr.func):
                name = "_t%d" % next(self.counter)
                self.pre.append(ast.Assign(targets=[ast.Name(id=name, ctx=ast.Store())], value=expr))
                return ast.Name(id=name, ctx=ast.Load())
            return expr
        stmt.value = rec(value, True)
        return self.pre + [stmt]


def _is_self_attr(func):
    return isinstance(func, ast.Attribute) and isinstance(func.value, ast.Name) and func.value.id == "self"


def _expr_to_scoped(e):
    if isinstance(e, ast.Name):
        return ScopedValue.create_naming_value(e.id)
    if isinstance(e, ast.Attribute) and isinstance(e.value, ast.Name):
        return ScopedValue.create_naming_value(e.attr, e.value.id)
    if isinstance(e, ast.Constant):
        return ScopedValue.create_variable_value(e.value)
    return ScopedValue(ValueType.NamingValue, "", ast.unparse(e))        # arbitrary expression, kept verbatim


class SymbolTree:
    def __init__(self, network, nodes, arg_names, func_globals):
        self._origin, self._nodes, self._arg_names, self._globals = network, nodes, arg_names, func_globals
        for n in nodes:
            n._tree = self
        self._added = {}

    # ------------------------------------------------------------------ parse
    @classmethod
    def create(cls, network, flatten=True):
        if not isinstance(network, Cell):
            raise TypeError("SymbolTree.create needs a Cell, got %s" % type(network).__name__)
        fn = type(network).construct
        src = textwrap.dedent(inspect.getsource(fn))
        fdef = ast.parse(src).body[0]
        arg_names = [a.arg for a in fdef.args.args][1:]
        if fdef.args.vararg or fdef.args.kwarg:
            raise NotImplementedError("rewrite: construct with *args / **kwargs is not supported")
        counter = itertools.count()
        stmts = []
        for st in fdef.body:
            if isinstance(st, ast.Expr) and isinstance(st.value, ast.Constant) and isinstance(st.value.value, str):
                continue                                    # docstring
            if flatten and isinstance(st, (ast.Assign, ast.Return)) and st.value is not None:
                stmts += _Flatten(counter).hoist(st)
            else:
                stmts.append(st)
        nodes = [Node(NodeType.Input, a, targets=[a], source="") for a in arg_names]
        used = set(arg_names)
        # single assignment: a name that is assigned again gets a fresh name, so users are unambiguous
        current, taken = {a: a for a in arg_names}, set(arg_names)

        class _Loads(ast.NodeTransformer):
            def visit_Name(self, node):
                if isinstance(node.ctx, ast.Load) and node.id in current:
                    return ast.copy_location(ast.Name(id=current[node.id], ctx=ast.Load()), node)
                return node

        for st in stmts:
            if isinstance(st, ast.Assign):
                st.value = _Loads().visit(st.value)
                t = st.targets[0]
                for e in (t.elts if isinstance(t, ast.Tuple) else [t]):
                    if isinstance(e, ast.Name):
                        fresh = cls._unique(e.id, taken)
                        current[e.id] = fresh
                        e.id = fresh
            else:
                st = _Loads().visit(st)
                for sub in ast.walk(st):
                    if isinstance(sub, ast.Name) and isinstance(sub.ctx, ast.Store):
                        current[sub.id] = sub.id
                        taken.add(sub.id)
            ast.fix_missing_locations(st)
            nodes.append(cls._node_of(st, network, used))
        return cls(network, nodes, arg_names, fn.__globals__)

    @staticmethod
    def _unique(base, used):
        name, i = base, 1
        while name in used:
            name, i = "%s_%d" % (base, i), i + 1
        used.add(name)
        return name

    @classmethod
    def _node_of(cls, st, network, used):
        if isinstance(st, ast.Return):
            vals = st.value.elts if isinstance(st.value, ast.Tuple) else ([st.value] if st.value is not None else [])
            return Node(NodeType.Output, "return", args=[_expr_to_scoped(v) for v in vals])
        if isinstance(st, (ast.If, ast.For, ast.While, ast.With, ast.Try)):
            return Node(NodeType.ControlFlow, cls._unique("control", used), source=ast.unparse(st))
        call = st.value if isinstance(st, (ast.Assign, ast.Expr)) else None
        if isinstance(call, ast.Call) and not any(isinstance(a, ast.Starred) for a in call.args):
            targets = []
            if isinstance(st, ast.Assign):
                t = st.targets[0]
                targets = [_expr_to_scoped(e) for e in (t.elts if isinstance(t, ast.Tuple) else [t])]
            args = [_expr_to_scoped(a) for a in call.args]
            kwargs = {k.arg: _expr_to_scoped(k.value) for k in call.keywords if k.arg}
            func = _expr_to_scoped(call.func)
            if _is_self_attr(call.func):
                inst = getattr(network, call.func.attr, None)
                from .ops.primitive import Primitive
                kind = NodeType.CallCell if isinstance(inst, Cell) else \
                    NodeType.CallPrimitive if isinstance(inst, Primitive) else NodeType.CallMethod
                return Node(kind, cls._unique(call.func.attr, used), targets, func, args, kwargs, inst)
            return Node(NodeType.CallFunction, cls._unique(ast.unparse(call.func).replace(".", "_"), used), targets, func,
                        args, kwargs, None)
        if isinstance(st, ast.Assign) and isinstance(st.value, ast.BinOp):
            t = st.targets[0]
            n = Node(NodeType.MathOps, cls._unique("math", used), source=ast.unparse(st))
            n._targets = [_expr_to_scoped(e) for e in (t.elts if isinstance(t, ast.Tuple) else [t])]
            return n
        return Node(NodeType.Python, cls._unique("python", used), source=ast.unparse(st))

    # ------------------------------------------------------------------ queries
    def nodes(self, all_nodes=False):
        return list(self._nodes)

    def get_node(self, name):
        for n in self._nodes:
            if n._name == name:
                return n
        return None

    def get_network_origin(self):
        return self._origin

    def unique_name(self, name="output"):
        return self._unique(name, {n._name for n in self._nodes} | {t.value for n in self._nodes for t in n._targets})

    # ------------------------------------------------------------------ edits
    def before(self, node):
        return ("before", self._resolve(node))

    def after(self, node):
        return ("after", self._resolve(node))

    def _resolve(self, node):
        n = self.get_node(node) if isinstance(node, str) else node
        if n is None or n not in self._nodes:
            raise ValueError("node %r is not in this tree" % (node,))
        return n

    def _adopt(self, node):
        names = {n._name for n in self._nodes}
        if node._name in names:
            node._name = self._unique(node._name, names)
        if node._type in (NodeType.CallCell, NodeType.CallFunction) and node._instance is not None and \
                node._func is not None and node._func.scope == "self":
            node._func = ScopedValue.create_naming_value(node._name, "self")
            self._added[node._name] = node._instance
        node._tree = self

    def insert(self, position, node):
        where, ref = position
        self._adopt(node)
        i = self._nodes.index(ref)
        self._nodes.insert(i if where == "before" else i + 1, node)
        return node

    def erase(self, node):
        n = self._resolve(node)
        if n.get_users():
            raise RuntimeError("node %s still has users: %s" % (n._name, [u._name for u in n.get_users()]))
        self._nodes.remove(n)
        n._tree = None
        return n

    def replace(self, old_node, new_nodes):
        old = self._resolve(old_node)
        i = self._nodes.index(old)
        self._nodes.pop(i)
        old._tree = None
        for k, n in enumerate(new_nodes):
            self._adopt(n)
            self._nodes.insert(i + k, n)
        return new_nodes[-1] if new_nodes else None

    # ------------------------------------------------------------------ code generation
    def get_code(self):
        cls_name = type(self._origin).__name__ + "Opt"
        lines = ["class %s(Cell):" % cls_name,
                 "    def __init__(self, origin, added):",
                 "        super().__init__()",
                 "        for k, v in origin.__dict__.items():",
                 "            if not k.startswith('__') and k not in ('_cells', '_params', '_ordered'):",
                 "                object.__setattr__(self, k, v)",
                 "        for k, v in list(origin._cells.items()):",
                 "            setattr(self, k, v)",
                 "        for k, v in list(origin._params.items()):",
                 "            setattr(self, k, v)",
                 "        for k, v in added.items():",
                 "            setattr(self, k, v) if isinstance(v, Cell) else object.__setattr__(self, k, v)",
                 "",
                 "    def construct(self, %s):" % ", ".join(self._arg_names)]
        body = []
        for n in self._nodes:
            code = n.code()
            if code:
                body += code.splitlines()
        lines += ["        " + ln for ln in (body or ["pass"])]
        return "\n".join(lines) + "\n"

    def print_node_tabulate(self, all_nodes=False):
        rows = ["%-14s %-20s %s" % (n._type.name, n._name, n.code().splitlines()[0] if n.code() else "") for n in self._nodes]
        print("\n".join(rows))

    def get_network(self):
        code = self.get_code()
        ns = dict(self._globals)
        ns["Cell"] = Cell
        exec(compile(code, "<rewrite:%s>" % type(self._origin).__name__, "exec"), ns)      # noqa: S102
        cls = ns[type(self._origin).__name__ + "Opt"]
        net = cls(self._origin, self._added)
        net._rewrite_source = code
        return net


# ------------------------------------------------------------------------------------------------ pattern engine
class PatternNode:
    """One node of a pattern: matches a tree node whose instance is of ``instance_type`` (None matches any), with
    ``inputs`` matched against the producers of that node's arguments (python/mindspore/rewrite/api/pattern_engine.py).
    """

    def __init__(self, pattern_node_name, instance_type=None, inputs=None):
        self._name = pattern_node_name
        self._type = instance_type
        self._inputs = list(inputs or [])

    @staticmethod
    def from_node(node):
        return PatternNode(node.get_name(), node.get_instance_type(),
                           [PatternNode.from_node(i) for i in node.get_inputs()])

    @staticmethod
    def create_pattern_from_list(type_list):
        """A chain: type_list[0] feeds type_list[1] feeds ...; returns the last (root) pattern node."""
        cur = None
        for i, t in enumerate(type_list):
            cur = PatternNode("pattern_%d" % i, t, [cur] if cur is not None else [])
        return cur

    def add_input(self, node):
        self._inputs.append(node)

    def set_inputs(self, inputs):
        self._inputs = list(inputs)

    def get_inputs(self):
        return list(self._inputs)

    def name(self):
        return self._name

    def type(self):
        return self._type

    def match(self, node):
        return self._type is None or (node.get_instance_type() is not None and
                                      issubclass(node.get_instance_type(), self._type))


class VarNode(PatternNode):
    """Matches any node (a wildcard input of a pattern)."""

    def __init__(self):
        super().__init__("placeholder", None, [])


class Replacement:
    """``build(pattern, is_chain_pattern, matched) -> [Node]``: the nodes that take the place of a match; the last
    one provides the value the matched root provided."""

    def build(self, pattern, is_chain_pattern, matched):
        raise NotImplementedError


class PatternEngine:
    """Finds every match of ``pattern`` (a PatternNode tree, or a list of types for a chain) in a SymbolTree and
    replaces it by what ``replacement.build`` returns.  Interior nodes of a match must have no users outside it."""

    def __init__(self, pattern, replacement=None):
        if isinstance(pattern, (list, tuple)):
            self._is_chain = True
            self._pattern = PatternNode.create_pattern_from_list(list(pattern))
        else:
            self._is_chain = False
            self._pattern = pattern
        self._replacement = replacement

    def pattern(self):
        return self._pattern

    def _match(self, pat, node, matched):
        if isinstance(pat, VarNode):
            return True
        if not pat.match(node):
            return False
        matched[pat.name()] = node
        inputs = node.get_inputs()
        pins = pat.get_inputs()
        if not pins:
            return True
        if len(pins) > len(inputs):
            return False
        return all(self._match(p, n, matched) for p, n in zip(pins, inputs))

    def apply(self, stree):
        """Returns True if anything was replaced."""
        changed = False
        for node in list(stree.nodes()):
            if node.get_symbol_tree() is None:
                continue
            matched = {}
            if not self._match(self._pattern, node, matched):
                continue
            inside = set(id(n) for n in matched.values())
            interior_ok = all(all(id(u) in inside for u in n.get_users()) for n in matched.values() if n is not node)
            if not interior_ok or self._replacement is None:
                continue
            new_nodes = self._replacement.build(self._pattern, self._is_chain, matched)
            if not new_nodes:
                continue
            stree.replace(node, list(new_nodes))
            for n in reversed([m for m in stree.nodes() if id(m) in inside]):
                if not n.get_users():
                    stree.erase(n)
            changed = True
        return changed


__all__ += ["PatternEngine", "PatternNode", "Replacement", "VarNode"]
