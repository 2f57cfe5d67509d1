"""Graph passes: dead-code elimination, common-subexpression elimination and the pass manager.

CSE merges identical pure nodes - notably the duplicate forward that ``loss = net(x); grads = grad(net)(x)``
traces twice, the way the reference's ``cse`` pass does after ``meta_fg_expand``
(ccsrc/frontend/optimizer/cse.cc; pass order in pipeline/jit/ps/pass.cc:489-527).  Nodes with side effects
(parameter updates, collectives, RNG) are never merged or removed.
"""
import operator
import os

import torch
import torch.fx as fx

from . import autodiff
from .ir import dump_graph

_IMPURE_NAMES = {"dropout", "rand", "randn", "randint", "bernoulli", "normal_", "uniform_", "multinomial",
                 "rand_like", "randn_like", "copy_", "add_", "sub_", "mul_", "div_", "zero_", "fill_", "set_"}


def _is_primitive(t):
    return hasattr(t, "name") and hasattr(t, "attrs") and hasattr(t, "_run")


def is_impure(node):
    if node.op != "call_function":
        return False
    t = node.target
    if t is autodiff.vjp:
        return True
    if getattr(t, "is_collective", False) or type(t).__name__ in ("Switch", "While"):
        return True
    if _is_primitive(t):
        if t._update_parameter:
            return True
        mod = type(t).__module__
        if mod.endswith("comm_ops") and not t.name.startswith("_Virtual"):
            return True
        return t.name in ("Dropout", "Print", "StandardNormal", "UniformReal", "UniformInt", "Multinomial")
    name = getattr(t, "__name__", "")
    return name in _IMPURE_NAMES or name.endswith("_") and not name.endswith("__")


def dead_code_elimination(fg):
    removed = 0
    for n in reversed(list(fg.graph.nodes)):
        if n.op in ("output", "placeholder"):
            continue
        if not n.users and not is_impure(n):
            fg.graph.erase_node(n)
            removed += 1
    return removed


def _key(a):
    if isinstance(a, fx.Node):
        return ("n", a.name)
    if isinstance(a, (tuple, list)):
        return (type(a).__name__,) + tuple(_key(x) for x in a)
    if isinstance(a, dict):
        return ("d",) + tuple((k, _key(v)) for k, v in sorted(a.items()))
    if isinstance(a, slice):
        return ("s", _key(a.start), _key(a.stop), _key(a.step))
    if isinstance(a, torch.Tensor):
        return ("t", id(a))
    try:
        hash(a)
        return ("c", type(a).__name__, a)
    except TypeError:
        return ("o", id(a))


def common_subexpression_elimination(fg):
    seen = {}
    merged = 0
    for n in list(fg.graph.nodes):
        if n.op != "call_function" or is_impure(n):
            continue
        t = n.target
        tk = ("prim", t.name, tuple(sorted((k, repr(v)) for k, v in t.attrs.items()))) if _is_primitive(t) else ("f", id(t))
        key = (tk, _key(n.args), _key(n.kwargs))
        prev = seen.get(key)
        if prev is None:
            seen[key] = n
            continue
        if n.meta.get("requires_vjp"):
            if prev.meta.get("requires_vjp") and any(
                    m.op == "call_function" and m.target is autodiff.vjp and m.args[0] == prev.name
                    for m in fg.graph.nodes):
                continue          # both copies are differentiated: each vjp node consumes its own saved forward
            prev.meta["requires_vjp"] = True
            # the vjp node refers to the forward node by name: redirect it
            for m in fg.graph.nodes:
                if m.op == "call_function" and m.target is autodiff.vjp and m.args[0] == n.name:
                    m.args = (prev.name,) + tuple(m.args[1:])
        n.replace_all_uses_with(prev)
        fg.graph.erase_node(n)
        merged += 1
    return merged


class PassManager:
    def __init__(self, name="opt"):
        self.name = name
        self.passes = []

    def add(self, name, fn):
        self.passes.append((name, fn))
        return self

    def run(self, fg, tag, save_level=0, path="."):
        changed = False
        for i, (name, fn) in enumerate(self.passes):
            c = fn(fg)
            changed = changed or bool(c)
            if save_level >= 2:
                dump_graph(fg, os.path.join(path, "%s_%02d_%s.ir" % (tag, i + 1, name)))
        return changed


def run_default_passes(fg, tag, save_level=0, path="."):
    """opt_a: simplification to a fixed point; opt_b: communication passes (merge, bucket fusion, hoisting, stream
    marking) with the effect chains they respect.  Pass order follows pipeline/jit/ps/pass.cc:424-527 in spirit:
    simplify first so that the communication passes see the final producers."""
    from . import opt_passes as O
    from .fusion import fuse_patterns
    pm = PassManager("opt_a")
    pm.add("cast_eliminate", O.cast_eliminate)
    pm.add("arithmetic_simplify", O.arithmetic_simplify)
    pm.add("cse", common_subexpression_elimination)
    pm.add("dce", dead_code_elimination)
    pm.add("fuse_patterns", lambda g: len(fuse_patterns(g)))
    for _ in range(4):
        if not pm.run(fg, tag, save_level, path):
            break
    from .. import context as _context
    if _context.get_context("enable_graph_kernel"):
        from .graph_kernel import fuse_elementwise
        pk = PassManager("graph_kernel")
        pk.add("fuse_elementwise", fuse_elementwise)
        pk.run(fg, tag + "_graph_kernel", save_level, path)
    pb = PassManager("opt_b")
    pb.add("merge_comm", O.merge_comm)
    pb.add("allreduce_fusion", O.allreduce_fusion)
    pb.add("comm_reorder", O.comm_reorder)
    pb.add("mark_comm_stream", O.mark_comm_stream)
    pb.run(fg, tag + "_comm", save_level, path)
    O.effect_chains(fg)
    if save_level:
        dump_graph(fg, os.path.join(path, "%s_validate.ir" % tag))
    return fg
