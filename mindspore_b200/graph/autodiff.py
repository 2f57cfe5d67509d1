"""IR-level reverse-mode autodiff.

For the forward nodes of a differentiated region this pass appends, in reverse order, one ``vjp`` node per
forward node (it maps the output gradient to the gradients of the node's tensor inputs) and ``accumulate``
nodes where a value has several users.  At run time a ``vjp`` node evaluates the primitive's own backward rule:
the forward node ran with detached inputs under ``enable_grad``, so its local autograd tape *is* the
primitive's bprop - for communication primitives that is the dual collective (AllGather <-> ReduceScatter,
AllReduce <-> AllReduce, _MirrorOperator -> AllReduce ...), which therefore shows up as an explicit backward
node that scheduling passes can move.

Parity (role): ccsrc/frontend/optimizer/ad/dfunctor.cc (J expansion), kprim.cc (per-primitive bprop),
ops/_grad_experimental/grad_comm_ops.py (rules for the communication primitives).
"""
import operator

import torch
import torch.fx as fx


def vjp(fwd_name, out_grad):  # executed by graph.executor, which owns the saved forward values
    raise RuntimeError("vjp marker must be run by GraphExecutor")


def accumulate(*grads):
    out = None
    for g in grads:
        if g is None:
            continue
        out = g if out is None else out + g
    return out


def ones_like(x):
    return torch.ones_like(x)


def zeros_like_if_none(g, ref):
    return torch.zeros_like(ref.detach()) if g is None else g


def grad_or_none(g, ref):
    """The gradient as it came out of reverse mode, ``None`` included (an operator that adds its weight gradient
    into the parameter's accumulator hands back nothing): for callers that fold gradients themselves and must not
    pay a zero tensor of every weight's size per run."""
    return g


def seed_like(sens, ref):
    if isinstance(sens, torch.Tensor):
        s = sens.to(ref.dtype)
        return s.expand_as(ref) if s.shape != ref.shape else s
    return torch.full_like(ref, float(sens))


def _tensor_arg_nodes(node):
    out = []

    def visit(a):
        if isinstance(a, fx.Node):
            out.append(a)
        elif isinstance(a, (tuple, list)):
            for x in a:
                visit(x)
        elif isinstance(a, dict):
            for x in a.values():
                visit(x)
        elif isinstance(a, slice):
            visit(a.start), visit(a.stop), visit(a.step)

    visit(node.args)
    visit(node.kwargs)
    return out


def build_backward(fg, fwd_nodes, out_nodes, target_nodes, seeds=None, none_as_zero=True):
    g = fg.graph
    fwd_set = set(fwd_nodes)
    for n in fwd_nodes:
        if n.op == "call_function" and n.target is not operator.getitem:
            n.meta["requires_vjp"] = True
    contrib = {}
    slot_grads = {}

    def add(node, grad_node):
        contrib.setdefault(node, []).append(grad_node)

    for i, o in enumerate(out_nodes):
        if seeds is None:
            add(o, g.call_function(ones_like, (o,)))
        else:
            s = seeds[i] if i < len(seeds) else seeds[-1]
            add(o, g.call_function(seed_like, (s, o)))

    def total(node):
        lst = contrib.get(node)
        if not lst:
            return None
        return lst[0] if len(lst) == 1 else g.call_function(accumulate, tuple(lst))

    for n in reversed(fwd_nodes):
        if n.op != "call_function":
            continue
        if n.target is operator.getitem and isinstance(n.args[0], fx.Node) and n.args[0] in fwd_set:
            gn = total(n)
            if gn is not None:
                slot_grads.setdefault(n.args[0], {})[n.args[1]] = gn
            continue
        gn = total(n)
        slots = slot_grads.get(n)
        if gn is None and not slots:
            continue
        ins = _tensor_arg_nodes(n)
        if not ins:
            continue
        spec = gn if not slots else dict(slots)
        v = g.call_function(vjp, (n.name, spec))
        v.meta["vjp_of"] = n.name
        prim = n.meta.get("primitive")
        if prim:
            v.meta["primitive"] = "Grad" + prim
        for i, inp in enumerate(ins):
            add(inp, g.call_function(operator.getitem, (v, i)))
        n.meta["vjp_inputs"] = [x.name for x in ins]
    grads = []
    for t in target_nodes:
        gn = total(t)
        grads.append(g.call_function(zeros_like_if_none if none_as_zero else grad_or_none, (gn, t)))
    return grads
