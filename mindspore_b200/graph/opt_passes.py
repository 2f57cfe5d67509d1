"""Optimisation and scheduling passes over the traced graph.

* ``cast_eliminate``       Cast to the dtype a value already has; widening cast followed by a cast back.
* ``arithmetic_simplify``  x * 1, x / 1, x + 0, x - 0, Neg(Neg(x)), Transpose o Transpose = identity,
                           Reshape o Reshape -> one Reshape (ccsrc/frontend/optimizer/irpass/arithmetic_simplify.cc,
                           cast_eliminate.cc, transpose_eliminate.cc, reshape_eliminate.cc).
* ``merge_comm``           identical collectives on the same value and group become one
                           (ccsrc/frontend/parallel/pass/merge_comm.cc).
* ``allreduce_fusion``     gradient all-reduces get fusion ids by walking them in graph order and closing a bucket
                           when it reaches the ``comm_fusion`` threshold; all-reduces of one bucket (same group, op
                           and dtype) are replaced by ONE all-reduce of the concatenated buffer plus slices
                           (ccsrc/frontend/parallel/allreduce_fusion/allreduce_fusion.cc:82-176,
                           backend/common/pass/communication_op_fusion.cc:88-146).
* ``comm_reorder``         collectives are hoisted to right after the value they wait for; what consumes a
                           collective's result is sunk as late as its own users allow - independent compute ends up
                           between issue and first use, where the executor's communication stream overlaps it
                           (ccsrc/frontend/parallel/pass/overlap_grad_comm.cc, comp_comm_scheduling.cc).

Side effects.  Nodes that write state or communicate are *effect nodes*.  ``effect_chains`` gives each the effect
node it must stay behind (``node.meta['after']``): collectives form one chain (every rank must issue them in the
same order), writes and reads of one parameter form a chain per parameter.  No pass moves a node across its chain
predecessor - the job of the reference's auto-monad edges (pipeline/jit/ps/static_analysis/auto_monad.cc).
"""
from __future__ import annotations

import operator

import torch
import torch.fx as fx

from . import autodiff
from .passes import _is_primitive, is_impure

_WIDTH = {torch.bool: 0, torch.uint8: 1, torch.int8: 1, torch.int16: 2, torch.int32: 3, torch.int64: 4,
          torch.bfloat16: 5, torch.float16: 5, torch.float32: 6, torch.float64: 7}


def _prim_name(n):
    return n.target.name if n.op == "call_function" and _is_primitive(n.target) else None


def _fname(n):
    return getattr(n.target, "__name__", "") if n.op == "call_function" else ""


def _dtype(n):
    return n.meta.get("dtype") if isinstance(n, fx.Node) else None


def _shape(n):
    return n.meta.get("shape") if isinstance(n, fx.Node) else None


def _vjp_of(fg, node):
    for m in fg.graph.nodes:
        if m.op == "call_function" and m.target is autodiff.vjp and m.args[0] == node.name:
            return m
    return None


def _differentiated(fg, node):
    return bool(node.meta.get("requires_vjp")) and _vjp_of(fg, node) is not None


def _replace(fg, node, by):
    """``node`` computes the identity of ``by``: uses move to ``by``; if the backward graph holds a vjp node for it,
    the gradient of its (only tensor) input is the incoming gradient itself."""
    if by.op == "get_attr" and "param" in by.meta:
        # x * 1 of a parameter is a snapshot of its current value: replacing it by the parameter itself would make
        # later readers see writes (Assign, optimizer updates) that happen in between
        return False
    v = _vjp_of(fg, node) if node.meta.get("requires_vjp") else None
    if v is not None:
        spec = v.args[1]
        if not isinstance(spec, fx.Node):
            return False
        for u in list(v.users):
            u.replace_all_uses_with(spec)
            fg.graph.erase_node(u)
        fg.graph.erase_node(v)
    node.replace_all_uses_with(by)
    fg.graph.erase_node(node)
    return True


# ------------------------------------------------------------------------------------------------ casts
def _cast_target(n):
    """(input node, dtype) when ``n`` is a dtype conversion, else None."""
    if n.op != "call_function" or not n.args or not isinstance(n.args[0], fx.Node):
        return None
    if _prim_name(n) == "Cast" and len(n.args) >= 2 and isinstance(n.args[1], torch.dtype):
        return n.args[0], n.args[1]
    name = _fname(n)
    if name == "to" and len(n.args) == 2 and isinstance(n.args[1], torch.dtype) and not n.kwargs:
        return n.args[0], n.args[1]
    simple = {"float": torch.float32, "bfloat16": torch.bfloat16, "half": torch.float16, "double": torch.float64}
    if name in simple and len(n.args) == 1 and not n.kwargs:
        return n.args[0], simple[name]
    return None


def cast_eliminate(fg):
    changed = 0
    for n in list(fg.graph.nodes):
        ct = _cast_target(n)
        if ct is None:
            continue
        src, dt = ct
        if _dtype(src) == dt:
            changed += bool(_replace(fg, n, src))
            continue
        inner = _cast_target(src)
        if inner is not None:
            src2, mid = inner
            s2 = _dtype(src2)
            # x -> wider -> dt : the detour through a type that holds every value of x exactly is the identity
            if s2 is not None and s2 in _WIDTH and mid in _WIDTH and _WIDTH[mid] > _WIDTH[s2] and \
                    (mid.is_floating_point or not s2.is_floating_point):
                if _differentiated(fg, n) or _differentiated(fg, src):
                    continue               # the backward graph routes gradients through both casts
                if s2 == dt:
                    changed += bool(_replace(fg, n, src2))
                else:
                    n.args = (src2,) + tuple(n.args[1:])
                    changed += 1
    return changed


# ------------------------------------------------------------------------------------------------ arithmetic
def _is_number(a, v):
    return isinstance(a, (int, float)) and not isinstance(a, bool) and float(a) == v


def _same_result(n, x):
    """Replacing n by x keeps shape and dtype."""
    return isinstance(x, fx.Node) and _shape(n) is not None and _shape(n) == _shape(x) and _dtype(n) == _dtype(x)


def arithmetic_simplify(fg):
    changed = 0
    for n in list(fg.graph.nodes):
        if n.op != "call_function" or is_impure(n) or n.kwargs:
            continue
        name = _prim_name(n) or _fname(n).strip("_")
        a = n.args
        if name in ("Mul", "mul", "RealDiv", "Div", "div", "truediv") and len(a) == 2:
            if _is_number(a[1], 1.0) and _same_result(n, a[0]):
                changed += bool(_replace(fg, n, a[0]))
            elif name in ("Mul", "mul") and _is_number(a[0], 1.0) and _same_result(n, a[1]):
                changed += bool(_replace(fg, n, a[1]))
        elif name in ("Add", "add", "Sub", "sub") and len(a) == 2:
            if _is_number(a[1], 0.0) and _same_result(n, a[0]):
                changed += bool(_replace(fg, n, a[0]))
            elif name in ("Add", "add") and _is_number(a[0], 0.0) and _same_result(n, a[1]):
                changed += bool(_replace(fg, n, a[1]))
        elif name in ("Neg", "neg") and len(a) == 1 and isinstance(a[0], fx.Node):
            inner = a[0]
            if inner.op == "call_function" and (_prim_name(inner) or _fname(inner)) in ("Neg", "neg") and \
                    not is_impure(inner) and not _differentiated(fg, n) and not _differentiated(fg, inner):
                changed += bool(_replace(fg, n, inner.args[0]))
        elif name == "Transpose" and len(a) == 2 and isinstance(a[0], fx.Node) and _prim_name(a[0]) == "Transpose" \
                and not _differentiated(fg, n) and not _differentiated(fg, a[0]):
            p2, p1 = tuple(a[1]), tuple(a[0].args[1])
            comp = tuple(p1[i] for i in p2)
            if comp == tuple(range(len(comp))):
                changed += bool(_replace(fg, n, a[0].args[0]))
            else:
                n.args = (a[0].args[0], comp); changed += 1
        elif name == "Reshape" and len(a) == 2 and isinstance(a[0], fx.Node) and _prim_name(a[0]) == "Reshape" \
                and "forward_comm" not in n.meta and "layout" not in a[0].meta \
                and not _differentiated(fg, n) and not _differentiated(fg, a[0]):
            n.args = (a[0].args[0], a[1]); changed += 1
    return changed


# ------------------------------------------------------------------------------------------------ collectives
def is_collective(n):
    if n.op != "call_function":
        return False
    t = n.target
    if getattr(t, "is_collective", False):
        return True
    if _is_primitive(t):
        return type(t).__module__.endswith("comm_ops") and not t.name.startswith("_Virtual")
    return False


def _comm_key(n):
    t = n.target
    if getattr(t, "is_collective", False):
        return (t.__name__,) + tuple(("n", a.name) if isinstance(a, fx.Node) else ("c", repr(a)) for a in n.args)
    if _is_primitive(t):
        return ("prim", t.name, getattr(t, "group", None), getattr(t, "op", None),
                tuple(sorted((k, repr(v)) for k, v in t.attrs.items() if k not in ("input_names", "output_names")))) + \
            tuple(("n", a.name) if isinstance(a, fx.Node) else ("c", repr(a)) for a in n.args)
    return None


def merge_comm(fg):
    """Out-of-place collectives with identical inputs, group and attributes are performed once."""
    seen, merged = {}, 0
    for n in list(fg.graph.nodes):
        if not is_collective(n):
            continue
        name = _prim_name(n) or _fname(n)
        if name in ("all_reduce_node", "Send", "Receive", "Barrier", "Broadcast", "_MirrorOperator",
                    "_MirrorMicroStepOperator", "_MirrorMiniStepOperator"):
            continue                       # in-place, point-to-point or carrying a backward effect: never merged
        key = _comm_key(n)
        prev = seen.get(key)
        if prev is None:
            seen[key] = n
            continue
        _replace(fg, n, prev)
        merged += 1
    return merged


def _numel(n):
    s = _shape(n)
    if s is None:
        return 0
    k = 1
    for d in s:
        k *= int(d)
    return k


def fused_all_reduce(op, gname, sizes, *tensors):
    """ONE all-reduce for a bucket of tensors: flatten + concatenate, reduce, write the slices back in place."""
    from ..communication import comm_func as CF
    flat = torch.cat([t.reshape(-1) for t in tensors])
    CF.all_reduce_node(flat, op, gname)
    off = 0
    with torch.no_grad():
        for t, n in zip(tensors, sizes):
            t.copy_(flat[off:off + n].view(t.shape))
            off += n
    return tensors


fused_all_reduce.is_collective = True


def allreduce_fusion(fg, threshold_bytes=None):
    """In-place all-reduce nodes (``all_reduce_node``) over the same group / op / dtype are grouped in graph order
    into buckets of at least ``threshold_bytes`` (default: the ``comm_fusion`` all-reduce threshold of the
    auto-parallel context, in MB) and each bucket is replaced by one ``fused_all_reduce``.  Buckets only hold
    all-reduces with no other effect node between them, so the order of collectives across ranks is unchanged.
    Every node gets ``meta['fusion']`` = its bucket id (0: not fused)."""
    from .. import context
    if threshold_bytes is None:
        cfg = context.get_auto_parallel_context("comm_fusion") or {}
        ar = cfg.get("allreduce", {}) if isinstance(cfg, dict) else {}
        mode = ar.get("mode", "auto")
        if mode == "size":
            threshold_bytes = float(ar.get("config", 64)) * 1024 * 1024
        elif mode == "auto":
            threshold_bytes = 64 * 1024 * 1024
        else:
            return 0                      # index-based fusion is planned on parameters, not on the graph
    nodes = list(fg.graph.nodes)
    buckets, cur, cur_key, cur_bytes = [], [], None, 0

    def close():
        nonlocal cur, cur_key, cur_bytes
        if len(cur) > 1:
            buckets.append(cur)
        cur, cur_key, cur_bytes = [], None, 0

    for n in nodes:
        if n.op == "call_function" and _fname(n) == "all_reduce_node" and isinstance(n.args[0], fx.Node):
            key = (n.args[1], n.args[2], _dtype(n.args[0]))
            if cur and key != cur_key:
                close()
            cur.append(n)
            cur_key = key
            es = torch.empty((), dtype=_dtype(n.args[0]) or torch.float32).element_size()
            cur_bytes += _numel(n.args[0]) * es
            if cur_bytes >= threshold_bytes:
                close()
        elif cur and n.op == "call_function" and (is_collective(n) or is_impure(n)) and n not in cur:
            # another effect between two all-reduces: allowed only if it does not touch the bucket's tensors
            users = {a for m in cur for a in m.all_input_nodes}
            if is_collective(n) or any(a in users or a in cur for a in n.all_input_nodes):
                close()
    close()
    for bid, bucket in enumerate(buckets, start=1):
        last = bucket[-1]
        ins = [m.args[0] for m in bucket]
        # every bucket tensor must exist before the fused node: it goes where the last member was
        with fg.graph.inserting_after(last):
            fused = fg.graph.call_function(fused_all_reduce, (bucket[0].args[1], bucket[0].args[2],
                                                              tuple(_numel(x) for x in ins)) + tuple(ins))
        fused.meta["fusion"] = bid
        fused.meta["primitive"] = "AllReduce"
        prev = fused
        for i, m in enumerate(bucket):
            with fg.graph.inserting_after(prev):
                piece = fg.graph.call_function(operator.getitem, (fused, i))
            piece.meta.update({k: v for k, v in m.meta.items() if k in ("shape", "dtype")})
            piece.meta["fusion"] = bid
            prev = piece
            # users of an early member that sit before the fused node now need the reduced value later: only
            # legal when there are none (checked by construction: in-place reduces are consumed after backward)
            m.replace_all_uses_with(piece)
            fg.graph.erase_node(m)
    return len(buckets)


# ------------------------------------------------------------------------------------------------ effects / order
def effect_chains(fg):
    """Assigns ``meta['after']`` (name of the effect node this one must follow) and returns {node: predecessor}."""
    last_comm = None
    last_write = {}          # parameter / buffer node -> last effect node that touched it
    pred = {}
    for n in fg.graph.nodes:
        if n.op != "call_function":
            continue
        impure = is_impure(n) or is_collective(n)
        touched = [a for a in n.all_input_nodes if a.op == "get_attr" and "param" in a.meta]
        after = []
        if is_collective(n):
            if last_comm is not None:
                after.append(last_comm)
            last_comm = n
        for p in touched:
            if p in last_write and last_write[p] is not n:
                after.append(last_write[p])        # read-after-write / write-after-write on one parameter
            if impure:
                last_write[p] = n
        if after:
            pred[n] = after
            n.meta["after"] = [a.name for a in after]
    return pred


def comm_reorder(fg):
    """Moves every out-of-place collective (AllGather / ReduceScatter / AllToAll nodes and sharded primitives'
    communication is inside their node and stays) up to just behind the latest of: its inputs, its effect-chain
    predecessor.  Returns how many nodes moved."""
    pred = effect_chains(fg)
    order = {n: i for i, n in enumerate(fg.graph.nodes)}
    moved = 0
    for n in list(fg.graph.nodes):
        if not is_collective(n) or _fname(n) in ("all_reduce_node", "fused_all_reduce"):
            continue
        deps = list(n.all_input_nodes) + list(pred.get(n, []))
        if not deps:
            continue
        anchor = max(deps, key=lambda d: order[d])
        if anchor.op == "placeholder":
            # needs graph inputs only: it can start first, behind the last input node
            anchor = [m for m in fg.graph.nodes if m.op == "placeholder"][-1]
        if order[anchor] + 1 >= order[n]:
            continue
        # getitem nodes that unpack the anchor stay glued to it
        nxt = anchor.next
        while nxt is not n and nxt.op == "call_function" and nxt.target is operator.getitem and \
                nxt.args[0] is anchor:
            anchor = nxt
            nxt = anchor.next
        if anchor.next is n:
            continue
        anchor.append(n)
        n.meta["hoisted"] = True
        moved += 1
        order = {m: i for i, m in enumerate(fg.graph.nodes)}
    return moved


def mark_comm_stream(fg):
    """Out-of-place collectives whose result is first used at least two nodes later run on the executor's
    communication stream (``meta['comm_stream']``): the nodes in between overlap the transfer."""
    order = {n: i for i, n in enumerate(fg.graph.nodes)}
    marked = 0
    for n in fg.graph.nodes:
        if not is_collective(n) or _fname(n) in ("all_reduce_node", "fused_all_reduce") or not n.users:
            continue
        first_use = min(order[u] for u in n.users)
        if first_use - order[n] >= 2:
            n.meta["comm_stream"] = True
            marked += 1
    return marked
