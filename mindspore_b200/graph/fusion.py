"""Pattern fusion on the traced graph: chains of small operators that this framework has ONE kernel for are rewritten
to that kernel before reverse mode is built, so that forward and backward both run fused.

  Add(x, r) -> RmsNorm(., gamma)                      =>  AddRmsNorm(x, r, gamma)        (sum and norm in one pass)
  Split(axis=-1, 2)(gu) -> Mul(SiLU(a), b)            =>  SwiGLU(gu)
  BiasAdd(x, b) -> GeLU                               =>  bias + tanh-GELU in one kernel
  MatMul(x, w; transpose_b) -> BiasAdd(., b)          =>  GEMM with the bias in its epilogue

This is the role of the reference's graph-kernel / backend fusion passes (backend/common/graph_kernel/*,
plugin/device/gpu/optimizer/{matmul_biasadd_fusion,add_relu_v2_fusion,...}.cc), restricted to the patterns that have
a hand-written sm_100a kernel here.  Patterns whose primitives carry shard strategies keep them: the fused
primitive gets the strategy of the pattern's inputs."""
from __future__ import annotations

import operator

import torch.fx as fx

from .opt_passes import _differentiated, _prim_name


def _only_user(n, allow_getitem=False):
    users = list(n.users)
    return users[0] if len(users) == 1 else None


def _getitem_users(n):
    """{index: node} for a multi-output node whose users are all getitem nodes, else None."""
    out = {}
    for u in n.users:
        if u.op == "call_function" and u.target is operator.getitem and u.args[0] is n:
            out.setdefault(u.args[1], []).append(u)
        else:
            return None
    return out


def _attr(prim, name, default=None):
    return prim.attrs.get(name, getattr(prim, name, default))


def _copy_meta(dst, src, keys=("shape", "dtype")):
    for k in keys:
        if k in src.meta:
            dst.meta[k] = src.meta[k]


def fuse_patterns(fg):
    """Returns {replaced node: replacement}."""
    from .. import ops
    g = fg.graph
    replaced = {}

    def busy(*nodes):
        return any(_differentiated(fg, n) for n in nodes)

    for n in list(g.nodes):
        if n.op != "call_function" or n not in set(g.nodes):
            continue
        name = _prim_name(n)
        # ---- Add -> RmsNorm
        if name == "RmsNorm" and len(n.args) == 2 and isinstance(n.args[0], fx.Node) and _prim_name(n.args[0]) == "Add":
            add = n.args[0]
            outs = _getitem_users(n)
            if outs is None or any(u.users for u in outs.get(1, [])) or busy(n, add) or len(add.args) != 2 or \
                    not all(isinstance(a, fx.Node) for a in add.args):
                continue
            a, b = add.args
            if a.meta.get("shape") != b.meta.get("shape") or a.meta.get("shape") is None:
                continue                                       # a broadcasting add is not the residual pattern
            order = {m: i for i, m in enumerate(g.nodes)}
            if any(order[u] < order[n] for u in add.users):
                continue                                       # the sum is read before the norm: it stays where it is
            prim = ops.AddRmsNorm(float(_attr(n.target, "epsilon", 1e-6)))
            if n.target.in_strategy is not None and len(n.target.in_strategy) == 2:
                xs, gs = n.target.in_strategy
                prim.shard((tuple(xs), tuple(xs), tuple(gs)))
            with g.inserting_before(n):
                fused = g.call_function(prim, (a, b, n.args[1]))
                y = g.call_function(operator.getitem, (fused, 0))
                s = g.call_function(operator.getitem, (fused, 1))
            fused.meta["primitive"] = "AddRmsNorm"
            _copy_meta(s, add)
            for u in outs.get(0, []):
                _copy_meta(y, u)
                u.replace_all_uses_with(y)
                replaced[u] = y
                g.erase_node(u)
            for u in outs.get(1, []):                          # the rstd output: recorded but unread
                g.erase_node(u)
            g.erase_node(n)
            add.replace_all_uses_with(s)
            replaced[add] = s
            g.erase_node(add)
            continue
        # ---- Split -> SiLU * .
        if name == "Mul" and len(n.args) == 2 and all(isinstance(a, fx.Node) for a in n.args):
            for silu, other in ((n.args[0], n.args[1]), (n.args[1], n.args[0])):
                if _prim_name(silu) != "SiLU" or not isinstance(silu.args[0], fx.Node):
                    continue
                ga, gb = silu.args[0], other
                if not (ga.op == gb.op == "call_function" and ga.target is operator.getitem and gb.target is operator.getitem):
                    continue
                sp = ga.args[0]
                if sp is not gb.args[0] or _prim_name(sp) != "Split" or (ga.args[1], gb.args[1]) != (0, 1):
                    continue
                rank = len(sp.meta.get("shape", ())) or len(n.meta.get("shape", ()))
                ax = int(_attr(sp.target, "axis", 0))
                if int(_attr(sp.target, "output_num", 1)) != 2 or (ax != -1 and ax != rank - 1):
                    continue
                if len(sp.users) != 2 or len(ga.users) != 1 or len(gb.users) != 1 or len(silu.users) != 1 or \
                        busy(n, silu, sp):
                    continue
                prim = ops.SwiGLU()
                with g.inserting_before(n):
                    fused = g.call_function(prim, (sp.args[0],))
                fused.meta["primitive"] = "SwiGLU"
                _copy_meta(fused, n)
                n.replace_all_uses_with(fused)
                replaced[n] = fused
                for dead in (n, silu, ga, gb, sp):
                    g.erase_node(dead)
                break
            continue
        # ---- BiasAdd -> GeLU
        if name == "GeLU" and len(n.args) == 1 and isinstance(n.args[0], fx.Node) and _prim_name(n.args[0]) == "BiasAdd":
            ba = n.args[0]
            shp = ba.meta.get("shape")
            if len(ba.users) != 1 or busy(n, ba) or shp is None or len(shp) != 2 or \
                    n.target.in_strategy is not None or ba.target.in_strategy is not None:
                continue
            from ..ops import fused as F
            with g.inserting_before(n):
                fz = g.call_function(F.gelu_tanh, (ba.args[0], ba.args[1]))
            fz.meta["primitive"] = "BiasGeLU"
            _copy_meta(fz, n)
            n.replace_all_uses_with(fz)
            replaced[n] = fz
            g.erase_node(n)
            g.erase_node(ba)
            continue
        # ---- MatMul -> BiasAdd
        if name == "BiasAdd" and len(n.args) == 2 and isinstance(n.args[0], fx.Node) and _prim_name(n.args[0]) == "MatMul":
            mm = n.args[0]
            if len(n.users) == 1 and _prim_name(next(iter(n.users))) == "GeLU" and len(mm.meta.get("shape", ())) == 2:
                continue                                       # bias + GELU fuse instead (the pattern above)
            if len(mm.users) != 1 or busy(n, mm) or not _attr(mm.target, "transpose_b", False) or \
                    _attr(mm.target, "transpose_a", False) or mm.target.in_strategy is not None or \
                    n.target.in_strategy is not None or len(mm.meta.get("shape", ())) != 2:
                continue
            from ..ops import fused as F
            with g.inserting_before(n):
                fz = g.call_function(F.linear, (mm.args[0], mm.args[1], n.args[1]))
            fz.meta["primitive"] = "Dense"
            _copy_meta(fz, n)
            n.replace_all_uses_with(fz)
            replaced[n] = fz
            g.erase_node(n)
            g.erase_node(mm)
    return replaced
