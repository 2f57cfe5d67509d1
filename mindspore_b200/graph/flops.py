"""FLOPs of a traced graph: what ``flops_collection`` reports and what ``FlopsUtilizationCollector`` divides by.

Contractions are counted from the shapes the trace recorded on every node (2 x multiply-adds): MatMul / BatchMatMul /
Dense / linear, Conv2D, FlashAttentionScore (causal halves the score and value products).  Everything else counts
one operation per output element.  A node that the autodiff pass differentiates adds its backward: two more
contractions of the same size (input and weight gradients; five half-products for attention), one more pass for
element-wise nodes.  "Hardware" FLOPs add the forward of nodes inside recomputed cells once more; "shard" figures
divide each node by the product of its sharding strategy.

Parity (role): ccsrc/pipeline/jit/ps/pipeline.cc GraphExecutorPy::FlopsCollection, used by
python/mindspore/train/callback/_flops_collector.py."""
from __future__ import annotations

import math

import torch.fx as fx

_last = {}          # phase -> (FuncGraph, has_backward)

_MATMUL = ("MatMul", "BatchMatMul", "MatMulExt", "BatchMatMulExt", "Dense", "linear", "matmul", "bmm", "mm", "addmm")
_CONV = ("Conv2D", "conv2d", "Convolution")
_ATTN = ("FlashAttentionScore", "flash_attention", "qkv_rope_attention", "scaled_dot_product_attention")


def _name(n):
    t = n.target
    if hasattr(t, "name") and hasattr(t, "attrs"):
        return t.name
    return getattr(t, "__name__", str(t))


def _shape(a):
    if isinstance(a, fx.Node):
        s = a.meta.get("shape")
        if s is None and "example" in a.meta:
            s = a.meta["example"][0]
        if s is None and a.meta.get("param") is not None:
            s = tuple(a.meta["param"].shape)
        return tuple(s) if s is not None else None
    return None


def _numel(s):
    return int(math.prod(s)) if s is not None else 0


def node_flops(n):
    """(forward flops, backward flops if differentiated) of one call_function node."""
    name = _name(n)
    out = _shape(n)
    ins = [_shape(a) for a in n.args]
    attrs = getattr(n.target, "attrs", {}) if hasattr(n.target, "attrs") else {}
    if name in _MATMUL and out is not None and ins and ins[0] is not None:
        a = ins[0]
        ta = bool(attrs.get("transpose_a", n.kwargs.get("transpose_a", False)))
        k = a[-2] if ta and len(a) >= 2 else a[-1]
        if name == "addmm" and len(ins) > 1 and ins[1] is not None:
            k = ins[1][-1]
        f = 2 * _numel(out) * int(k)
        return f, 2 * f
    if name in _CONV and out is not None and len(ins) > 1 and ins[1] is not None:
        w = ins[1]                                               # [Cout, Cin / groups, kh, kw]
        f = 2 * _numel(out) * int(math.prod(w[1:]))
        return f, 2 * f
    if name in _ATTN and ins and ins[0] is not None:
        q = ins[0]
        if name == "qkv_rope_attention":
            return 0, 0                                           # packed form: shapes are in the arguments, not here
        if len(q) == 4:                                           # [B, S, H, D] (or [B, H, S, D]: same product)
            b, s1, s2, d = q
            kv = ins[1] if len(ins) > 1 and ins[1] is not None else q
            skv = kv[1] if name != "scaled_dot_product_attention" else kv[2]
            sq = s1 if name != "scaled_dot_product_attention" else s2
            heads = s2 if name != "scaled_dot_product_attention" else s1
            f = 4 * b * heads * sq * skv * d
            causal = attrs.get("sparse_mode", 0) in (2, 3) or bool(n.kwargs.get("causal", n.kwargs.get("is_causal", False)))
            if causal:
                f //= 2
            return f, 5 * f // 2
    e = _numel(out)
    return e, e


def graph_flops(fg, backward=None):
    """{"model", "hardware", "shard_model", "shard_hardware", "by_op"} for a FuncGraph.  ``backward``: count the
    backward of differentiated nodes (default: when the graph holds any)."""
    nodes = [n for n in fg.graph.nodes if n.op == "call_function"]
    if backward is None:
        backward = any(n.meta.get("requires_vjp") for n in nodes)
    total = {"model": 0, "hardware": 0, "shard_model": 0, "shard_hardware": 0, "by_op": {}}
    for n in nodes:
        if n.meta.get("vjp_of") is not None or _name(n) in ("getitem", "vjp", "accumulate"):
            continue
        fwd, bwd = node_flops(n)
        f = fwd + (bwd if backward and n.meta.get("requires_vjp") else 0)
        hw = f + (fwd if n.meta.get("recompute") and backward else 0)
        strat = n.meta.get("strategy")
        div = 1
        if strat:
            first = strat[0] if isinstance(strat[0], (tuple, list)) else strat
            div = max(1, int(math.prod(first)))
            if len(strat) > 1 and isinstance(strat[1], (tuple, list)) and _name(n) in _MATMUL:
                div = max(div, int(math.prod(first)) * int(strat[1][-1] if not getattr(n.target, "attrs", {}).get(
                    "transpose_b") else strat[1][0]))
        total["model"] += f
        total["hardware"] += hw
        total["shard_model"] += f // div
        total["shard_hardware"] += hw // div
        total["by_op"][_name(n)] = total["by_op"].get(_name(n), 0) + f
    return total


def note_compiled(phase, fg):
    _last[phase] = fg


def flops_collection(phase="train"):
    """(full model FLOPs, full hardware FLOPs, shard model FLOPs, shard hardware FLOPs, is_dynamic_shape) of the
    graph most recently compiled for ``phase`` ('train' / 'eval' / 'predict'); raises if none was compiled."""
    fg = _last.get(phase)
    if fg is None and phase in ("eval", "predict"):
        fg = _last.get("predict") or _last.get("eval")
    if fg is None:
        raise RuntimeError("flops_collection: no graph has been compiled for phase %r (run a step in GRAPH_MODE "
                           "first)" % (phase,))
    t = graph_flops(fg)
    return t["model"], t["hardware"], t["shard_model"], t["shard_hardware"], False
