"""Post-trace parallel passes over a graph compiled in semi_auto_parallel / auto_parallel mode.

Sharded primitives go through the SPMD dispatcher while the graph is being traced (``parallel.spmd.dispatch``):
each becomes one graph node whose metadata lists the redistribution operators, the forward collective and the
mirror operators its execution performs (and performs again on every replay).  What is left for a pass over that
graph is what the reference does at the end of ``StepParallel`` and in the communication-fusion passes:

* annotate every node with the strategy / stage it ran under and collect ``parameter_layout_dict`` on the owner
  cell (pipeline/jit/ps/pipeline.cc GetParameterLayout; step_parallel.cc:2832-2893 CheckpointStrategy);
* assign ``fusion`` ids to gradient all-reduces (mirror operators) by cumulative size, so the executor can issue
  one collective per bucket (frontend/parallel/allreduce_fusion/step_allreduce_fusion.cc:31-104,
  allreduce_fusion.cc:82-176);
* write the strategy checkpoint when ``strategy_ckpt_save_file`` is set;
* report the communication volume of the step (graph_util/flops_collection-style accounting), used by tests and by
  the cost model."""
from __future__ import annotations

import torch

from .. import context
from . import spmd
from .strategy_ckpt import save_strategy_file

_COMM_NAMES = ("AllReduce", "AllGather", "ReduceScatter", "AlltoAll", "AlltoAllV", "Broadcast", "_MirrorOperator",
               "_MirrorMicroStepOperator", "_MirrorMiniStepOperator", "_MiniStepAllGather", "_MicroStepAllGather",
               "_VirtualDiv", "Send", "Receive", "NeighborExchange", "NeighborExchangeV2")


def _prim(node):
    t = node.target
    return t if node.op == "call_function" and hasattr(t, "name") and hasattr(t, "attrs") else None


def _example_bytes(node):
    shape, dtype = node.meta.get("shape"), node.meta.get("dtype")
    if shape is None or dtype is None:
        return 0
    n = 1
    for d in shape:
        n *= d
    return n * torch.empty(0, dtype=dtype).element_size()


def comm_nodes(fg):
    return [n for n in fg.graph.nodes if _prim(n) is not None and _prim(n).name in _COMM_NAMES]


def assign_fusion_ids(fg, threshold_mb=None):
    """Groups gradient all-reduces (mirror operators) into buckets of about ``threshold_mb`` and stores the bucket
    id in ``node.meta['fusion']`` (and the primitive attribute ``fusion``).  Returns [(fusion id, [nodes])]."""
    cfg = context.get_auto_parallel_context("comm_fusion") or {}
    if threshold_mb is None:
        ar = cfg.get("allreduce", {}) if isinstance(cfg, dict) else {}
        threshold_mb = ar.get("config", 64) if ar.get("mode", "auto") in ("auto", "size") else 64
        if isinstance(threshold_mb, (list, tuple)):
            threshold_mb = 64
    limit = float(threshold_mb) * 2 ** 20
    buckets, cur, size, fid = [], [], 0.0, 1
    for n in fg.graph.nodes:
        p = _prim(n)
        if p is None or not p.name.startswith("_Mirror"):
            continue
        cur.append(n)
        size += _example_bytes(n)
        n.meta["fusion"] = fid
        p.add_prim_attr("fusion", fid)
        if size >= limit:
            buckets.append((fid, cur))
            cur, size, fid = [], 0.0, fid + 1
    if cur:
        buckets.append((fid, cur))
    return buckets


def communication_volume(fg):
    """{collective name: (count, bytes of the operands)}: explicit communication primitives of the graph plus the
    collectives that sharded primitives perform around their local kernel (``node.meta['forward_comm']``,
    ``['redistribution']``, ``['mirror']``)."""
    out = {}

    def add(name, nbytes):
        c, b = out.get(name, (0, 0))
        out[name] = (c + 1, b + nbytes)

    for n in fg.graph.nodes:
        p = _prim(n)
        if p is None:
            continue
        if p.name in _COMM_NAMES:
            add(p.name, _example_bytes(n))
        fc = n.meta.get("forward_comm")
        if fc:
            add("AllReduce" if fc[0].startswith("AllReduce") else fc[0], _example_bytes(n))
        for name in n.meta.get("redistribution", ()):
            add(name, 0)
        for _ in range(n.meta.get("mirror", 0)):
            add("_MirrorOperator", 0)
    return out


def annotate_graph(fg, owner):
    """Runs the passes above on a freshly traced graph and publishes the parallel facts on ``owner``."""
    stage = 0
    for n in fg.graph.nodes:
        p = _prim(n)
        if p is None:
            continue
        if p.in_strategy is not None:
            n.meta["strategy"] = p.in_strategy
        if p.stage is not None:
            stage = p.stage
            n.meta["stage"] = stage
    buckets = assign_fusion_ids(fg)
    layouts = dict(spmd.parameter_layouts)
    names = {p.name for p in owner.get_parameters()} if hasattr(owner, "get_parameters") else set(layouts)
    owner_layouts = {k: v for k, v in layouts.items() if k in names}
    object.__setattr__(owner, "parameter_layout_dict", {k: v.to_dict() for k, v in owner_layouts.items()})
    object.__setattr__(owner, "parallel_parameter_name_list", sorted(owner_layouts))
    object.__setattr__(owner, "_comm_volume", communication_volume(fg))
    object.__setattr__(owner, "_fusion_buckets", [(fid, len(ns)) for fid, ns in buckets])
    path = context.get_auto_parallel_context("strategy_ckpt_save_file")
    if path:
        strategies = {}
        for i, n in enumerate(fg.graph.nodes):
            p = _prim(n)
            if p is not None and p.in_strategy is not None:
                strategies["%s-op%d" % (p.name, i)] = p.in_strategy
        rank = context.get_auto_parallel_context("global_rank")
        per = max(1, context.get_auto_parallel_context("device_num") //
                  context.get_auto_parallel_context("pipeline_stages"))
        save_strategy_file(path, owner_layouts, strategies, stage=rank // per)
    return fg
