"""Strategy search for ``parallel_mode="auto_parallel"``.

The graph is traced once on full (unsharded) shapes; every primitive that has an ``OperatorInfo`` becomes a node of
a cost graph with its candidate strategies (``OperatorInfo.generate_strategies``; a strategy given by the user with
``Primitive.shard`` is the only candidate of that node), an edge between a producer and a consumer costs the tensor
redistribution between the producer's output layout and the layout the consumer requires, and a candidate costs its
local memory traffic plus its forward communication.  The search itself is native (``csrc/host/planner.cpp``):

* ``sharding_propagation``   - breadth-first from the configured operators, each neighbour takes the candidate with
  the cheapest edge (auto_parallel/graph_costmodel.cc:94-116,196-319 in the reference);
* ``dynamic_programming`` / ``recursive_programming`` - exact dynamic programming when the operators form a chain,
  otherwise propagation followed by coordinate descent on the total cost (the reference eliminates the cost graph,
  dp_algo_costmodel.cc, or bipartitions recursively, rec_core/rec_partition.cc).

The chosen strategies are written onto the primitives (``in_strategy``), so the second trace - the one that is
compiled - runs them through the SPMD dispatcher exactly like hand-written ``shard`` calls."""
from __future__ import annotations

import operator

import torch

from . import operator_info as OI
from . import planner
from . import redistribution as RD

_COMM_WEIGHT = 4.0        # a byte over NVLink is charged like this many bytes of local memory traffic


def _numel(shape):
    n = 1
    for d in shape:
        n *= d
    return n


def _prim(node):
    t = node.target
    return t if node.op == "call_function" and hasattr(t, "name") and hasattr(t, "attrs") else None


def _source(node):
    """Producer node looking through tuple indexing."""
    while node.op == "call_function" and node.target is operator.getitem:
        node = node.args[0]
    return node


class _Op:
    def __init__(self, node, prim, in_nodes, in_shapes):
        self.node, self.prim, self.in_nodes, self.in_shapes = node, prim, in_nodes, in_shapes
        self.cands, self.infos, self.costs = [], [], []


def _candidates(op, device_num):
    prim = op.prim
    cls = OI.get_info_class(prim.name)
    fixed = prim.in_strategy is not None
    if fixed:
        cands = [tuple(tuple(s) for s in prim.in_strategy)]
    elif cls is not None:
        kw = {}
        if prim.name in ("MatMul", "BatchMatMul"):
            kw["transpose_b"] = bool(prim.attrs.get("transpose_b", False))
        try:
            cands = list(cls.generate_strategies(op.in_shapes, device_num, **kw))
        except TypeError:
            cands = list(cls.generate_strategies(op.in_shapes, device_num))
    else:
        cands = [tuple(tuple(1 for _ in s) for s in op.in_shapes)]
    extra = {}
    for cand in cands:
        try:
            info = OI.make_info(prim, op.in_shapes, cand, prim.out_strategy if fixed else None, device_num, **extra)
            ins, outs = info.input_layouts(), info.output_layouts()
        except Exception:  # noqa: BLE001  (candidate not applicable to these shapes)
            continue
        traffic = sum(_numel(l.slice_shape()) for l in ins) + sum(_numel(l.slice_shape()) for l in outs)
        comm = 0.0
        if info.forward_comm:
            comm = float(_numel(outs[0].slice_shape())) * (2.0 if info.forward_comm[0].startswith("AllReduce") else 1.0)
        op.cands.append(cand)
        op.infos.append((ins, outs))
        op.costs.append(traffic + _COMM_WEIGHT * comm)
    if not op.cands:
        raise OI.StrategyError("no applicable strategy for %s with input shapes %s" % (prim.name, op.in_shapes))
    return fixed


def _redistribution_cost(have, need):
    """0 when every rank already holds the slice it needs; the native cost of the operator list when both layouts
    share a device matrix; the price of a full gather otherwise (what ``redistribution.apply`` then does)."""
    from . import spmd
    if spmd.layouts_equivalent(have, need):
        return 0.0
    try:
        ops = RD.infer(have, need)
    except Exception:  # noqa: BLE001
        ops = None
    if ops is None:
        return _COMM_WEIGHT * float(_numel(need.shape))
    return _COMM_WEIGHT * float(RD.cost(ops, _numel(have.slice_shape())))


def _edge_matrix(src, dst, slot):
    rows = []
    for (_, outs) in src.infos:
        row = []
        for (ins, _) in dst.infos:
            need = ins[slot]
            have = outs[0]
            if have.shape != need.shape:
                row.append(float(_numel(need.shape)))        # reshaped in between: charge a full gather
                continue
            row.append(_redistribution_cost(have, need))
        rows.append(row)
    return rows


def _total(ops, edges, mats, choice):
    c = sum(op.costs[choice[i]] for i, op in enumerate(ops))
    for (a, b), m in zip(edges, mats):
        c += m[choice[a]][choice[b]]
    return c


def search(fg, device_num, search_mode="sharding_propagation"):
    """Chooses a strategy for every distributable primitive of ``fg`` and writes it to the primitive.
    Returns {node name: strategy}."""
    ops, index = [], {}
    for node in fg.graph.nodes:
        prim = _prim(node)
        if prim is None or type(prim).__module__.endswith("comm_ops"):
            continue
        in_nodes = [a for a in node.args if hasattr(a, "meta") and a.meta.get("shape") is not None]
        if not in_nodes or (OI.get_info_class(prim.name) is None and prim.in_strategy is None):
            continue
        op = _Op(node, prim, in_nodes, [tuple(a.meta["shape"]) for a in in_nodes])
        try:
            fixed = _candidates(op, device_num)
        except OI.StrategyError:
            continue
        index[node] = len(ops)
        ops.append((op, fixed))
    if not ops:
        return {}
    fixed_idx = [0 if f else -1 for _, f in ops]
    ops = [o for o, _ in ops]
    edges, mats = [], []
    for j, op in enumerate(ops):
        for slot, a in enumerate(op.in_nodes):
            src = _source(a)
            if src in index and index[src] != j:
                edges.append((index[src], j))
                mats.append(_edge_matrix(ops[index[src]], op, slot))
    n_cand = [len(o.cands) for o in ops]
    is_chain = all(b == a + 1 for a, b in edges) and len(edges) == len(ops) - 1 and all(f < 0 for f in fixed_idx)
    if search_mode in ("dynamic_programming", "recursive_programming") and is_chain:
        choice, _ = planner.chain_dp_search([o.costs for o in ops], mats)
    else:
        if all(f < 0 for f in fixed_idx):
            # nothing configured: seed the propagation at the most expensive operator with its cheapest candidate
            heavy = max(range(len(ops)), key=lambda i: min(ops[i].costs))
            seed = list(fixed_idx)
            seed[heavy] = min(range(n_cand[heavy]), key=lambda c: ops[heavy].costs[c])
        else:
            seed = fixed_idx
        choice = planner.propagate_strategies(n_cand, seed, edges, mats) if edges else \
            [s if s >= 0 else min(range(n), key=lambda c, i=i: ops[i].costs[c])
             for i, (s, n) in enumerate(zip(seed, n_cand))]
        if search_mode != "sharding_propagation":
            improved = True
            while improved:
                improved = False
                for i in range(len(ops)):
                    if fixed_idx[i] >= 0:
                        continue
                    best, best_c = choice[i], _total(ops, edges, mats, choice)
                    for c in range(n_cand[i]):
                        trial = list(choice)
                        trial[i] = c
                        t = _total(ops, edges, mats, trial)
                        if t < best_c - 1e-9:
                            best, best_c = c, t
                    if best != choice[i]:
                        choice[i] = best
                        improved = True
    out = {}
    for op, c in zip(ops, choice):
        strat = tuple(tuple(int(v) for v in s) for s in op.cands[c])
        if op.prim.in_strategy is None:
            op.prim.in_strategy = strat
            op.prim.add_prim_attr("in_strategy", strat)
        out[op.node.name] = strat
    return out
