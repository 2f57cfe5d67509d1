"""Strategy search for ``parallel_mode="auto_parallel"``.

The graph is traced once on full (unsharded) shapes; every primitive that has an ``OperatorInfo`` becomes a node of
a cost graph with its candidate strategies (``OperatorInfo.generate_strategies``; a strategy given by the user with
``Primitive.shard`` is the only candidate of that node), an edge between a producer and a consumer costs the tensor
redistribution between the producer's output layout and the layout the consumer requires, and a candidate costs its
local memory traffic plus its forward communication.  The search itself is native (``csrc/host/planner.cpp``):

* ``sharding_propagation``   - breadth-first from the configured operators, each neighbour takes the candidate with
  the cheapest edge (auto_parallel/graph_costmodel.cc:94-116,196-319 in the reference);
* ``dynamic_programming``     - the exact minimum over the whole cost graph by node elimination (operator / edge /
  merge / contract / triangle / star eliminations of auto_parallel/graph_costmodel.cc:866-1776 are its degree-1 to
  degree-3 cases); graphs whose eliminated neighbourhoods grow too large fall back to propagation + coordinate descent;
* ``recursive_programming``   - the device count is halved level by level (rec_core/rec_partition.cc,
  rec_generate_strategy.cc): at each level every operator, heaviest first, picks which of its dims to cut in two -
  the cut whose own cost plus redistribution towards already decided neighbours is least - and the product of
  the cuts is the strategy.  Linear in the graph size and independent of the number of full-size candidates.

Costs come from ``parallel/cost_model.py`` (alpha * computation + beta * communication, memory per candidate); a
result that does not fit ``device_memory_capacity`` is searched again with a growing price on memory.

The chosen strategies are written onto the primitives (``in_strategy``), so the second trace - the one that is
compiled - runs them through the SPMD dispatcher exactly like hand-written ``shard`` calls."""
from __future__ import annotations

import operator

import torch

from . import cost_model as CM
from . import operator_info as OI
from . import planner
from . import redistribution as RD


def _comm_weight():
    return CM.get_cost_model_context("costmodel_beta")


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
        self.cands, self.infos, self.costs, self.mems = [], [], [], []
        self.param_inputs = [i for i, a in enumerate(in_nodes) if a.op == "get_attr" and "param" in a.meta]


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
        if not fixed and _fully_use() and info.repeat > 1 and len(cands) > 1 and \
                any(_uses_all(c, device_num) for c in cands):
            continue                         # fully_use_devices: drop candidates that leave devices idle
        cost, mem = CM.candidate_cost(prim, info, op.param_inputs)
        op.cands.append(cand)
        op.infos.append((ins, outs))
        op.costs.append(cost)
        op.mems.append(mem)
    if not op.cands:
        raise OI.StrategyError("no applicable strategy for %s with input shapes %s" % (prim.name, op.in_shapes))
    return fixed


def _fully_use():
    from ..common.api import get_algo_parameters
    return bool(get_algo_parameters("fully_use_devices"))


def _uses_all(cand, device_num):
    """Cheap pre-filter on the raw tuple: some input is split as many ways as there are devices (the OperatorInfo
    knows exactly: repeat == 1)."""
    best = 1
    for st in cand:
        p = 1
        for s in st:
            p *= s
        best = max(best, p)
    return best >= device_num


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
        have2 = spmd.rebase(have, need.device_matrix)
        if have2 is not None:
            try:
                ops = RD.infer(have2, need)
            except Exception:  # noqa: BLE001
                ops = None
    if ops is None:
        return _comm_weight() * CM.comm_bytes_cost(2.0 * _numel(need.shape))
    return _comm_weight() * CM.comm_bytes_cost(2.0 * float(RD.cost(ops, _numel(have.slice_shape()))))


def _edge_matrix(src, dst, slot):
    rows = []
    for (_, outs) in src.infos:
        row = []
        for (ins, _) in dst.infos:
            need = ins[slot]
            have = outs[0]
            if have.shape != need.shape:
                row.append(_comm_weight() * 2.0 * float(_numel(need.shape)))   # reshaped in between: a full gather
                continue
            row.append(_redistribution_cost(have, need))
        rows.append(row)
    return rows


def _solve(ops, edges, mats, fixed_idx, search_mode, costs):
    """One search over the cost graph with the given per-candidate costs."""
    n_cand = [len(o.cands) for o in ops]
    if search_mode == "dynamic_programming":
        choice, _ = planner.elimination_search(n_cand, costs, edges, mats, fixed_idx)
        if choice is not None:
            return choice
    if all(f < 0 for f in fixed_idx):
        # nothing configured: seed the propagation at the most expensive operator with its cheapest candidate
        heavy = max(range(len(ops)), key=lambda i: min(costs[i]))
        seed = list(fixed_idx)
        seed[heavy] = min(range(n_cand[heavy]), key=lambda c: costs[heavy][c])
    else:
        seed = fixed_idx
    choice = planner.propagate_strategies(n_cand, seed, edges, mats) if edges else \
        [s if s >= 0 else min(range(n), key=lambda c, i=i: costs[i][c]) for i, (s, n) in enumerate(zip(seed, n_cand))]
    if search_mode == "sharding_propagation":
        return choice

    def total(ch):
        return sum(costs[i][ch[i]] for i in range(len(ops))) + sum(m[ch[a]][ch[b]] for (a, b), m in zip(edges, mats))
    improved = True
    while improved:
        improved = False
        for i in range(len(ops)):
            if fixed_idx[i] >= 0:
                continue
            best, best_c = choice[i], total(choice)
            for c in range(n_cand[i]):
                trial = list(choice)
                trial[i] = c
                t = total(trial)
                if t < best_c - 1e-9:
                    best, best_c = c, t
            if best != choice[i]:
                choice[i] = best
                improved = True
    return choice


def _halvings(cand_small, cand_big):
    """True when ``cand_big`` is ``cand_small`` with the splits of ONE device-matrix dim doubled (the same factor 2
    may show up in several inputs, e.g. the K dim of both MatMul operands)."""
    ratio = []
    for a, b in zip(cand_small, cand_big):
        if len(a) != len(b):
            return False
        for x, y in zip(a, b):
            if y % x:
                return False
            ratio.append(y // x)
    return all(r in (1, 2) for r in ratio) and any(r == 2 for r in ratio)


def _recursive(ops, edges, fixed_idx, device_num):
    """Recursive bipartition: log2(device_num) levels; at each level the operators are visited in decreasing weight
    and each takes the refinement (one dim cut in two, or none = repeated computation) of its previous-level
    strategy that minimises its own cost plus the redistribution towards neighbours already decided at this level."""
    levels = []
    d = 2
    while d <= device_num:
        levels.append(d)
        d *= 2
    if not levels or levels[-1] != device_num:
        return None                                   # device count is not a power of two
    nbrs = {i: [] for i in range(len(ops))}
    for (a, b) in edges:
        slot = None
        for sl, node in enumerate(ops[b].in_nodes):
            if _source(node) is ops[a].node:
                slot = sl
        nbrs[a].append((b, slot, True))
        nbrs[b].append((a, slot, False))
    weight = [max((_numel(s) for s in op.in_shapes), default=0) for op in ops]
    # visiting order: breadth-first from the configured operators (else from the heaviest one), heavier neighbours
    # first - every operator but the seeds then sees at least one decided neighbour when it chooses its cut
    seeds = [i for i, f in enumerate(fixed_idx) if f >= 0] or [max(range(len(ops)), key=lambda i: weight[i])]
    order, seen, queue = [], set(seeds), list(seeds)
    while queue:
        i = queue.pop(0)
        order.append(i)
        for j in sorted({j for j, _, _ in nbrs[i]}, key=lambda j: -weight[j]):
            if j not in seen:
                seen.add(j)
                queue.append(j)
    order += sorted((i for i in range(len(ops)) if i not in seen), key=lambda i: -weight[i])
    prev = [tuple(tuple(1 for _ in s) for s in op.in_shapes) for op in ops]
    prev_lay = [None] * len(ops)
    for dev in levels:
        cur, cur_lay = [None] * len(ops), [None] * len(ops)
        for i in order:
            op = ops[i]
            level_op = _Op(op.node, op.prim, op.in_nodes, op.in_shapes)
            saved = op.prim.in_strategy
            try:
                if fixed_idx[i] >= 0:
                    # a configured operator follows its final strategy as far as this level's device count allows
                    final = tuple(tuple(s) for s in saved)
                    cands = [final] if _prod_devices(final) <= dev else [prev[i]]
                    op.prim.in_strategy = None
                    level_op.cands, level_op.infos, level_op.costs = [], [], []
                    for c in cands:
                        try:
                            info = OI.make_info(op.prim, op.in_shapes, c, None, dev)
                            level_op.cands.append(c)
                            level_op.infos.append((info.input_layouts(), info.output_layouts()))
                            level_op.costs.append(CM.candidate_cost(op.prim, info, op.param_inputs)[0])
                        except Exception:  # noqa: BLE001
                            pass
                else:
                    _candidates(level_op, dev)
            except OI.StrategyError:
                level_op.cands = []
            finally:
                op.prim.in_strategy = saved
            options = [k for k, c in enumerate(level_op.cands) if c == prev[i] or _halvings(prev[i], c)] or \
                list(range(len(level_op.cands)))
            if not options:
                return None
            best, best_cost = None, None
            for k in options:
                cost = level_op.costs[k]
                ins_k, outs_k = level_op.infos[k]
                for (j, slot, i_is_src) in nbrs[i]:
                    if cur_lay[j] is None or slot is None:
                        continue
                    ins_j, outs_j = cur_lay[j]
                    have, need = (outs_k[0], ins_j[slot]) if i_is_src else (outs_j[0], ins_k[slot])
                    if have.shape == need.shape:
                        cost += _redistribution_cost(have, need)
                if best_cost is None or cost < best_cost - 1e-9:
                    best, best_cost = k, cost
            cur[i] = level_op.cands[best]
            cur_lay[i] = level_op.infos[best]
        prev, prev_lay = cur, cur_lay
    choice = []
    for i, op in enumerate(ops):
        if prev[i] in op.cands:
            choice.append(op.cands.index(prev[i]))
        else:
            op.cands.append(prev[i])
            op.infos.append(prev_lay[i])
            op.costs.append(0.0)
            op.mems.append(0.0)
            choice.append(len(op.cands) - 1)
    return choice


def _prod_devices(cand):
    best = 1
    for st in cand:
        p = 1
        for s in st:
            p *= s
        best = max(best, p)
    return best


def fit_memory(ops, edges, mats, fixed_idx, search_mode, device_num):
    """Search; while the chosen strategies need more than ``device_memory_capacity`` per rank, search again with
    memory priced into every candidate (price doubling each round)."""
    cap = CM.get_cost_model_context("device_memory_capacity")
    choice = None
    if search_mode == "recursive_programming":
        choice = _recursive(ops, edges, fixed_idx, device_num)
    if choice is None:
        mode = "dynamic_programming" if search_mode == "recursive_programming" else search_mode
        choice = _solve(ops, edges, mats, fixed_idx, mode, [o.costs for o in ops])
    price = 0.0
    for _ in range(12):
        used = sum(o.mems[c] for o, c in zip(ops, choice) if c < len(o.mems))
        if used <= cap:
            break
        price = 1.0 if price == 0.0 else price * 4.0
        costs = [[c + price * m for c, m in zip(o.costs, o.mems)] for o in ops]
        mode = "dynamic_programming" if search_mode != "sharding_propagation" else search_mode
        choice = _solve(ops, edges, mats, fixed_idx, mode, costs)
    return choice


def total_cost(ops, edges, mats, choice):
    return sum(op.costs[choice[i]] for i, op in enumerate(ops)) + \
        sum(m[choice[a]][choice[b]] for (a, b), m in zip(edges, mats))


last_search = {}          # what the most recent ``search`` built: ops, edges, matrices, choice (for inspection / tests)


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
    choice = fit_memory(ops, edges, mats, fixed_idx, search_mode, device_num)
    last_search.clear()
    last_search.update(ops=ops, edges=edges, mats=mats, choice=list(choice), mode=search_mode,
                       memory=sum(o.mems[c] for o, c in zip(ops, choice) if c < len(o.mems)))
    out = {}
    for op, c in zip(ops, choice):
        strat = tuple(tuple(int(v) for v in s) for s in op.cands[c])
        if op.prim.in_strategy is None:
            op.prim.in_strategy = strat
            op.prim.add_prim_attr("in_strategy", strat)
        out[op.node.name] = strat
    return out
