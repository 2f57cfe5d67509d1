"""Execution of shard strategies: the step-parallel transformation, applied where the primitive is called.

In ``semi_auto_parallel`` / ``auto_parallel`` mode a primitive that carries a strategy (``Primitive.shard``), or
whose inputs carry layouts, goes through ``dispatch``:

1. the OperatorInfo of the primitive turns the strategy into required input layouts, output layouts and the
   forward communication;
2. every tensor input is redistributed from its current layout to the required one (``redistribution.apply``:
   StridedSlice / AllGather / AlltoAll); Parameters are sliced once according to the layout and remember it
   (``parameter_layout_dict``), and a replicated Parameter gets a ``_MirrorOperator`` so that its gradient is
   all-reduced over the replica group;
3. the primitive runs on the local slices (with shape-like arguments localised);
4. the forward communication (AllReduce or ReduceScatter over the contraction device dims) is applied;
5. outputs are tagged with their layouts.

Because the collectives are differentiable primitives, backward communication needs no separate pass, and when
this happens under graph tracing the comm primitives are recorded as graph nodes - the traced graph *is* the
step-parallel graph.  This replaces the compile-time rewrite of ccsrc/frontend/parallel/step_parallel.cc
:2738-2793 (ParallelCommunication: InsertForwardOps, StepRedistribution, InsertMirrorOps, InsertVirtualDivOp).
"""
from __future__ import annotations

import numpy as np
import torch

from .. import context
from ..common.parameter import Parameter
from ..communication import management as M
from . import operator_info as OI
from . import redistribution as RD
from .layout import TensorLayout, slice_for_rank

_ATTR = "_ms_layout"

parameter_layouts = {}      # name -> TensorLayout, filled as parameters get sliced
_mirror_cache = {}


def active():
    mode = context.get_auto_parallel_context("parallel_mode")
    return mode in (context.ParallelMode.SEMI_AUTO_PARALLEL, context.ParallelMode.AUTO_PARALLEL)


def get_layout(t):
    return getattr(t, _ATTR, None) if isinstance(t, torch.Tensor) else None


def set_layout(t, layout):
    if isinstance(t, torch.Tensor):
        setattr(t, _ATTR, layout)
    return t


def stage_devices():
    n = context.get_auto_parallel_context("device_num")
    return n // context.get_auto_parallel_context("pipeline_stages")


def _rank():
    return context.get_auto_parallel_context("global_rank")


def _stage_base():
    per = stage_devices()
    return (_rank() // per) * per


def full_shape(t):
    lay = get_layout(t)
    if lay is not None:
        return lay.shape
    if isinstance(t, Parameter) and t.full_shape is not None:
        return t.full_shape
    return tuple(t.shape)


def needs_dispatch(prim, args):
    if prim.in_strategy is not None:
        return True
    return any(get_layout(a) is not None for a in args if isinstance(a, torch.Tensor)) or \
        any(isinstance(a, (tuple, list)) and any(get_layout(x) is not None for x in a) for a in args)


def _group_for(dev_matrix, dev_dims):
    ranks = RD.group_ranks(dev_matrix, _rank() - _stage_base(), list(dev_dims), _stage_base())
    return M.group_for_ranks(ranks), ranks


def _mirror(param, layout):
    """Replicated parameter -> identity whose backward all-reduces the gradient over the replica group.

    A parameter whose gradient accumulates in an optimizer arena (``main_grad``) is not wrapped: it is flagged
    (``tp_grad_reduce`` + ``mirror_group``) and the optimizer all-reduces its accumulated gradient once per step,
    after the last micro-batch - what the reference's ``_MirrorMicroStepOperator`` does under gradient accumulation
    (ops/operations/comm_ops.py:1722, frontend/parallel/step_parallel.cc:1234-1322)."""
    from ..ops import comm_ops
    dims = layout.unused_dev_dims()
    if not dims or not param._ms_requires_grad:
        return param
    gname, ranks = _group_for(layout.device_matrix, dims)
    if getattr(param, "main_grad", None) is not None:
        if getattr(param, "mirror_group", None) != gname:
            param.tp_grad_reduce = True
            param.mirror_group = gname
        if _record is not None:
            _record["mirror"] += 1
        return param
    key = (gname, len(ranks))
    op = _mirror_cache.get(key)
    if op is None:
        op = comm_ops._MirrorOperator(gname, len(ranks), context.get_auto_parallel_context("gradients_mean"))
        _mirror_cache[key] = op
    if _record is not None:
        _record["mirror"] += 1
    out = op._run(_plain(param))
    return out


_equiv_cache = {}

# what the most recent ``dispatch`` inserted around its primitive; the graph tracer copies it onto the node:
# {"forward_comm": (kind, dev dims) or None, "redistribution": [operator names], "mirror": n}
last_dispatch = None
_record = None


def layouts_equivalent(a: TensorLayout, b: TensorLayout):
    """True when both layouts give every rank the same slice (e.g. device matrices that differ only by
    size-1 dims or by how the repeat dim is written)."""
    if a == b:
        return True
    key = (a, b)
    if key not in _equiv_cache:
        ok = a.shape == b.shape and a.num_devices() == b.num_devices() and \
            a.tensor_strategy() == b.tensor_strategy() and a.opt_shard_size == b.opt_shard_size and \
            all(a.slice_index(r) == b.slice_index(r) for r in range(a.num_devices()))
        _equiv_cache[key] = ok
    return _equiv_cache[key]


def _plain(t):
    return t.as_subclass(torch.Tensor) if type(t) is not torch.Tensor else t


_rebase_cache = {}


def rebase(cur: TensorLayout, device_matrix):
    """``cur`` rewritten over ``device_matrix`` (same slices on every rank), or None when that matrix has no axis
    that walks the ranks the way a split of ``cur`` does.  Producer and consumer operators each derive their own
    device matrix from their strategy (e.g. [mp, 1] for a token-split norm, [1, 1, mp] for the column-parallel
    MatMul behind it); bringing both layouts over one matrix lets redistribution inference find the single
    AllGather / StridedSlice / AlltoAll between them instead of falling back to gather-everything-then-slice."""
    dm = tuple(int(d) for d in device_matrix)
    if tuple(cur.device_matrix) == dm:
        return cur
    key = (cur, dm)
    if key in _rebase_cache:
        return _rebase_cache[key]
    out = None
    n = int(np.prod(dm)) if dm else 1
    if n == cur.num_devices() and not any(isinstance(m, tuple) for m in cur.tensor_map):
        probe = TensorLayout(dm, [-1] * len(cur.shape), cur.shape)
        coords = [probe.coord(r) for r in range(n)]
        idx = [cur.slice_index(r) for r in range(n)]
        new_map, used, ok = [], set(), True
        for i in range(len(cur.shape)):
            c = cur.split_count(i)
            if c == 1:
                new_map.append(-1)
                continue
            found = None
            for k in range(len(dm)):
                a = len(dm) - 1 - k
                if k in used or dm[a] != c:
                    continue
                if all(coords[r][a] == idx[r][i] for r in range(n)):
                    found = k
                    break
            if found is None:
                ok = False
                break
            used.add(found)
            new_map.append(found)
        if ok:
            out = TensorLayout(dm, new_map, cur.shape, cur.opt_shard_size, cur.opt_shard_step)
    _rebase_cache[key] = out
    return out


def _redistribute(x, cur, need):
    if layouts_equivalent(cur, need):
        return x
    cur = rebase(cur, need.device_matrix) or cur
    if _record is not None:
        try:
            _record["redistribution"] += RD.lowered_names(RD.infer(cur, need))
        except Exception:  # noqa: BLE001  (bookkeeping only)
            _record["redistribution"].append("Redistribution")
    return RD.apply(_plain(x), cur, need, _rank(), _stage_base())


def _prepare_input(x, need: TensorLayout):
    if isinstance(x, Parameter):
        if x.param_layout is None:
            x.init_data(need, set_sliced=True)
            parameter_layouts[x.name] = need
            set_layout(x, need)
            if any(m != -1 for m in need.tensor_map):
                x.tp_sharded = True          # ranks hold different slices: its squared norm adds up over the group
        cur = x.param_layout
        y = _redistribute(_mirror(x, cur), cur, need)
        return set_layout(y, need)
    cur = get_layout(x)
    if cur is None:
        # an untagged activation holds the full tensor on every rank (full_batch inputs, constants)
        if tuple(x.shape) == tuple(need.slice_shape()) and tuple(need.shape) != tuple(x.shape):
            return set_layout(x, need)          # already a local slice (dataset sharded by the loader)
        y = slice_for_rank(_plain(x), need, _rank() - _stage_base())
        return set_layout(y if y.is_contiguous() else y.contiguous(), need)
    from ..common.tensor import as_tensor
    return set_layout(as_tensor(_redistribute(x, cur, need)), need)


def _forward_comm(y, info, out_index=0):
    from ..communication import comm_func as CF
    fc = info.forward_comm
    if fc is None or out_index != 0:
        return y
    kind, dims = fc[0], fc[1]
    y = _plain(y)
    gname, ranks = _group_for(info.dev_matrix, dims)
    if kind == "AllReduce":
        return CF.all_reduce_autograd(y, "sum", gname)
    if kind == "AllReduceMean":
        return CF.all_reduce_autograd(y, "sum", gname) / len(ranks)
    if kind in ("AllReduceMax", "AllReduceMin"):
        return CF.all_reduce_autograd(y, kind[9:].lower(), gname)
    if kind == "ReduceScatter":
        dim = fc[2]
        if dim == 0:
            return CF.reduce_scatter_autograd(y.contiguous(), "sum", gname)
        return CF.reduce_scatter_autograd(y.movedim(dim, 0).contiguous(), "sum", gname).movedim(0, dim).contiguous()
    raise NotImplementedError(kind)


def shard_parameter(param, prim, index, shapes=None, **extra):
    """Slices ``param`` now according to what input ``index`` of ``prim`` (a primitive with a shard strategy) needs.
    ``shapes``: full shapes of all tensor inputs of ``prim`` (default: only the parameter's own is known and the
    other inputs are taken from the strategy as one row / column per split).  Models call it from ``__init__`` so
    that full weights never stay resident and an optimizer built afterwards packs the slices."""
    if not active() or prim.in_strategy is None or param.param_layout is not None:
        return param
    strategy = prim.in_strategy
    if shapes is None:
        shapes = [tuple(s) for s in strategy]
        shapes[index] = tuple(param.shape)
        if prim.name in ("MatMul", "BatchMatMul") and len(strategy) == 2:
            ta, tb = bool(getattr(prim, "transpose_a", False)), bool(getattr(prim, "transpose_b", False))
            if index == 1:
                kdim = param.shape[-1] if tb else param.shape[-2]
                m = strategy[0][-1] if ta else strategy[0][-2]
                shapes[0] = (kdim, m) if ta else (m, kdim)
    info = OI.make_info(prim, shapes, strategy, prim.out_strategy, stage_devices(), **extra)
    need = info.input_layouts()[index]
    param.init_data(need, set_sliced=True)
    parameter_layouts[param.name] = need
    set_layout(param, need)
    if any(m != -1 for m in need.tensor_map):
        param.tp_sharded = True
    return param


def _tp_group(gname):
    from . import tp as TP
    return TP.TPGroup(name=gname)


def _fused_matmul(prim, info, x, w, need):
    """Row-parallel MatMul whose forward communication is a ReduceScatter over the token rows, and column-parallel
    MatMul whose first input only needs an AllGather of its token rows, run as ONE kernel each over NVLink
    (``fused_comm``): the GEMM epilogue pushes / reduces its tiles into the owning rank, the GEMM loader pulls the
    peers' shards.  Returns the local output or NotImplemented (then redistribution + MatMul + collective run as
    separate operators).  Reference: forward ops of ops_info/matmul_info.cc:361-403 and the AllGather that
    tensor_layout/redistribution_operator_infer.cc:98-231 emits in front of the MatMul."""
    from . import fused_comm as FC
    if getattr(prim, "transpose_a", False) or not getattr(prim, "transpose_b", False):
        return NotImplemented
    if x.dim() != 2 or w.dim() != 2 or not isinstance(w, Parameter):
        return NotImplemented
    fc = info.forward_comm
    if fc is not None and fc[0] == "ReduceScatter" and fc[2] == 0:
        gname, ranks = _group_for(info.dev_matrix, fc[1])
        if not FC.available(M._group(gname)):
            return NotImplemented
        xl = _plain(_prepare_input(x, need[0]))
        wl = _prepare_input(w, need[1])
        if _record is not None:
            _record["fused"] = "MatMulReduceScatter"
        return FC.matmul_reduce_scatter(xl, wl, _tp_group(gname))
    if fc is None:
        cur = get_layout(x)
        if cur is None or layouts_equivalent(cur, need[0]):
            return NotImplemented
        cur = rebase(cur, need[0].device_matrix) or cur
        try:
            ops = RD.infer(cur, need[0])
        except Exception:  # noqa: BLE001
            return NotImplemented
        if ops is None or len(ops) != 1 or ops[0].type != RD.CONCAT or ops[0].dim != 0:
            return NotImplemented
        gname, ranks = _group_for(cur.device_matrix, [ops[0].dev_dim])
        if not FC.available(M._group(gname)):
            return NotImplemented
        wl = _prepare_input(w, need[1])
        if _record is not None:
            _record["fused"] = "AllGatherMatMul"
            _record["redistribution"].append("AllGather")
        return FC.allgather_matmul(_plain(x), wl, _tp_group(gname))
    return NotImplemented


def _vocab_parallel_loss(info, logits, labels, need):
    """SparseSoftmaxCrossEntropyWithLogits with a split class dim: per-shard (max, sum-exp, target) statistics
    from one pass over the local logits, combined over the class group; the gradient of the local shard is written
    in one pass too (``parallel.tp._VocabParallelCE``)."""
    from . import tp as TP
    k = info.inputs_tensor_map[0][1]
    gname, ranks = _group_for(info.dev_matrix, [k])
    pos = RD._coord_along(info.dev_matrix, _rank() - _stage_base(), k)
    ll = _plain(_prepare_input(logits, need[0])).contiguous()
    lb = _plain(_prepare_input(labels, need[1]))
    if _record is not None:
        _record["fused"] = "VocabParallelCrossEntropy"
    return TP._VocabParallelCE.apply(ll, lb, gname, pos, -100)


def _follow_strategy(prim, tensors):
    """Strategy of an un-annotated primitive: follow the first sharded input when shapes allow (elementwise
    'strategy follow'), else replicate."""
    lays = [get_layout(t) for t in tensors]
    first = next((l for l in lays if l is not None), None)
    if first is None:
        return None
    strat = []
    for t, l in zip(tensors, lays):
        shp = full_shape(t)
        if l is not None:
            strat.append(l.tensor_strategy())
        elif len(shp) == len(first.shape) and all(a == b or a == 1 for a, b in zip(shp, first.shape)):
            fs = first.tensor_strategy()
            strat.append(tuple(1 if a == 1 else s for a, s in zip(shp, fs)))
        else:
            strat.append(tuple(1 for _ in shp))
    return tuple(strat)


# Non-tensor call arguments that the OperatorInfo of a primitive needs by name (position among the non-tensor
# arguments of the call).
_EXTRA_ARGS = {
    "Transpose": ("perm",), "Reshape": ("shape",), "Gather": ("axis",), "SparseGatherV2": ("axis",),
    "OneHot": ("depth",), "StridedSlice": ("begin", "end", "strides"), "Slice": ("begin", "size"),
    "SliceExt": ("begin", "size"), "Tile": ("multiples",), "ExpandDims": ("axis",), "CumSum": ("axis",),
    "CumProd": ("axis",), "Cummax": ("axis",), "Cummin": ("axis",), "TopK": ("k",), "TopkExt": ("k",),
    "GatherD": ("dim",), "UnsortedSegmentSum": ("num_segments",), "UnsortedSegmentProd": ("num_segments",),
    "ReverseV2": ("axis",), "PadV3": ("paddings",),
}
_REDUCE = ("ReduceSum", "ReduceMean", "ReduceMax", "ReduceMin", "ReduceAll", "ReduceAny", "ReduceProd")


def _flatten_args(args):
    """Tensor arguments of a call in order; a tuple / list of tensors (Concat, Stack, AddN) contributes its members.
    Returns (tensors, slots) with slots[i] = (position, index inside the sequence or None)."""
    tensors, slots = [], []
    for i, a in enumerate(args):
        if isinstance(a, torch.Tensor):
            tensors.append(a)
            slots.append((i, None))
        elif isinstance(a, (tuple, list)) and a and all(isinstance(x, torch.Tensor) for x in a):
            for j, x in enumerate(a):
                tensors.append(x)
                slots.append((i, j))
    return tensors, slots


def build_info(prim, tensors, others, strategy=None):
    """OperatorInfo of ``prim`` for these tensor inputs (full shapes are taken from their layouts) and non-tensor
    arguments; ``strategy`` defaults to the primitive's own, else to following the sharded inputs.  Returns None
    when the call carries nothing to shard."""
    strategy = prim.in_strategy if strategy is None else strategy
    if strategy is None:
        strategy = _follow_strategy(prim, tensors)
        if strategy is None:
            return None
    if len(strategy) < len(tensors) and not (len(strategy) == 1 and prim.name in ("Concat", "Stack", "AddN")):
        strategy = tuple(strategy) + tuple(tuple(1 for _ in full_shape(t)) for t in tensors[len(strategy):])
    shapes = [full_shape(t) for t in tensors]
    extra = {}
    name = prim.name
    if name in _REDUCE:
        extra["axis"] = others[0] if others else ()
    else:
        for key, val in zip(_EXTRA_ARGS.get(name, ()), others):
            extra[key] = val
        if name in ("Gather", "SparseGatherV2"):
            extra.setdefault("axis", 0)
    n = len(shapes) if len(strategy) == 1 and len(shapes) > 1 else len(strategy)
    return OI.make_info(prim, shapes[:n], strategy[:len(shapes)], prim.out_strategy, stage_devices(), **extra)


def _sync_batch_norm(prim, info, x, scale, bias, mean, var):
    """Training-mode BatchNorm on a batch (or spatially) split input: per-channel sums are all-reduced over the
    device dims that spread a channel's samples, then every rank normalises its slice with the global statistics and
    applies the same moving-average update (reference: the forward AllReduce of ops_info/batchnorm_info.cc)."""
    from ..communication import comm_func as CF
    gname, ranks = _group_for(info.dev_matrix, info.stat_dev_dims())
    c = x.shape[1]
    dims = [0] + list(range(2, x.dim()))
    xf = x.float()
    local = torch.cat([xf.sum(dims), (xf * xf).sum(dims), xf.new_full((1,), float(x.numel() // c))])
    tot = CF.all_reduce_autograd(local, "sum", gname)
    n = tot[-1]
    m = tot[:c] / n
    v = (tot[c:2 * c] / n - m * m).clamp_min(0)
    shp = [1, c] + [1] * (x.dim() - 2)
    y = ((xf - m.view(shp)) * torch.rsqrt(v.view(shp) + prim.epsilon) * scale.float().view(shp)
         + bias.float().view(shp)).to(x.dtype)
    with torch.no_grad():
        mom = float(prim.momentum)
        unbiased = v * (n / (n - 1).clamp_min(1))
        torch.Tensor.mul_(mean, 1 - mom).add_(m.to(mean.dtype) * mom)
        torch.Tensor.mul_(var, 1 - mom).add_(unbiased.to(var.dtype) * mom)
    return y, mean, var, mean, var


def run_local(prim, info, local, other_pos, others, tensor_pos, kwargs, rank_in_stage, sync_bn=None):
    """The primitive on one rank's slices: ``local`` is the argument list with tensors already replaced by their
    slices; shape-like arguments and attributes are rewritten the way ``info`` says the slice must see them."""
    name = prim.name
    la = info.local_attrs()
    if name == "Reshape" and "shape" in la:
        local[other_pos[0]] = la["shape"]
    else:
        for pos, v in zip(other_pos, info.localize_args(others)):
            local[pos] = v
    saved = {}
    for k, v in la.items():
        if (k != "shape" or name != "Reshape") and hasattr(prim, k):
            saved[k] = getattr(prim, k)
            setattr(prim, k, v)
    try:
        if name in ("Gather", "EmbeddingLookup", "SparseGatherV2") and info.vocab_split() > 1:
            from ..ops import fused
            k = info.inputs_tensor_map[0][0]
            pos = RD._coord_along(info.dev_matrix, rank_in_stage, k)
            return fused.embedding(local[tensor_pos[0]], local[tensor_pos[1]], pos * local[tensor_pos[0]].shape[0])
        if name == "BatchNorm" and info.needs_sync_stats():
            fn = sync_bn or _sync_batch_norm
            return fn(prim, info, *[local[i] for i in tensor_pos][:5])
        return prim._run(*local, **kwargs)
    finally:
        for k, v in saved.items():
            setattr(prim, k, v)


def dispatch(prim, args, kwargs):
    """Runs ``prim`` under its shard strategy.  Returns NotImplemented when the primitive takes no tensor."""
    tensors, slots = _flatten_args(args)
    if not tensors:
        return NotImplemented
    tensor_positions = {i for i, _ in slots}
    other_pos = [i for i in range(len(args)) if i not in tensor_positions]
    others = [args[i] for i in other_pos]
    name = prim.name
    try:
        info = build_info(prim, tensors, others)
    except OI.StrategyError:
        if prim.in_strategy is not None:
            raise
        return _run_replicated(prim, args, kwargs)
    if info is None:
        return NotImplemented
    global _record, last_dispatch
    _record = {"forward_comm": tuple(info.forward_comm[:2]) if info.forward_comm else None, "redistribution": [],
               "mirror": 0, "fused": None}
    need = info.input_layouts()
    from ..common.tensor import as_tensor
    fused_out = NotImplemented
    if name == "MatMul" and len(tensors) == 2:
        fused_out = _fused_matmul(prim, info, tensors[0], tensors[1], need)
    elif name == "SparseSoftmaxCrossEntropyWithLogits" and info.class_split() > 1 and len(tensors) == 2:
        fused_out = _vocab_parallel_loss(info, tensors[0], tensors[1], need)
        if fused_out is not NotImplemented:
            fused_out = _forward_comm(fused_out, info)
    if fused_out is not NotImplemented:
        last_dispatch, _record = _record, None
        return set_layout(as_tensor(fused_out), info.output_layouts()[0])
    # inputs -> required layouts (redistribution, parameter slicing, mirrors)
    prepared = []
    for j, t in enumerate(tensors):
        if j < len(need):
            v = _prepare_input(t, need[j])
            prepared.append(v if isinstance(v, Parameter) else _plain(v))
        else:
            prepared.append(t)
    local = list(args)
    seqs = {}
    for (pos, sub), v in zip(slots, prepared):
        if sub is None:
            local[pos] = v
        else:
            seqs.setdefault(pos, list(args[pos]))[sub] = v
    for pos, seq in seqs.items():
        local[pos] = type(args[pos])(seq)
    out = run_local(prim, info, local, other_pos, others, sorted(tensor_positions), kwargs,
                    _rank() - _stage_base())
    last_dispatch, _record = _record, None
    if isinstance(out, torch.Tensor):
        out_lays = info.output_layouts([tuple(out.shape)])
        out = as_tensor(_forward_comm(out, info))
        return set_layout(out, out_lays[0])
    if isinstance(out, (tuple, list)):
        out_lays = info.output_layouts([tuple(o.shape) if isinstance(o, torch.Tensor) else () for o in out])
        res = []
        for i, o in enumerate(out):
            if isinstance(o, torch.Tensor) and i < len(out_lays):
                res.append(set_layout(as_tensor(_forward_comm(o, info, i)), out_lays[i]))
            else:
                res.append(o)
        return type(out)(res)
    return out


def _run_replicated(prim, args, kwargs):
    """Gathers every sharded input to its full value and runs the primitive replicated."""
    local = []
    for a in args:
        lay = get_layout(a)
        if lay is not None:
            full = TensorLayout(lay.device_matrix, [-1] * len(lay.shape), lay.shape)
            a = RD.apply(_plain(a), lay, full, _rank(), _stage_base())
        local.append(a)
    return prim._run(*local, **kwargs)


def to_full(t):
    """Full (replicated) value of a possibly sharded tensor."""
    lay = get_layout(t)
    if lay is None:
        return t
    full = TensorLayout(lay.device_matrix, [-1] * len(lay.shape), lay.shape)
    out = RD.apply(_plain(t), lay, full, _rank(), _stage_base())
    from ..common.tensor import as_tensor
    return as_tensor(out)


def virtual_div_loss(loss):
    """Applies _VirtualDiv when the (scalar) loss is replicated over r ranks and ``loss_repeated_mean`` is on."""
    from ..ops import comm_ops
    lay = get_layout(loss)
    r = lay.repeat_num() if lay is not None else stage_devices()
    if r > 1 and context.get_auto_parallel_context("loss_repeated_mean"):
        return comm_ops._VirtualDiv(r)(loss)
    return loss


def reset():
    parameter_layouts.clear()
    _mirror_cache.clear()


_SHAPE_CHANGING = ("sum", "mean", "amax", "amin", "max", "min", "prod", "matmul", "mm", "bmm", "reshape", "view",
                   "permute", "transpose", "cat", "stack", "softmax", "log_softmax", "layer_norm", "linear",
                   "__getitem__", "narrow", "index_select", "gather", "cumsum", "norm", "flatten", "squeeze",
                   "unsqueeze", "expand", "repeat", "var", "std", "argmax", "argmin", "topk", "sort")


def propagate_elementwise(func, args, out):
    """Layout propagation for plain tensor arithmetic (``y * y``, ``x + 1`` ...) that does not go through a
    Primitive: a shape-preserving function of sharded operands yields a result with the same layout.  Any other
    torch function applied to a sharded tensor is refused, because its result would silently be a partial value:
    use the ``ops`` primitives (which know their distributed semantics) instead."""
    if not isinstance(out, torch.Tensor):
        return
    lay = None
    for a in args:
        l = get_layout(a)
        if l is not None:
            if lay is not None and l != lay:
                return
            lay = l
    if lay is None:
        return
    name = getattr(func, "__name__", "")
    if name in ("detach", "clone", "contiguous", "to", "type", "float", "bfloat16", "half", "requires_grad_",
                "view_as", "alias", "__get__", "__set__", "data", "as_subclass", "size", "dim", "numel", "stride",
                "is_contiguous", "element_size", "storage_offset", "data_ptr", "backward", "register_hook",
                "__repr__", "__format__", "item", "tolist", "cpu", "cuda", "numpy", "is_floating_point",
                "is_complex", "__hash__", "__bool__", "__len__", "isfinite", "isnan"):
        if tuple(out.shape) == tuple(lay.slice_shape()):
            set_layout(out, lay)
        return
    if name in _SHAPE_CHANGING:
        raise NotImplementedError("torch function %r was applied to a tensor sharded as %s; in (semi_)auto_parallel "
                                  "mode use the ops primitives, which carry distributed semantics" % (name, lay))
    if tuple(out.shape) == tuple(lay.slice_shape()):
        set_layout(out, lay)
