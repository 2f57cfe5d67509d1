"""Virtual execution of a sharded primitive: every rank of a device matrix is played in turn inside one process.

``run_sharded(prim, args, in_strategy, out_strategy, device_num)`` slices the full inputs the way the primitive's
OperatorInfo asks for, runs the local operator per virtual rank (with the shape arguments and attributes of a
slice), applies the forward communication over the rank groups, and re-assembles the full outputs from the
per-rank results with the output layouts.  The result must equal the unsharded operator: that is the contract every
OperatorInfo is tested against (random legal strategies), and a way to look at what a strategy does without
starting a job.  No communication library is involved.
"""
from __future__ import annotations

import numpy as np
import torch

from . import operator_info as OI
from . import redistribution as RD
from .layout import slice_for_rank


def _reduce(kind, parts):
    st = torch.stack([p.float() for p in parts])
    if kind in ("AllReduce", "ReduceScatter"):
        return st.sum(0)
    if kind == "AllReduceMean":
        return st.mean(0)
    if kind == "AllReduceMax":
        return st.amax(0)
    if kind == "AllReduceMin":
        return st.amin(0)
    raise NotImplementedError(kind)


def run_sharded(prim, args, in_strategy, out_strategy=None, device_num=4, kwargs=None):
    """-> (full outputs as a list of tensors, info).  ``args`` are the full (unsharded) call arguments."""
    from . import spmd
    kwargs = kwargs or {}
    tensors, slots = spmd._flatten_args(args)
    tensor_positions = sorted({i for i, _ in slots})
    other_pos = [i for i in range(len(args)) if i not in tensor_positions]
    others = [args[i] for i in other_pos]
    saved = (prim.in_strategy, prim.out_strategy)
    prim.in_strategy, prim.out_strategy = tuple(in_strategy), out_strategy
    try:
        extra = {}
        if prim.name in spmd._REDUCE:
            extra["axis"] = others[0] if others else ()
        else:
            for key, val in zip(spmd._EXTRA_ARGS.get(prim.name, ()), others):
                extra[key] = val
            if prim.name in ("Gather", "SparseGatherV2"):
                extra.setdefault("axis", 0)
        shapes = [tuple(t.shape) for t in tensors]
        n = len(shapes) if len(in_strategy) == 1 and len(shapes) > 1 else len(in_strategy)
        info = OI.make_info(prim, shapes[:n], tuple(in_strategy)[:len(shapes)], out_strategy, device_num, **extra)
    finally:
        prim.in_strategy, prim.out_strategy = saved
    need = info.input_layouts()
    world = int(np.prod(info.dev_matrix)) if info.dev_matrix else 1

    # BatchNorm on a split batch needs the statistics of all ranks: compute them once from the full input
    def sync_bn(p, inf, x, scale, bias, mean, var):
        full = tensors[0].float()
        c = full.shape[1]
        dims = [0] + list(range(2, full.dim()))
        shp = [1, c] + [1] * (full.dim() - 2)
        cm = inf.inputs_tensor_map[0][1]
        if cm != -1:                       # this rank's channel slice of the global statistics
            cnt = inf.dev_matrix[len(inf.dev_matrix) - 1 - cm]
            pos = RD._coord_along(inf.dev_matrix, sync_bn.rank, cm)
            full = full.chunk(cnt, 1)[pos]
            c = full.shape[1]
            shp[1] = c
        m, v = full.mean(dims), full.var(dims, unbiased=False)
        y = ((x.float() - m.view(shp)) * torch.rsqrt(v.view(shp) + p.epsilon) * scale.float().view(shp)
             + bias.float().view(shp)).to(x.dtype)
        return y, mean, var, mean, var

    per_rank = []
    for r in range(world):
        sync_bn.rank = r
        local = list(args)
        seqs = {}
        for j, ((pos, sub), t) in enumerate(zip(slots, tensors)):
            v = slice_for_rank(t, need[j], r).contiguous() if j < len(need) else t
            if sub is None:
                local[pos] = v
            else:
                seqs.setdefault(pos, list(args[pos]))[sub] = v
        for pos, seq in seqs.items():
            local[pos] = type(args[pos])(seq)
        out = spmd.run_local(prim, info, local, other_pos, others, tensor_positions, kwargs, r, sync_bn=sync_bn)
        per_rank.append(list(out) if isinstance(out, (tuple, list)) else [out])
    n_out = len(per_rank[0])
    # forward communication on output 0
    fc = info.forward_comm
    if fc is not None:
        kind, dims = fc[0], fc[1]
        reduced = []
        for r in range(world):
            group = RD.group_ranks(info.dev_matrix, r, list(dims))
            full = _reduce(kind, [per_rank[q][0] for q in group]).to(per_rank[r][0].dtype)
            if kind == "ReduceScatter":
                full = full.chunk(len(group), fc[2])[group.index(r)]
            reduced.append(full)
        for r in range(world):
            per_rank[r][0] = reduced[r]
    lays = info.output_layouts([tuple(o.shape) if isinstance(o, torch.Tensor) else () for o in per_rank[0]])
    fulls = []
    from .layout import assemble_full
    for i in range(n_out):
        if not isinstance(per_rank[0][i], torch.Tensor) or i >= len(lays):
            fulls.append(per_rank[0][i])
            continue
        parts = {r: per_rank[r][i].detach().float().numpy() for r in range(world)}
        fulls.append(torch.from_numpy(assemble_full(parts, lays[i])))
    return fulls, info
