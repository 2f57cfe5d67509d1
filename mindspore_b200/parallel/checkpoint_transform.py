"""Transformation of distributed checkpoints between shard strategies.

A parameter saved under one layout is a set of rectangular regions of the full tensor, one per rank.  Converting
to another layout is region arithmetic: for the region a destination rank needs, copy the overlapping part of
every source region.  That covers tensor-parallel resharding, optimizer-shard (dim-0 sub-slices over replicas)
merging and pipeline-stage regrouping with one routine, without building the operator lists the reference
replays on numpy arrays.

Parity: mindspore/python/mindspore/parallel/checkpoint_transform.py:36 (merge_pipeline_strategys),
:76 (rank_list_for_transform), :140 (transform_checkpoint_by_rank), :361 (transform_checkpoints),
:474 (sync_pipeline_shared_parameters); parallel/_parallel_serialization.py (_transform_parallel_checkpoint);
train/serialization.py:2266 (merge_sliced_parameter), :2353 (load_distributed_checkpoint)."""
from __future__ import annotations

import glob
import os
import re

import numpy as np
import torch

from .strategy_ckpt import ParamLayoutEntry, StrategyFile
from .layout import TensorLayout


# ------------------------------------------------------------------------------------ regions
def region(layout: TensorLayout, rank):
    """[(start, stop)] per tensor dim of the part of the full tensor that ``rank`` holds."""
    idx = layout.slice_index(rank)
    reg = []
    for i, d in enumerate(layout.shape):
        step = d // layout.split_count(i)
        reg.append([idx[i] * step, (idx[i] + 1) * step])
    if layout.opt_shard_size and layout.opt_shard_size > 1 and reg:
        group = layout.replica_group(rank % layout.num_devices())
        pos = group.index(rank % layout.num_devices()) % layout.opt_shard_size
        step = (reg[0][1] - reg[0][0]) // layout.opt_shard_size
        reg[0] = [reg[0][0] + pos * step, reg[0][0] + (pos + 1) * step]
    return [tuple(r) for r in reg]


def _overlap(a, b):
    out = []
    for (a0, a1), (b0, b1) in zip(a, b):
        lo, hi = max(a0, b0), min(a1, b1)
        if lo >= hi:
            return None
        out.append((lo, hi))
    return out


def merge_opt_shard_slices(slices_by_rank, layout: TensorLayout):
    """Full numpy array from per-rank slices of a layout that may carry optimizer sharding."""
    first = next(iter(slices_by_rank.values()))
    full = np.zeros(layout.shape, dtype=first.dtype)
    for rank, sl in slices_by_rank.items():
        reg = region(layout, rank)
        full[tuple(slice(a, b) for a, b in reg)] = np.asarray(sl).reshape([b - a for a, b in reg])
    return full


def _full_layout(shape):
    return TensorLayout((1,), [-1] * len(shape), shape)


def _needed_src_ranks(src_layout, dst_region, src_ranks):
    """Smallest prefix-ordered set of source ranks whose regions tile ``dst_region``."""
    need, seen = [], set()
    for r in src_ranks:
        reg = tuple(region(src_layout, r))
        if reg in seen:
            continue
        if _overlap(reg, dst_region) is not None:
            need.append(r)
            seen.add(reg)
    return need


# ------------------------------------------------------------------------------------ strategy files
def _load_strategy(path):
    return None if path is None else StrategyFile.load(path)


def merge_pipeline_strategys(src_strategy_dirs, dst_strategy_file):
    """Merges the per-stage strategy files found in ``src_strategy_dirs`` into one file covering every stage."""
    files = sorted(glob.glob(os.path.join(src_strategy_dirs, "*.ckpt")) +
                   glob.glob(os.path.join(src_strategy_dirs, "*.json")))
    if not files:
        raise ValueError("no strategy files (*.ckpt, *.json) in %s" % src_strategy_dirs)
    merged = StrategyFile(0)
    for f in files:
        sf = StrategyFile.load(f)
        for n, e in sf.layouts.items():
            e.stage = sf.current_stage
            merged.layouts.setdefault(n, e)
        for n, s in sf.strategies.items():
            merged.strategies.setdefault(n, s)
    merged.save(dst_strategy_file)
    return merged


def _stage_device_num(sf):
    for e in sf.layouts.values():
        return int(np.prod(e.dev_matrix))
    return 1


def _world_of(sf):
    """(devices per stage, stages) of a merged strategy file."""
    if sf is None:
        return 1, 1
    stages = max([e.stage for e in sf.layouts.values()] + [0]) + 1
    return _stage_device_num(sf), stages


def rank_list_for_transform(rank_id, src_strategy_file=None, dst_strategy_file=None):
    """Source ranks whose checkpoints are needed to build the checkpoint of destination rank ``rank_id``."""
    src, dst = _load_strategy(src_strategy_file), _load_strategy(dst_strategy_file)
    src_per, src_stages = _world_of(src)
    dst_per, _ = _world_of(dst)
    need = set()
    names = set(src.layouts if src else ()) | set(dst.layouts if dst else ())
    if not names:
        return [0]
    for n in names:
        se = src.layouts.get(n) if src else None
        de = dst.layouts.get(n) if dst else None
        if dst is not None and de is not None and de.stage != rank_id // dst_per:
            continue
        if dst is not None and de is None:
            continue
        # shapes are unknown here: work on a virtual tensor large enough to be divisible by every split
        if se is None:
            need.add(0)                    # not sharded at the source: any rank holds all of it
            continue
        unit = [a * b for a, b in zip(se.split_counts(), de.split_counts() if de else [1] * len(se.tensor_map))]
        if unit:
            unit[0] *= max(se.opt_shard_size, 1) * max(de.opt_shard_size if de else 1, 1)
        s_lay = se.to_layout(full_shape=unit)
        d_lay = de.to_layout(full_shape=unit) if de else _full_layout(unit)
        d_reg = region(d_lay, rank_id % dst_per if de else 0)
        base = se.stage * src_per
        for r in _needed_src_ranks(s_lay, d_reg, range(src_per)):
            need.add(base + r)
    return sorted(need)


# ------------------------------------------------------------------------------------ transformation
def _to_numpy(t):
    t = t.detach() if isinstance(t, torch.Tensor) else torch.as_tensor(t)
    t = t.as_subclass(torch.Tensor)
    if t.dtype == torch.bfloat16:
        return t.float().cpu().numpy(), torch.bfloat16
    return t.cpu().numpy(), t.dtype


def transform_param(name, src_slices, src_entry, dst_entry, dst_rank_in_stage):
    """One parameter: ``src_slices`` {rank in stage: array} under ``src_entry`` -> array for the destination rank.
    ``None`` entries mean "not sharded" (the full tensor on every rank)."""
    any_slice = next(iter(src_slices.values()))
    if src_entry is None:
        full_shape = list(any_slice.shape)
        s_lay = _full_layout(full_shape)
    else:
        s_lay = src_entry.to_layout(slice_shape=list(any_slice.shape))
        full_shape = list(s_lay.shape)
    d_lay = _full_layout(full_shape) if dst_entry is None else dst_entry.to_layout(full_shape=full_shape)
    d_reg = region(d_lay, dst_rank_in_stage if dst_entry is not None else 0)
    out = np.zeros([b - a for a, b in d_reg], dtype=any_slice.dtype)
    covered = 0
    seen = set()
    for r, sl in src_slices.items():
        s_reg = tuple(region(s_lay, r if src_entry is not None else 0))
        if s_reg in seen:
            continue
        ov = _overlap(s_reg, d_reg)
        if ov is None:
            continue
        seen.add(s_reg)
        src_sel = tuple(slice(lo - s0, hi - s0) for (lo, hi), (s0, _) in zip(ov, s_reg))
        dst_sel = tuple(slice(lo - d0, hi - d0) for (lo, hi), (d0, _) in zip(ov, d_reg))
        out[dst_sel] = np.asarray(sl)[src_sel]
        covered += int(np.prod([hi - lo for lo, hi in ov])) if ov else 1
    if covered < out.size:
        raise ValueError("parameter %s: the given source checkpoints cover %d of %d elements needed by the "
                         "destination rank" % (name, covered, out.size))
    return out


def transform_checkpoint_by_rank(rank_id, checkpoint_files_map, save_checkpoint_file_name,
                                 src_strategy_file=None, dst_strategy_file=None):
    """Builds the checkpoint of destination rank ``rank_id`` from source checkpoints ``{src rank: file}``."""
    from ..train.serialization import load_checkpoint, save_checkpoint
    if not isinstance(checkpoint_files_map, dict):
        raise TypeError("checkpoint_files_map must be a dict {rank: file}")
    for r, f in checkpoint_files_map.items():
        if not os.path.isfile(f):
            raise ValueError("checkpoint file %s of rank %s does not exist" % (f, r))
    src, dst = _load_strategy(src_strategy_file), _load_strategy(dst_strategy_file)
    src_per, _ = _world_of(src)
    dst_per, _ = _world_of(dst)
    loaded = {r: load_checkpoint(f) for r, f in checkpoint_files_map.items()}
    names = []
    for d in loaded.values():
        for n in d:
            if n not in names:
                names.append(n)
    out = []
    for n in names:
        se = src.layouts.get(n) if src else None
        de = dst.layouts.get(n) if dst else None
        if dst is not None and de is not None and de.stage != rank_id // dst_per:
            continue
        slices, dtype = {}, None
        for r, d in loaded.items():
            if n in d:
                arr, dtype = _to_numpy(d[n])
                slices[r % src_per if se is not None else r] = arr
        if se is None and de is None:
            arr = next(iter(slices.values()))
        else:
            arr = transform_param(n, slices, se, de, rank_id % dst_per)
        out.append({"name": n, "data": torch.from_numpy(np.ascontiguousarray(arr)).to(dtype)})
    save_checkpoint(out, save_checkpoint_file_name)


def _rank_of_dir(d):
    m = re.search(r"rank_(\d+)$", d.rstrip("/"))
    return int(m.group(1)) if m else None


def transform_checkpoints(src_checkpoints_dir, dst_checkpoints_dir, ckpt_prefix, src_strategy_file=None,
                          dst_strategy_file=None, process_num=1, output_format="ckpt"):
    """``src_checkpoints_dir/rank_{i}/*.ckpt`` under the source strategy -> ``dst_checkpoints_dir/rank_{j}/
    {ckpt_prefix}{j}.ckpt`` under the destination strategy, for every destination rank."""
    if not os.path.isdir(src_checkpoints_dir):
        raise NotADirectoryError("src_checkpoints_dir %s is not a directory" % src_checkpoints_dir)
    files = {}
    for d in glob.glob(os.path.join(src_checkpoints_dir, "rank_*")):
        r = _rank_of_dir(d)
        cks = sorted(glob.glob(os.path.join(d, "*.ckpt")), key=os.path.getmtime)
        if r is not None and cks:
            files[r] = cks[-1]
    if not files:
        raise ValueError("no rank_*/ *.ckpt under %s" % src_checkpoints_dir)
    dst = _load_strategy(dst_strategy_file)
    dst_per, dst_stages = _world_of(dst)
    for rank in range(dst_per * dst_stages):
        need = rank_list_for_transform(rank, src_strategy_file, dst_strategy_file)
        missing = [r for r in need if r not in files]
        if missing:
            raise ValueError("destination rank %d needs checkpoints of source ranks %s" % (rank, missing))
        out_dir = os.path.join(dst_checkpoints_dir, "rank_%d" % rank)
        os.makedirs(out_dir, exist_ok=True)
        transform_checkpoint_by_rank(rank, {r: files[r] for r in need},
                                     os.path.join(out_dir, "%s%d.ckpt" % (ckpt_prefix, rank)),
                                     src_strategy_file, dst_strategy_file)


# ------------------------------------------------------------------------------------ loading helpers
def merge_sliced_parameter(sliced_parameters, strategy=None):
    """Full Parameter from the list of per-rank slices (rank order) of one parameter."""
    from ..common.parameter import Parameter
    if not sliced_parameters:
        raise ValueError("sliced_parameters is empty")
    name = sliced_parameters[0].name
    arrs = [_to_numpy(p) for p in sliced_parameters]
    dtype = arrs[0][1]
    slices = {r: a for r, (a, _) in enumerate(arrs)}
    entry = None
    if strategy:
        if name not in strategy:
            raise KeyError("parameter %s is not in the strategy" % name)
        e = strategy[name]
        entry = e if isinstance(e, ParamLayoutEntry) else ParamLayoutEntry(e[0], e[1], e[2], e[3], e[4], e[5], e[6])
    if entry is None:
        if any(a.shape != arrs[0][0].shape or not np.array_equal(a, arrs[0][0]) for a, _ in arrs[1:]):
            raise ValueError("without a strategy every slice of %s must be identical" % name)
        full = arrs[0][0]
    else:
        full = transform_param(name, slices, entry, None, 0)
    return Parameter(torch.from_numpy(np.ascontiguousarray(full)).to(dtype), name=name,
                     requires_grad=sliced_parameters[0].requires_grad)


def load_distributed_checkpoint(network, checkpoint_filenames, predict_strategy=None, train_strategy_filename=None,
                                strict_load=False, dec_key=None, dec_mode="AES-GCM"):
    """Loads checkpoints saved by every training rank (``checkpoint_filenames`` in rank order) into ``network``
    laid out by ``predict_strategy`` (None = stand-alone full parameters)."""
    from .. import context
    from ..common.parameter import Parameter
    from ..train.serialization import load_checkpoint, load_param_into_net
    train = StrategyFile.load(train_strategy_filename) if train_strategy_filename else None
    rank = context.get_auto_parallel_context("global_rank") if predict_strategy else 0
    loaded = {r: load_checkpoint(f, dec_key=dec_key, dec_mode=dec_mode) for r, f in enumerate(checkpoint_filenames)
              if f and os.path.isfile(f)}
    if not loaded:
        raise ValueError("none of the checkpoint files exists")
    per, _ = _world_of(train)
    params = {}
    names = []
    for d in loaded.values():
        names += [n for n in d if n not in names]
    for n in names:
        se = train.layouts.get(n) if train else None
        de = None
        if predict_strategy and n in predict_strategy:
            e = predict_strategy[n]
            de = e if isinstance(e, ParamLayoutEntry) else ParamLayoutEntry(*e[:7])
        slices, dtype = {}, None
        for r, d in loaded.items():
            if n in d:
                arr, dtype = _to_numpy(d[n])
                slices[r % per if se is not None else r] = arr
        arr = transform_param(n, slices, se, de, rank % int(np.prod(de.dev_matrix)) if de else 0) \
            if (se is not None or de is not None) else next(iter(slices.values()))
        params[n] = Parameter(torch.from_numpy(np.ascontiguousarray(arr)).to(dtype), name=n)
    load_param_into_net(network, params, strict_load=strict_load)
    return params


def sync_pipeline_shared_parameters(net):
    """Makes parameters that live on several pipeline stages (tied embeddings) identical: the lowest stage that
    owns the parameter broadcasts it to the others."""
    import torch.distributed as dist
    from .. import context
    stages = context.get_auto_parallel_context("pipeline_stages")
    if stages <= 1 or not dist.is_initialized():
        return
    world = context.get_auto_parallel_context("device_num")
    rank = context.get_auto_parallel_context("global_rank")
    per = world // stages
    for p in net.get_parameters():
        st = sorted(getattr(p, "_pipeline_stage_list", []))
        if len(st) < 2:
            continue
        from ..communication import management as M
        # every rank takes part in creating every group (group creation is collective over the world)
        for pos in range(per):
            ranks = [s * per + pos for s in st]
            g = M.group_for_ranks(ranks)
            if rank in ranks:
                dist.broadcast(p.detach().as_subclass(torch.Tensor), ranks[0], group=M._group(g).pg)


def load_segmented_checkpoints(ckpt_file_dir, net=None, strict_load=False, filter_prefix=None, dec_key=None,
                               dec_mode="AES-GCM", specify_prefix=None, choice_func=None):
    """Loads every ``*.ckpt`` of a directory into one parameter dict (parallel/checkpoint_transform.py)."""
    from ..train.serialization import load_segmented_checkpoints as impl
    return impl(ckpt_file_dir, net, strict_load, filter_prefix, dec_key, dec_mode, specify_prefix, choice_func)
