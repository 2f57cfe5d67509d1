"""Tensor redistribution between layouts.

``infer(from_layout, to_layout)`` asks the native library for the operator list (SplitByAxis / PermuteByAxis /
ConcatByAxis); ``apply`` executes it on this rank with real collectives (differentiable: AllGather <->
ReduceScatter, AlltoAll <-> AlltoAll, StridedSlice <-> zero-pad); ``apply_virtual`` executes it for all ranks at
once on NumPy arrays - the path used by checkpoint transformation where no devices are involved.

Parity: ccsrc/frontend/parallel/tensor_layout/tensor_redistribution.cc:35-143,977-1066,
redistribution_operator_infer.cc:98-231, construct_operator.cc:51-390; python/mindspore/parallel/_tensor.py:342-626.
"""
from __future__ import annotations

import ctypes

import numpy as np
import torch

from .. import _native, context
from ..communication import comm_func as CF
from ..communication import management as M
from .layout import TensorLayout, ranks_along_dims

SPLIT, CONCAT, PERMUTE = 1, 2, 3
_NAMES = {SPLIT: "StridedSlice", CONCAT: "AllGather", PERMUTE: "AlltoAll"}

_lib = None


def _host():
    global _lib
    if _lib is None:
        lib = _native.host()
        I32P = ctypes.POINTER(ctypes.c_int32)
        lib.msb_redistribution_infer.restype = ctypes.c_int
        lib.msb_redistribution_infer.argtypes = [I32P, ctypes.c_int, I32P, I32P, ctypes.c_int, ctypes.c_int, I32P,
                                                 ctypes.c_int]
        lib.msb_group_ranks.restype = ctypes.c_int
        lib.msb_group_ranks.argtypes = [I32P, ctypes.c_int, ctypes.c_int, I32P, ctypes.c_int, ctypes.c_int, I32P,
                                        ctypes.c_int]
        lib.msb_redistribution_cost.restype = ctypes.c_double
        lib.msb_redistribution_cost.argtypes = [I32P, ctypes.c_int, ctypes.c_double]
        _lib = lib
    return _lib


def _i32(seq):
    arr = (ctypes.c_int32 * max(len(seq), 1))()
    for i, v in enumerate(seq):
        arr[i] = int(v)
    return arr


class RedistOp:
    __slots__ = ("type", "dim", "concat_dim", "dev_dim", "count")

    def __init__(self, t, a, b, k, c):
        self.type, self.dim, self.concat_dim, self.dev_dim, self.count = t, a, b, k, c

    @property
    def name(self):
        return _NAMES[self.type]

    def __repr__(self):
        if self.type == PERMUTE:
            return "AlltoAll(split_dim=%d, concat_dim=%d, dev_dim=%d, n=%d)" % (self.dim, self.concat_dim,
                                                                               self.dev_dim, self.count)
        return "%s(dim=%d, dev_dim=%d, n=%d)" % (self.name, self.dim, self.dev_dim, self.count)


def _flat_map(layout):
    out = []
    for m in layout.tensor_map:
        if isinstance(m, tuple):
            raise NotImplementedError("multi-axis tensor_map entries are redistributed through a full gather")
        out.append(m)
    return out


def infer(src: TensorLayout, dst: TensorLayout, enable_alltoall=None):
    """Operator list turning ``src`` into ``dst``.  Layouts over different device matrices (or with composite map
    entries) fall back to gather-everything-then-slice, which is always valid."""
    if tuple(src.shape) != tuple(dst.shape):
        raise ValueError("redistribution needs equal tensor shapes, got %s and %s" % (src.shape, dst.shape))
    if enable_alltoall is None:
        enable_alltoall = context.get_auto_parallel_context("enable_alltoall")
    composite = any(isinstance(m, tuple) for m in src.tensor_map + dst.tensor_map)
    if src.device_matrix != dst.device_matrix or composite:
        return None
    lib = _host()
    cap = 8 * (len(src.shape) + 2)
    out = (ctypes.c_int32 * (5 * cap))()
    n = lib.msb_redistribution_infer(_i32(src.device_matrix), len(src.device_matrix), _i32(_flat_map(src)),
                                     _i32(_flat_map(dst)), len(src.shape), int(bool(enable_alltoall)), out, cap)
    if n < 0:
        raise RuntimeError("redistribution inference failed (%d) for %s -> %s" % (n, src, dst))
    return [RedistOp(*out[5 * i:5 * i + 5]) for i in range(n)]


def lowered_names(ops):
    """Primitive-name sequence as the reference lowers it (AllGather on dim != 0 needs Split + Concat)."""
    names = []
    for op in ops:
        if op.type == SPLIT:
            names.append("StridedSlice")
        elif op.type == CONCAT:
            names.append("AllGather")
            if op.dim != 0:
                names += ["Split", "Concat"]
        else:
            names.append("AlltoAll")
    return names


def cost(ops, slice_elems):
    flat = []
    for op in ops:
        flat += [op.type, op.dim, op.concat_dim, op.dev_dim, op.count]
    return _host().msb_redistribution_cost(_i32(flat), len(ops), float(slice_elems))


def group_ranks(device_matrix, rank, dev_dims, base_rank=0):
    lib = _host()
    total = int(np.prod(device_matrix))
    out = (ctypes.c_int32 * total)()
    n = lib.msb_group_ranks(_i32(device_matrix), len(device_matrix), int(rank), _i32(dev_dims), len(dev_dims),
                            int(base_rank), out, total)
    if n < 0:
        raise RuntimeError("group computation failed")
    return [out[i] for i in range(n)]


def _coord_along(device_matrix, rank, dev_dim):
    n = len(device_matrix)
    stride = 1
    for a in range(n - dev_dim, n):
        stride *= device_matrix[a]
    return (rank // stride) % device_matrix[n - 1 - dev_dim]


# ------------------------------------------------------------------------------------ real execution
class _SliceFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, dim, idx, count, gname):
        ctx.meta = (dim, idx, count, gname, x.shape[dim])
        step = x.shape[dim] // count
        return x.narrow(dim, idx * step, step).contiguous()

    @staticmethod
    def backward(ctx, dy):
        dim, idx, count, gname, full = ctx.meta
        # gradient of "keep my chunk" is the all-gather of the chunks' gradients along that dim
        g = M._group(gname)
        parts = CF._all_gather(dy.movedim(dim, 0).contiguous(), g)
        return parts.movedim(0, dim).contiguous() if dim else parts, None, None, None, None


def apply(x, src: TensorLayout, dst: TensorLayout, rank=None, base_rank=0):
    """Redistributes this rank's slice ``x`` from ``src`` to ``dst`` (communicating with the needed groups)."""
    if src == dst:
        return x
    rank = context.get_auto_parallel_context("global_rank") if rank is None else rank
    ops = infer(src, dst)
    if ops is None:
        ops = infer(src, TensorLayout(src.device_matrix, [-1] * len(src.shape), src.shape))
        full = _run_ops(x, ops, src.device_matrix, rank, base_rank)
        from .layout import slice_for_rank
        return slice_for_rank(full, dst, rank - base_rank).contiguous()
    return _run_ops(x, ops, src.device_matrix, rank, base_rank)


def _run_ops(x, ops, device_matrix, rank, base_rank):
    local = rank - base_rank
    for op in ops:
        ranks = group_ranks(device_matrix, local, [op.dev_dim], base_rank)
        if op.type == SPLIT:
            idx = _coord_along(device_matrix, local, op.dev_dim)
            gname = M.group_for_ranks(ranks) if M.GlobalComm.INITED else None
            if gname is not None and torch.is_grad_enabled() and x.requires_grad:
                x = _SliceFn.apply(x, op.dim, idx, op.count, gname)
            else:
                step = x.shape[op.dim] // op.count
                x = x.narrow(op.dim, idx * step, step).contiguous()
        elif op.type == CONCAT:
            gname = M.group_for_ranks(ranks)
            if op.dim == 0:
                x = CF.all_gather_autograd(x.contiguous(), gname)
            else:
                y = CF.all_gather_autograd(x.movedim(op.dim, 0).contiguous(), gname)
                x = y.movedim(0, op.dim).contiguous()
        else:
            gname = M.group_for_ranks(ranks)
            x = CF.all_to_all_autograd(x, op.dim, op.concat_dim, gname)
    return x


# ------------------------------------------------------------------------------------ virtual (all ranks, NumPy)
def apply_virtual(slices, src: TensorLayout, dst: TensorLayout):
    """``slices``: {rank: ndarray} for every rank of the device matrix -> {rank: ndarray} in layout ``dst``."""
    ops = infer(src, dst, enable_alltoall=False)
    world = src.num_devices()
    if ops is None:
        from .layout import assemble_full, slice_for_rank
        full = assemble_full(slices, src)
        return {r: np.ascontiguousarray(_np_slice(full, dst, r)) for r in range(dst.num_devices())}
    cur = dict(slices)
    for op in ops:
        nxt = {}
        for r in range(world):
            ranks = group_ranks(src.device_matrix, r, [op.dev_dim])
            if op.type == SPLIT:
                idx = _coord_along(src.device_matrix, r, op.dev_dim)
                nxt[r] = np.split(cur[r], op.count, axis=op.dim)[idx]
            elif op.type == CONCAT:
                nxt[r] = np.concatenate([cur[q] for q in ranks], axis=op.dim)
            else:
                me = ranks.index(r)
                nxt[r] = np.concatenate([np.split(cur[q], op.count, axis=op.dim)[me] for q in ranks],
                                        axis=op.concat_dim)
        cur = nxt
    return cur


def _np_slice(full, layout, rank):
    idx = layout.slice_index(rank)
    sel = []
    for i, d in enumerate(layout.shape):
        step = d // layout.split_count(i)
        sel.append(slice(idx[i] * step, (idx[i] + 1) * step))
    return full[tuple(sel)]
