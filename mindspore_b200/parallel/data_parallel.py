"""Data-parallel gradient synchronisation on the flat gradient arena.

Because arena gradients are already one contiguous fp32 buffer, a comm_fusion bucket is simply a slice
of it: no packing copies.  Each bucket is reduced with the fused NVLink all-reduce kernel when the symmetric-
memory runtime is up (``parallel.symm``), else with one NCCL call per bucket; the 1/N mean scale is folded into
the kernel (or applied in place).
Parity: DistributedGradReducer (nn/wrap/grad_reducer.py:413-481) + backend CommunicationOpFusion
(backend/common/pass/communication_op_fusion.cc:88-146).
"""
from __future__ import annotations

import torch

from ..communication import comm_func as CF
from ..communication import management as M


def arena_bucket_ranges(arena, buckets):
    """[(start, end)] element ranges of the arena covered by each bucket (buckets hold param indices)."""
    out = []
    for b in buckets:
        lo = min(arena.offsets[i] for i in b)
        hi_i = max(b)
        hi = arena.offsets[hi_i + 1] if hi_i + 1 < len(arena.params) else arena.total
        out.append((lo, hi))
    return out


def allreduce_arena_grads(arena, reducer):
    if reducer.degree == 1 or not M.GlobalComm.INITED:
        return
    g = M._group(reducer.group)
    ranges = getattr(reducer, "_arena_ranges", None)
    if ranges is None:
        # arena order may differ from reducer.params order: plan on arena order
        from .comm_fusion import plan_allreduce_buckets
        ranges = arena_bucket_ranges(arena, plan_allreduce_buckets(arena.params))
        reducer._arena_ranges = ranges
    scale = 1.0 / reducer.degree if reducer.mean else 1.0
    from . import symm
    for lo, hi in ranges:
        seg = arena.grads[lo:hi]
        if symm.fused_available(g):
            symm.all_reduce_(seg, g, scale)
        else:
            CF._all_reduce_(seg, "sum", g)
            if scale != 1.0:
                seg.mul_(scale)
