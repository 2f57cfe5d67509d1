"""Communication-fusion bucket planning.

Gradients (data-parallel AllReduce), optimizer-shard AllGathers and ReduceScatters are grouped into buckets
that travel as one flat buffer.  Policies follow ``set_auto_parallel_context``:

* ``all_reduce_fusion_config=[i0, i1, ...]`` / ``comm_fusion={"allreduce": {"mode": "index", "config": [...]}}``
  - split points as parameter indices;
* ``comm_fusion={"allreduce": {"mode": "size", "config": MB}}`` - close a bucket when it reaches the size;
* ``mode: "auto"`` - 64 MB threshold (the reference default, parallel_context.h:61);
* ``Parameter.comm_fusion`` / ``Cell.set_comm_fusion`` ids: parameters with the same id > 1 share a bucket.

Buckets are listed in *reverse* parameter order, because backward produces the last layers' gradients
first (reference: frontend/parallel/allreduce_fusion/allreduce_fusion.cc:82-176 walks forward order so that
backward fills buckets from the end).
"""
from __future__ import annotations

from .. import context

DEFAULT_THRESHOLD_MB = 64


def _policy(kind):
    cf = context.get_auto_parallel_context("comm_fusion") or {}
    if cf.get("openstate", True) is False:
        return ("none", None)
    if kind in cf:
        c = cf[kind]
        mode = c.get("mode", "auto")
        if mode == "auto":
            return ("size", DEFAULT_THRESHOLD_MB)
        return (mode, c.get("config"))
    if kind == "allreduce":
        idx = context.get_auto_parallel_context("all_reduce_fusion_config")
        if idx:
            return ("index", list(idx))
    return ("size", DEFAULT_THRESHOLD_MB)


def plan_buckets(sizes_bytes, kind="allreduce", fusion_ids=None):
    """Returns a list of buckets, each a list of indices into ``sizes_bytes``, in launch order (last first)."""
    n = len(sizes_bytes)
    mode, cfg = _policy(kind)
    if fusion_ids and any(f > 1 for f in fusion_ids):
        groups = {}
        order = []
        for i in reversed(range(n)):
            f = fusion_ids[i]
            key = ("id", f) if f > 1 else ("solo", i)
            if key not in groups:
                groups[key] = []
                order.append(key)
            groups[key].append(i)
        return [groups[k] for k in order]
    if mode == "none":
        return [[i] for i in reversed(range(n))]
    if mode == "index":
        cuts = sorted(set(int(c) for c in (cfg or []) if 0 < int(c) < n))
        bounds = [0] + cuts + [n]
        fwd = [list(range(bounds[j], bounds[j + 1])) for j in range(len(bounds) - 1) if bounds[j] < bounds[j + 1]]
        return [list(reversed(b)) for b in reversed(fwd)]
    limit = float(cfg if cfg is not None else DEFAULT_THRESHOLD_MB) * 1024 * 1024
    buckets, cur, cur_bytes = [], [], 0
    for i in reversed(range(n)):
        cur.append(i)
        cur_bytes += sizes_bytes[i]
        if cur_bytes >= limit:
            buckets.append(cur)
            cur, cur_bytes = [], 0
    if cur:
        buckets.append(cur)
    return buckets


def plan_allreduce_buckets(params):
    elem = 4 if context.get_auto_parallel_context("gradient_fp32_sync") else None
    sizes = [p.numel() * (elem or p.element_size()) for p in params]
    return plan_buckets(sizes, "allreduce", [getattr(p, "comm_fusion", 1) for p in params])
