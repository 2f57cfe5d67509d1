"""Tensor layouts over a device matrix.

A layout is (device_matrix, tensor_map, tensor_shape).  ``tensor_map[i] = k`` means tensor dim *i* is split
along the device-matrix dim counted *from the right* (``device_matrix[-k-1]``); ``-1`` means not split; a tuple
of indices splits one tensor dim over several device dims (major first).  Ranks map to device-matrix
coordinates row-major, last dim fastest.

The heavy algebra (rank lists of groups, redistribution operator inference) lives in the native library
(``csrc/host/layout.cpp``); this module is the Python face plus the user-facing ``Layout`` class.

Parity: mindspore/python/mindspore/parallel/shard.py:23-128 (Layout), parallel/_tensor.py:28-232
(slice arithmetic), ccsrc/frontend/parallel/device_matrix.cc:58-190, tensor_layout/tensor_layout.cc.
"""
from __future__ import annotations

import itertools

import numpy as np
import torch


class Layout:
    """``Layout((dp, mp), ("dp", "mp"))("dp", "None")`` - names device axes and maps tensor dims onto them."""

    def __init__(self, device_matrix, alias_name):
        if not isinstance(device_matrix, tuple):
            raise TypeError("device_matrix must be tuple type, but got %s" % type(device_matrix))
        if not isinstance(alias_name, tuple):
            raise TypeError("alias_name must be tuple type, but got %s" % type(alias_name))
        if len(device_matrix) != len(alias_name):
            raise ValueError("device_matrix length %d != alias_name length %d" % (len(device_matrix), len(alias_name)))
        for d in device_matrix:
            if not isinstance(d, int) or isinstance(d, bool):
                raise TypeError("The element of device_matrix must be int type, but got %s" % type(d))
        for a in alias_name:
            if not isinstance(a, str):
                raise TypeError("The element of alias_name must be str type, but got %s" % type(a))
            if not a:
                raise ValueError("The element of alias_name can not be empty.")
            if a == "None":
                raise ValueError("The alias name can not be set 'None', because 'None' means no sharding.")
        if len(set(alias_name)) != len(alias_name):
            raise ValueError("Each element of alias_name %s should be different" % (alias_name,))
        interleaved = [a for a in alias_name if a == "interleaved_parallel"]
        if interleaved and alias_name.index("interleaved_parallel") != len(alias_name) - 1:
            raise ValueError("When alias_name %s contains keyword 'interleaved_parallel', it should be at the last "
                             "dim of alias_name, which means the virtual sharding." % (alias_name,))
        self._device_shape = device_matrix
        self._alias_name = alias_name
        self._tensor_map = None

    def __call__(self, *tensor_map):
        new = Layout(self._device_shape, self._alias_name)
        tm, used = [], set()
        for ele in tensor_map:
            if isinstance(ele, tuple):
                sub = []
                for e in ele:
                    if e == "None":
                        sub.append(-1)
                        continue
                    if e not in self._alias_name:
                        raise ValueError("The axis %r is not found in %s" % (e, self._alias_name))
                    if e in used:
                        raise ValueError("The axis %r has been set more than one in %s" % (e, self._alias_name))
                    used.add(e)
                    sub.append(len(self._alias_name) - 1 - self._alias_name.index(e))
                tm.append(tuple(sub))
                continue
            if ele == "None":
                tm.append(-1)
                continue
            if ele not in self._alias_name:
                raise ValueError("The axis %r is not found in %s" % (ele, self._alias_name))
            if ele in used:
                raise ValueError("The axis %r has been set more than one in %s" % (ele, self._alias_name))
            used.add(ele)
            tm.append(len(self._alias_name) - 1 - self._alias_name.index(ele))
        new._tensor_map = tuple(tm)
        return new

    def to_dict(self):
        if self._tensor_map is None:
            raise ValueError("The tensor_map of layout is None")
        return {"device_matrix": self._device_shape, "tensor_map": self._tensor_map,
                "interleaved_parallel": "interleaved_parallel" in self._alias_name, "alias_name": self._alias_name}

    @property
    def device_matrix(self):
        return self._device_shape

    @property
    def tensor_map(self):
        return self._tensor_map


class TensorLayout:
    """Concrete layout of one tensor: device matrix, tensor map (ints, -1, or tuples), full shape."""

    __slots__ = ("device_matrix", "tensor_map", "shape", "opt_shard_size", "opt_shard_step")

    def __init__(self, device_matrix, tensor_map, shape, opt_shard_size=0, opt_shard_step=0):
        self.device_matrix = tuple(int(d) for d in device_matrix)
        self.tensor_map = tuple(tuple(m) if isinstance(m, (tuple, list)) else int(m) for m in tensor_map)
        self.shape = tuple(int(s) for s in shape)
        self.opt_shard_size = opt_shard_size   # extra dim-0 split over replicas (parallel optimizer)
        self.opt_shard_step = opt_shard_step
        if len(self.tensor_map) != len(self.shape):
            raise ValueError("tensor_map %s and shape %s differ in rank" % (self.tensor_map, self.shape))
        n = len(self.device_matrix)
        used = set()
        for i, m in enumerate(self.tensor_map):
            for k in (m if isinstance(m, tuple) else (m,)):
                if k == -1:
                    continue
                if k < 0 or k >= n:
                    raise ValueError("tensor_map entry %d out of range for device matrix %s" % (k, self.device_matrix))
                if k in used:
                    raise ValueError("device dim %d used twice in tensor_map %s" % (k, self.tensor_map))
                used.add(k)
            if self.shape[i] % self.split_count(i):
                raise ValueError("tensor dim %d of size %d is not divisible by its split count %d"
                                 % (i, self.shape[i], self.split_count(i)))

    @classmethod
    def from_strategy(cls, strategy, shape, stage_devices=None):
        """Layout of one input whose split counts are ``strategy``; the device matrix is the strategy itself
        (plus a leading replica dim when it does not use all ``stage_devices``)."""
        dm = [int(s) for s in strategy]
        prod = int(np.prod(dm)) if dm else 1
        lead = []
        if stage_devices and stage_devices > prod:
            if stage_devices % prod:
                raise ValueError("strategy %s does not divide the %d devices of the stage" % (strategy, stage_devices))
            lead = [stage_devices // prod]
        full = lead + dm
        n = len(full)
        tmap = [(n - 1 - (len(lead) + i)) if s > 1 else -1 for i, s in enumerate(dm)]
        return cls(full, tmap, shape)

    def dev_dim_size(self, k):
        return self.device_matrix[len(self.device_matrix) - 1 - k]

    def split_count(self, i):
        m = self.tensor_map[i]
        c = 1
        for k in (m if isinstance(m, tuple) else (m,)):
            if k != -1:
                c *= self.dev_dim_size(k)
        return c

    def tensor_strategy(self):
        return tuple(self.split_count(i) for i in range(len(self.shape)))

    def slice_shape(self):
        s = [d // self.split_count(i) for i, d in enumerate(self.shape)]
        if self.opt_shard_size and self.opt_shard_size > 1 and s:
            s[0] //= self.opt_shard_size
        return tuple(s)

    def num_devices(self):
        return int(np.prod(self.device_matrix)) if self.device_matrix else 1

    def coord(self, rank):
        rank %= self.num_devices()
        out = []
        for d in reversed(self.device_matrix):
            out.append(rank % d)
            rank //= d
        return tuple(reversed(out))

    def slice_index(self, rank):
        """Index of this rank's chunk along every tensor dim."""
        c = self.coord(rank)
        n = len(self.device_matrix)
        idx = []
        for m in self.tensor_map:
            i = 0
            for k in (m if isinstance(m, tuple) else (m,)):
                if k == -1:
                    continue
                i = i * self.dev_dim_size(k) + c[n - 1 - k]
            idx.append(i)
        return tuple(idx)

    def unused_dev_dims(self):
        used = set()
        for m in self.tensor_map:
            for k in (m if isinstance(m, tuple) else (m,)):
                if k != -1:
                    used.add(k)
        return [k for k in range(len(self.device_matrix)) if k not in used and self.dev_dim_size(k) > 1]

    def replica_group(self, rank, base_rank=0):
        """Ranks holding the identical slice: those that differ only along unused device dims."""
        return ranks_along_dims(self.device_matrix, rank - base_rank, self.unused_dev_dims(), base_rank)

    def repeat_num(self):
        r = 1
        for k in self.unused_dev_dims():
            r *= self.dev_dim_size(k)
        return r

    def to_dict(self):
        return {"device_matrix": list(self.device_matrix), "tensor_map": [list(m) if isinstance(m, tuple) else m
                                                                         for m in self.tensor_map],
                "shape": list(self.shape), "opt_shard_size": self.opt_shard_size, "opt_shard_step": self.opt_shard_step}

    @classmethod
    def from_dict(cls, d):
        return cls(d["device_matrix"], d["tensor_map"], d["shape"], d.get("opt_shard_size", 0),
                   d.get("opt_shard_step", 0))

    def __eq__(self, o):
        return isinstance(o, TensorLayout) and (self.device_matrix, self.tensor_map, self.shape, self.opt_shard_size) \
            == (o.device_matrix, o.tensor_map, o.shape, o.opt_shard_size)

    def __hash__(self):
        return hash((self.device_matrix, self.tensor_map, self.shape))

    def __repr__(self):
        return "TensorLayout(dev=%s, map=%s, shape=%s%s)" % (self.device_matrix, self.tensor_map, self.shape,
                                                            ", opt_shard=%d" % self.opt_shard_size if self.opt_shard_size else "")


def ranks_along_dims(device_matrix, rank, dev_dims, base_rank=0):
    """All ranks whose coordinates equal ``rank``'s except along the device dims ``dev_dims`` (indices from the
    right).  Sorted ascending; offsets by ``base_rank`` (first rank of the pipeline stage)."""
    n = len(device_matrix)
    coord = []
    r = rank
    for d in reversed(device_matrix):
        coord.append(r % d)
        r //= d
    coord = list(reversed(coord))
    axes = [n - 1 - k for k in dev_dims]
    ranges = [range(device_matrix[a]) if a in axes else [coord[a]] for a in range(n)]
    out = []
    for c in itertools.product(*ranges):
        v = 0
        for a in range(n):
            v = v * device_matrix[a] + c[a]
        out.append(v + base_rank)
    return sorted(out)


def slice_for_rank(tensor, layout, rank):
    """This rank's slice of a full tensor (view, no copy)."""
    idx = layout.slice_index(rank)
    sl = []
    for i, d in enumerate(layout.shape):
        n = layout.split_count(i)
        step = d // n
        sl.append(slice(idx[i] * step, (idx[i] + 1) * step))
    out = tensor[tuple(sl)]
    if layout.opt_shard_size and layout.opt_shard_size > 1:
        group = layout.replica_group(rank)
        pos = group.index(rank % layout.num_devices()) % layout.opt_shard_size
        step = out.shape[0] // layout.opt_shard_size
        out = out[pos * step:(pos + 1) * step]
    return out


def assemble_full(slices_by_rank, layout):
    """Inverse of ``slice_for_rank`` for layouts without optimizer sharding: rebuilds the full numpy array."""
    first = next(iter(slices_by_rank.values()))
    full = np.zeros(layout.shape, dtype=first.dtype)
    for rank, sl in slices_by_rank.items():
        idx = layout.slice_index(rank)
        sel = []
        for i, d in enumerate(layout.shape):
            step = d // layout.split_count(i)
            sel.append(slice(idx[i] * step, (idx[i] + 1) * step))
        full[tuple(sel)] = sl
    return full
