"""Strategy checkpoints: per-operator shard strategies and per-parameter layouts of one compiled network.

File formats follow the reference so that files are interchangeable: protobuf ``ParallelStrategyMap``
(ccsrc/utils/node_strategy.proto) or, for names ending in ``.json``, the JSON form written by
ccsrc/frontend/parallel/strategy_checkpoint/parallel_strategy_checkpoint.cc (Save / SaveGroupInfo).  A layout
entry holds dev_matrix, tensor_map, param_split_shape, indices_offset, field, opt_weight_shard_step and
opt_weight_shard_size; the full shape is not stored and is recovered from a slice shape when needed."""
from __future__ import annotations

import json
import os

from ..utils import proto as pb
from .layout import TensorLayout


class ParamLayoutEntry:
    __slots__ = ("dev_matrix", "tensor_map", "param_split_shape", "indices_offset", "field", "opt_shard_step",
                 "opt_shard_size", "stage")

    def __init__(self, dev_matrix, tensor_map, param_split_shape=(), indices_offset=(), field=0, opt_shard_step=0,
                 opt_shard_size=0, stage=0):
        self.dev_matrix = [int(d) for d in dev_matrix]
        self.tensor_map = [int(d) for d in tensor_map]
        self.param_split_shape = [int(d) for d in param_split_shape]
        self.indices_offset = [int(d) for d in indices_offset]
        self.field, self.opt_shard_step, self.opt_shard_size, self.stage = field, opt_shard_step, opt_shard_size, stage

    @classmethod
    def from_layout(cls, lay: TensorLayout, stage=0):
        tmap = []
        for m in lay.tensor_map:
            if isinstance(m, tuple):
                raise ValueError("strategy files hold one device dim per tensor dim; got %s" % (lay.tensor_map,))
            tmap.append(m)
        return cls(lay.device_matrix, tmap, (), (), 0, lay.opt_shard_step, lay.opt_shard_size, stage)

    def split_counts(self):
        n = len(self.dev_matrix)
        return [1 if m == -1 else self.dev_matrix[n - 1 - m] for m in self.tensor_map]

    def to_layout(self, slice_shape=None, full_shape=None):
        """TensorLayout, with the full shape given or rebuilt from the shape of one saved slice."""
        if full_shape is None:
            full_shape = [s * c for s, c in zip(slice_shape, self.split_counts())]
            if self.opt_shard_size and self.opt_shard_size > 1 and full_shape:
                full_shape[0] *= self.opt_shard_size
        return TensorLayout(self.dev_matrix, self.tensor_map, full_shape, self.opt_shard_size, self.opt_shard_step)

    def as_list(self):
        """The list form the reference's ``build_searched_strategy`` returns."""
        return [self.dev_matrix, self.tensor_map, self.param_split_shape, self.indices_offset, self.field,
                self.opt_shard_step, self.opt_shard_size]

    def __eq__(self, o):
        return isinstance(o, ParamLayoutEntry) and self.as_list() == o.as_list()

    def __repr__(self):
        return "ParamLayoutEntry(%s)" % self.as_list()


class StrategyFile:
    def __init__(self, current_stage=0, strategies=None, layouts=None):
        self.current_stage = current_stage
        self.strategies = strategies or {}     # node name -> (stage, [tuple, ...])
        self.layouts = layouts or {}           # param name -> ParamLayoutEntry

    # ------------------------------------------------------------------ protobuf
    def to_bytes(self):
        out = pb.f_varint(1, self.current_stage)
        for name, (stage, strat) in self.strategies.items():
            strs = pb.f_varint(1, stage)
            for s in strat:
                strs += pb.f_bytes(2, b"".join(pb.f_varint(1, d) for d in s))
            out += pb.f_bytes(2, pb.f_bytes(1, name) + pb.f_bytes(2, strs))
        for name, e in self.layouts.items():
            lay = pb.f_bytes(1, b"".join(pb.f_varint(1, d) for d in e.dev_matrix))
            lay += pb.f_bytes(2, b"".join(pb.f_varint(1, d) for d in e.tensor_map))
            lay += pb.f_bytes(3, b"".join(pb.f_varint(1, d) for d in e.param_split_shape))
            lay += pb.f_bytes(4, b"".join(pb.f_varint(1, d) for d in e.indices_offset))
            lay += pb.f_varint(5, e.field) + pb.f_varint(6, e.opt_shard_step) + pb.f_varint(7, e.opt_shard_size)
            out += pb.f_bytes(3, pb.f_bytes(1, name) + pb.f_bytes(2, lay))
        return out

    @classmethod
    def from_bytes(cls, buf):
        sf = cls()
        for f, _wt, v in pb.parse(buf):
            if f == 1:
                sf.current_stage = v
            elif f == 2:
                item = pb.parse(v)
                name = next(x for ff, _, x in item if ff == 1).decode()
                strs = pb.parse(next(x for ff, _, x in item if ff == 2))
                stage = next((x for ff, _, x in strs if ff == 1), 0)
                strat = [tuple(pb.repeated_ints(pb.parse(x), 1)) for ff, _, x in strs if ff == 2]
                sf.strategies[name] = (stage, strat)
            elif f == 3:
                item = pb.parse(v)
                name = next(x for ff, _, x in item if ff == 1).decode()
                lay = pb.parse(next(x for ff, _, x in item if ff == 2))

                def rep(field, sign=False):
                    vals = []
                    for ff, _, x in lay:
                        if ff == field:
                            vals += pb.repeated_ints(pb.parse(x), 1)
                    return [pb.signed(d) if sign else d for d in vals]

                scalar = lambda field: pb.signed(next((x for ff, _, x in lay if ff == field), 0))
                sf.layouts[name] = ParamLayoutEntry(rep(1), rep(2, True), rep(3, True), rep(4, True), scalar(5),
                                                    scalar(6), scalar(7), sf.current_stage)
        return sf

    # ------------------------------------------------------------------ json
    def to_json(self):
        return {
            "current_stage": self.current_stage,
            "parallel_strategy_item": {n: {"stage": st, "parallel_strategy": [list(s) for s in strat]}
                                       for n, (st, strat) in self.strategies.items()},
            "parallel_layout_item": {n: {"dev_matrix": e.dev_matrix, "tensor_map": e.tensor_map,
                                         "param_split_shape": e.param_split_shape,
                                         "indices_offset": e.indices_offset, "field": e.field,
                                         "opt_weight_shard_step": e.opt_shard_step,
                                         "opt_weight_shard_size": e.opt_shard_size}
                                     for n, e in self.layouts.items()},
        }

    @classmethod
    def from_json(cls, d):
        sf = cls(d.get("current_stage", 0))
        for n, it in d.get("parallel_strategy_item", {}).items():
            sf.strategies[n] = (it.get("stage", 0), [tuple(s) for s in it.get("parallel_strategy", [])])
        for n, it in d.get("parallel_layout_item", {}).items():
            sf.layouts[n] = ParamLayoutEntry(it["dev_matrix"], it["tensor_map"], it.get("param_split_shape", ()),
                                             it.get("indices_offset", ()), it.get("field", 0),
                                             it.get("opt_weight_shard_step", 0), it.get("opt_weight_shard_size", 0),
                                             sf.current_stage)
        return sf

    # ------------------------------------------------------------------ files
    def save(self, path):
        os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
        if path.endswith(".json"):
            with open(path, "w") as f:
                json.dump(self.to_json(), f)
        else:
            with open(path, "wb") as f:
                f.write(self.to_bytes())
        os.chmod(path, 0o400 | 0o200)

    @classmethod
    def load(cls, path):
        if not os.path.isfile(path):
            raise ValueError("strategy file %s does not exist" % path)
        if path.endswith(".json"):
            with open(path) as f:
                return cls.from_json(json.load(f))
        with open(path, "rb") as f:
            return cls.from_bytes(f.read())


def save_strategy_file(path, parameter_layouts, node_strategies=None, stage=0):
    """Writes the layouts recorded while a network ran in (semi-)auto-parallel mode (``spmd.parameter_layouts``)."""
    sf = StrategyFile(stage)
    for name, lay in parameter_layouts.items():
        sf.layouts[name] = ParamLayoutEntry.from_layout(lay, stage)
    for name, strat in (node_strategies or {}).items():
        sf.strategies[name] = (stage, [tuple(s) for s in strat])
    sf.save(path)
    return sf


def build_searched_strategy(strategy_filename):
    """{param name: [dev_matrix, tensor_map, param_split_shape, indices_offset, field, shard_step, shard_size]}
    (train/serialization.py:2211 build_searched_strategy)."""
    return {n: e.as_list() for n, e in StrategyFile.load(strategy_filename).layouts.items()}


def save_group_info(path, group_ranks, restore_rank_list):
    """``ParallelGroupMap``: communication groups of this rank + the ranks whose checkpoints cover the model."""
    out = b""
    for name, ranks in group_ranks.items():
        out += pb.f_bytes(1, pb.f_bytes(1, name) + pb.f_bytes(2, b"".join(pb.f_varint(1, r) for r in ranks)))
    out += pb.f_bytes(2, b"".join(pb.f_varint(1, r) for r in restore_rank_list))
    os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
    with open(path, "wb") as f:
        f.write(out)


def restore_group_info_list(group_info_file_name):
    """Ranks listed as ``ckpt_restore_rank_list`` (train/serialization.py restore_group_info_list)."""
    if not os.path.isfile(group_info_file_name):
        raise ValueError("group info file %s does not exist" % group_info_file_name)
    with open(group_info_file_name, "rb") as f:
        fields = pb.parse(f.read())
    ranks = []
    for f_, _wt, v in fields:
        if f_ == 2:
            ranks += pb.repeated_ints(pb.parse(v), 1)
    return ranks
