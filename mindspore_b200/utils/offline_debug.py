"""Offline debugger over dump files: read dumped tensors back, compute their statistics, and check watchpoints
(NaN / Inf, value thresholds, all-zero, ranges, change between iterations) after a run has finished.

The files are those that ``set_dump`` writes: ``<dump dir>/rank_<r>/<net>/<graph id>/<iteration>/<node>.<output|
input>.<slot>.npy``.  ``DbgServices(dump_dir).initialize(net_name)`` indexes them; a watchpoint is a condition id
(``HAS_NAN = 0`` ... ``RANGE = 21``, the numbering of the reference's debugger), the nodes it watches
(``{node name: {"rank_id": [...], "root_graph_id": [...], "is_output": True}}``; a name ending in ``*`` or the name
of a scope watches everything below) and its ``Parameter`` list.  ``check_watchpoints(iteration)`` returns one
``WatchpointHit`` per tensor that meets the condition, with the parameters that triggered marked ``hit`` and their
``actual_value`` filled in.

Parity: mindspore/python/mindspore/offline_debug/dbg_services.py (DbgServices, TensorInfo, TensorData, TensorBaseData,
TensorStatData, WatchpointHit, Parameter), ccsrc/debug/debug_services.cc (condition evaluation).
"""
from __future__ import annotations

import os
import re

import numpy as np

__all__ = ["DbgServices", "TensorInfo", "TensorData", "TensorBaseData", "TensorStatData", "WatchpointHit",
           "Parameter", "get_version"]

(HAS_NAN, HAS_INF, IS_OVERFLOW, MAX_GT, MAX_LT, MIN_GT, MIN_LT, MAX_MIN_GT, MAX_MIN_LT, MEAN_GT, MEAN_LT, SD_GT, SD_LT,
 GENERAL_OVERFLOW, INIT, TOO_LARGE, TOO_SMALL, ALL_ZERO, CHANGE_TOO_LARGE, CHANGE_TOO_SMALL, NOT_CHANGED,
 RANGE) = range(22)

_FILE = re.compile(r"^(?P<node>.+)\.(?P<kind>output|input)\.(?P<slot>\d+)\.npy$")


def get_version():
    from .. import __version__
    return __version__


class Parameter:
    def __init__(self, name, disabled, value, hit=False, actual_value=0.0):
        if not isinstance(name, str):
            raise TypeError("name must be a string")
        self.name, self.disabled, self.value, self.hit, self.actual_value = name, bool(disabled), float(value), \
            bool(hit), float(actual_value)

    def __repr__(self):
        return "Parameter(%s, disabled=%s, value=%g, hit=%s, actual_value=%g)" % (
            self.name, self.disabled, self.value, self.hit, self.actual_value)


class TensorInfo:
    def __init__(self, node_name, slot, iteration, rank_id, root_graph_id, is_output=True):
        for v, n in ((slot, "slot"), (iteration, "iteration"), (rank_id, "rank_id"), (root_graph_id, "root_graph_id")):
            if isinstance(v, bool) or not isinstance(v, int):
                raise TypeError("%s must be an int" % n)
        self.node_name, self.slot, self.iteration = node_name, slot, iteration
        self.rank_id, self.root_graph_id, self.is_output = rank_id, root_graph_id, bool(is_output)


class TensorData:
    def __init__(self, data_ptr, data_size, dtype, shape):
        self.data_ptr, self.data_size, self.dtype, self.shape = data_ptr, data_size, dtype, list(shape)


class TensorBaseData:
    def __init__(self, data_size, dtype, shape):
        self.data_size, self.dtype, self.shape = data_size, dtype, list(shape)

    def __str__(self):
        return "size in bytes = %d\ndebugger dtype = %s\nshape = %s" % (self.data_size, self.dtype, self.shape)


class TensorStatData:
    def __init__(self, data_size, dtype, shape, is_bool, max_value, min_value, avg_value, count, neg_zero_count,
                 pos_zero_count, nan_count, neg_inf_count, pos_inf_count, zero_count):
        self.data_size, self.dtype, self.shape, self.is_bool = data_size, dtype, list(shape), is_bool
        self.max_value, self.min_value, self.avg_value, self.count = max_value, min_value, avg_value, count
        self.neg_zero_count, self.pos_zero_count, self.zero_count = neg_zero_count, pos_zero_count, zero_count
        self.nan_count, self.neg_inf_count, self.pos_inf_count = nan_count, neg_inf_count, pos_inf_count

    def __str__(self):
        return ("size in bytes = %d\ndebugger dtype = %s\nshape = %s\nis_bool = %s\nmax_value = %s\nmin_value = %s\n"
                "avg_value = %s\ncount = %d\nneg_zero_count = %d\npos_zero_count = %d\nnan_count = %d\n"
                "neg_inf_count = %d\npos_inf_count = %d\nzero_count = %d"
                % (self.data_size, self.dtype, self.shape, self.is_bool, self.max_value, self.min_value,
                   self.avg_value, self.count, self.neg_zero_count, self.pos_zero_count, self.nan_count,
                   self.neg_inf_count, self.pos_inf_count, self.zero_count))


class WatchpointHit:
    def __init__(self, name, slot, condition, watchpoint_id, parameters, error_code, rank_id, root_graph_id):
        self.name, self.slot, self.condition, self.watchpoint_id = name, slot, condition, watchpoint_id
        self.parameters, self.error_code, self.rank_id, self.root_graph_id = parameters, error_code, rank_id, \
            root_graph_id


def _finite(a):
    a = a.astype(np.float64, copy=False).reshape(-1)
    return a[np.isfinite(a)]


class _Check:
    """Evaluates one condition on one tensor; fills ``hit`` / ``actual_value`` on copies of the parameters."""

    def __init__(self, condition, parameters):
        self.condition = condition
        self.params = [Parameter(p.name, p.disabled, p.value) for p in parameters]

    def _cmp(self, name, actual, greater):
        hit = False
        for p in self.params:
            if p.name == name and not p.disabled:
                p.actual_value = float(actual)
                p.hit = bool(actual > p.value) if greater else bool(actual < p.value)
                hit |= p.hit
        return hit

    def _ge(self, name, actual):
        hit = False
        for p in self.params:
            if p.name == name and not p.disabled:
                p.actual_value = float(actual)
                p.hit = bool(actual >= p.value)
                hit |= p.hit
        return hit

    def run(self, cur, prev):
        c = self.condition
        flat = cur.astype(np.float64, copy=False).reshape(-1) if cur.dtype != np.bool_ else \
            cur.reshape(-1).astype(np.float64)
        fin = _finite(flat)
        if c == HAS_NAN:
            return bool(np.isnan(flat).any())
        if c == HAS_INF:
            return bool(np.isinf(flat).any())
        if c in (IS_OVERFLOW, GENERAL_OVERFLOW):
            return bool((~np.isfinite(flat)).any())
        if fin.size == 0:
            return False
        mx, mn, mean = fin.max(), fin.min(), fin.mean()
        simple = {MAX_GT: (mx, True), MAX_LT: (mx, False), MIN_GT: (mn, True), MIN_LT: (mn, False),
                  MAX_MIN_GT: (mx - mn, True), MAX_MIN_LT: (mx - mn, False), MEAN_GT: (mean, True),
                  MEAN_LT: (mean, False), SD_GT: (fin.std(), True), SD_LT: (fin.std(), False)}
        if c in simple:
            actual, greater = simple[c]
            return self._cmp("param", actual, greater)
        zero_pct = 100.0 * float((flat == 0).sum()) / flat.size
        if c == ALL_ZERO:
            return self._ge("zero_percentage_ge", zero_pct)
        if c == INIT:
            return self._ge("zero_percentage_ge", zero_pct) | self._cmp("max_gt", mx, True) | \
                self._cmp("min_lt", mn, False)
        if c == TOO_LARGE:
            return self._cmp("abs_mean_gt", np.abs(fin).mean(), True) | self._cmp("max_gt", mx, True) | \
                self._cmp("min_gt", mn, True) | self._cmp("mean_gt", mean, True)
        if c == TOO_SMALL:
            return self._cmp("abs_mean_lt", np.abs(fin).mean(), False) | self._cmp("max_lt", mx, False) | \
                self._cmp("min_lt", mn, False) | self._cmp("mean_lt", mean, False)
        if c == RANGE:
            lo = next((p.value for p in self.params if p.name == "range_start_inclusive" and not p.disabled), -np.inf)
            hi = next((p.value for p in self.params if p.name == "range_end_inclusive" and not p.disabled), np.inf)
            pct = 100.0 * float(((fin >= lo) & (fin <= hi)).sum()) / flat.size
            return self._cmp("range_percentage_lt", pct, False) | self._cmp("range_percentage_gt", pct, True) | \
                self._cmp("max_min_lt", mx - mn, False) | self._cmp("max_min_gt", mx - mn, True)
        if c in (CHANGE_TOO_LARGE, CHANGE_TOO_SMALL, NOT_CHANGED):
            if prev is None or prev.shape != cur.shape:
                return False
            before = prev.astype(np.float64, copy=False).reshape(-1)
            if c == NOT_CHANGED:
                rtol = next((p.value for p in self.params if p.name == "rtol" and not p.disabled), 1e-5)
                atol = next((p.value for p in self.params if p.name == "atol" and not p.disabled), 1e-8)
                same = bool(np.allclose(flat, before, rtol=rtol, atol=atol, equal_nan=True))
                for p in self.params:
                    p.hit = same and not p.disabled
                return same
            eps = next((p.value for p in self.params if p.name == "epsilon" and not p.disabled), 1e-9)
            ratio = float(np.abs(flat - before).mean() / (np.abs(before).mean() + eps))
            return self._cmp("abs_mean_update_ratio_gt", ratio, True) if c == CHANGE_TOO_LARGE else \
                self._cmp("abs_mean_update_ratio_lt", ratio, False)
        raise ValueError("unknown watch condition %r" % (c,))


class DbgServices:
    def __init__(self, dump_file_path):
        if not isinstance(dump_file_path, str):
            raise TypeError("dump_file_path must be a string")
        self.dump_file_path = dump_file_path
        self.initialized = False
        self._watchpoints = {}
        self._files = {}          # (rank, graph, iteration, node, slot, is_output) -> path

    def initialize(self, net_name, is_sync_mode=True, max_mem_usage=0):
        if not isinstance(net_name, str):
            raise TypeError("net_name must be a string")
        self.net_name, self.is_sync_mode, self.max_mem_usage = net_name, bool(is_sync_mode), max_mem_usage
        self._files.clear()
        if os.path.isdir(self.dump_file_path):
            for rank_dir in sorted(os.listdir(self.dump_file_path)):
                if not rank_dir.startswith("rank_"):
                    continue
                net_dir = os.path.join(self.dump_file_path, rank_dir, net_name)
                if not os.path.isdir(net_dir):
                    continue
                for graph in sorted(os.listdir(net_dir)):
                    for iteration in sorted(os.listdir(os.path.join(net_dir, graph))):
                        it_dir = os.path.join(net_dir, graph, iteration)
                        if not (graph.isdigit() and iteration.isdigit() and os.path.isdir(it_dir)):
                            continue
                        for name in sorted(os.listdir(it_dir)):
                            m = _FILE.match(name)
                            if m:
                                key = (int(rank_dir[5:]), int(graph), int(iteration), m.group("node"),
                                       int(m.group("slot")), m.group("kind") == "output")
                                self._files[key] = os.path.join(it_dir, name)
        self.initialized = True
        return self

    def _need_init(self):
        if not self.initialized:
            raise RuntimeError("DbgServices is not initialized: call initialize(net_name) first")

    # -- watchpoints --
    def add_watchpoint(self, watchpoint_id, watch_condition, check_node_list, parameter_list):
        self._need_init()
        if not isinstance(watchpoint_id, int) or not isinstance(watch_condition, int):
            raise TypeError("watchpoint_id and watch_condition must be ints")
        if not 0 <= watch_condition <= RANGE:
            raise ValueError("watch_condition must be in [0, %d], but got %d" % (RANGE, watch_condition))
        if not isinstance(check_node_list, dict):
            raise TypeError("check_node_list must be a dict")
        for node, spec in check_node_list.items():
            if not isinstance(node, str) or not isinstance(spec, dict):
                raise TypeError("check_node_list maps node names to dicts")
            for key in spec:
                if key not in ("rank_id", "root_graph_id", "is_output"):
                    raise ValueError("unknown key %r in the node specification of %s" % (key, node))
        if not all(isinstance(p, Parameter) for p in parameter_list):
            raise TypeError("parameter_list must hold Parameter objects")
        self._watchpoints[watchpoint_id] = (watch_condition, dict(check_node_list), list(parameter_list))

    def remove_watchpoint(self, watchpoint_id):
        self._need_init()
        if watchpoint_id not in self._watchpoints:
            raise ValueError("there is no watchpoint %r" % (watchpoint_id,))
        del self._watchpoints[watchpoint_id]

    @staticmethod
    def _watches(pattern, node):
        if pattern == "*":
            return True
        if pattern.endswith("*"):
            return node.startswith(pattern[:-1])
        return node == pattern or node.startswith(pattern + "/") or node.startswith(pattern + ".")

    def check_watchpoints(self, iteration, error_on_no_value=False):
        self._need_init()
        hits = []
        for (rank, graph, it, node, slot, is_out), path in sorted(self._files.items()):
            if it != iteration:
                continue
            for wid, (cond, nodes, params) in sorted(self._watchpoints.items()):
                for pattern, spec in nodes.items():
                    if not self._watches(pattern, node) or bool(spec.get("is_output", True)) != is_out:
                        continue
                    if rank not in spec.get("rank_id", [rank]) or graph not in spec.get("root_graph_id", [graph]):
                        continue
                    cur = np.load(path)
                    prev_path = self._files.get((rank, graph, it - 1, node, slot, is_out))
                    prev = np.load(prev_path) if prev_path else None
                    check = _Check(cond, params)
                    if check.run(cur, prev):
                        hits.append(WatchpointHit(node, slot, cond, wid, check.params, 0, rank, graph))
                    elif error_on_no_value and prev is None and cond in (CHANGE_TOO_LARGE, CHANGE_TOO_SMALL,
                                                                         NOT_CHANGED):
                        hits.append(WatchpointHit(node, slot, cond, wid, check.params, 4, rank, graph))
                    break
        return hits

    def check_watchpoint_progress(self):
        return 100 if self.initialized else 0

    # -- tensors --
    def _load(self, info):
        if not isinstance(info, TensorInfo):
            raise TypeError("info must hold TensorInfo objects")
        path = self._files.get((info.rank_id, info.root_graph_id, info.iteration, info.node_name, info.slot,
                                info.is_output))
        return np.load(path) if path else None

    def read_tensors(self, info):
        self._need_init()
        out = []
        for i in info:
            a = self._load(i)
            if a is None:
                out.append(TensorData(b"", 0, 0, []))
            else:
                out.append(TensorData(a.tobytes(), a.nbytes, str(a.dtype), a.shape))
        return out

    def read_tensor_base(self, info):
        self._need_init()
        out = []
        for i in info:
            a = self._load(i)
            out.append(TensorBaseData(0, 0, []) if a is None else TensorBaseData(a.nbytes, str(a.dtype), a.shape))
        return out

    def read_tensor_stats(self, info):
        self._need_init()
        out = []
        for i in info:
            a = self._load(i)
            if a is None:
                out.append(TensorStatData(0, 0, [], False, 0.0, 0.0, 0.0, 0, 0, 0, 0, 0, 0, 0))
                continue
            flat = a.reshape(-1).astype(np.float64)
            fin = flat[np.isfinite(flat)]
            out.append(TensorStatData(
                a.nbytes, str(a.dtype), a.shape, a.dtype == np.bool_,
                float(fin.max()) if fin.size else 0.0, float(fin.min()) if fin.size else 0.0,
                float(fin.mean()) if fin.size else 0.0, int(flat.size), int((fin < 0).sum()), int((fin > 0).sum()),
                int(np.isnan(flat).sum()), int(np.isneginf(flat).sum()), int(np.isposinf(flat).sum()),
                int((flat == 0).sum())))
        return out


import sys as _sys  # noqa: E402

dbg_services = _sys.modules[__name__]          # `from ...offline_debug import dbg_services` names this module
