"""Python face of the native planners: pipeline schedules, static memory plans, strategy search."""
from __future__ import annotations

import ctypes

from .. import _native

_lib = None
I32P = ctypes.POINTER(ctypes.c_int32)
I64P = ctypes.POINTER(ctypes.c_int64)
F64P = ctypes.POINTER(ctypes.c_double)


def _host():
    global _lib
    if _lib is None:
        lib = _native.host()
        lib.msb_pipeline_schedule.restype = ctypes.c_int
        lib.msb_pipeline_schedule.argtypes = [ctypes.c_int] * 5 + [I32P, ctypes.c_int]
        lib.msb_pipeline_peak_activations.restype = ctypes.c_int
        lib.msb_pipeline_peak_activations.argtypes = [I32P, ctypes.c_int]
        lib.msb_memory_plan.restype = ctypes.c_int64
        lib.msb_memory_plan.argtypes = [ctypes.c_int, I64P, I32P, I32P, I32P, ctypes.c_int64, I64P]
        lib.msb_memory_plan_check.restype = ctypes.c_int
        lib.msb_memory_plan_check.argtypes = [ctypes.c_int, I64P, I32P, I32P, I64P]
        lib.msb_chain_dp_search.restype = ctypes.c_double
        lib.msb_chain_dp_search.argtypes = [ctypes.c_int, I32P, F64P, F64P, I32P]
        lib.msb_propagate_strategies.restype = ctypes.c_int
        lib.msb_propagate_strategies.argtypes = [ctypes.c_int, I32P, I32P, ctypes.c_int, I32P, I32P, I64P, F64P, I32P]
        _lib = lib
    return _lib


def _arr(ctype, seq):
    a = (ctype * max(len(seq), 1))()
    for i, v in enumerate(seq):
        a[i] = v
    return a


FORWARD, BACKWARD = 0, 1


def pipeline_schedule(stages, stage, micro, chunks=1, scheduler="1f1b"):
    """[(kind, micro_batch, chunk)] for one stage; kind 0 = forward, 1 = backward."""
    if scheduler not in ("1f1b", "gpipe"):
        raise ValueError("scheduler must be '1f1b' or 'gpipe'")
    cap = 2 * micro * chunks + 4
    out = (ctypes.c_int32 * (3 * cap))()
    n = _host().msb_pipeline_schedule(stages, stage, micro, chunks, 1 if scheduler == "1f1b" else 0, out, cap)
    if n < 0:
        raise ValueError("invalid pipeline configuration: stages=%d stage=%d micro=%d chunks=%d (interleaved "
                         "schedules need micro %% stages == 0)" % (stages, stage, micro, chunks))
    return [(out[3 * i], out[3 * i + 1], out[3 * i + 2]) for i in range(n)]


def pipeline_peak_activations(steps):
    flat = []
    for s in steps:
        flat += list(s)
    return _host().msb_pipeline_peak_activations(_arr(ctypes.c_int32, flat), len(steps))


def memory_plan(sizes, starts, ends, groups=None, align=512):
    """Offsets for tensors with lifetimes [start, end]; returns (offsets, arena_bytes)."""
    n = len(sizes)
    offs = (ctypes.c_int64 * max(n, 1))()
    total = _host().msb_memory_plan(n, _arr(ctypes.c_int64, sizes), _arr(ctypes.c_int32, starts),
                                    _arr(ctypes.c_int32, ends),
                                    _arr(ctypes.c_int32, groups if groups is not None else [-1] * n), align, offs)
    if total < 0:
        raise ValueError("invalid memory plan request")
    return [offs[i] for i in range(n)], total


def memory_plan_conflicts(sizes, starts, ends, offsets):
    n = len(sizes)
    return _host().msb_memory_plan_check(n, _arr(ctypes.c_int64, sizes), _arr(ctypes.c_int32, starts),
                                         _arr(ctypes.c_int32, ends), _arr(ctypes.c_int64, offsets))


def chain_dp_search(op_costs, edge_costs):
    """op_costs: list (per op) of candidate costs; edge_costs[t][a][b]: cost of candidate a -> b between op t, t+1."""
    n = len(op_costs)
    ncand = [len(c) for c in op_costs]
    flat_op = [float(v) for c in op_costs for v in c]
    flat_edge = [float(v) for e in edge_costs for row in e for v in row]
    choice = (ctypes.c_int32 * max(n, 1))()
    total = _host().msb_chain_dp_search(n, _arr(ctypes.c_int32, ncand), _arr(ctypes.c_double, flat_op),
                                        _arr(ctypes.c_double, flat_edge), choice)
    return [choice[i] for i in range(n)], total


def propagate_strategies(n_cand, fixed, edges, edge_costs):
    """edges: [(src, dst)]; edge_costs[e]: matrix [n_cand[src]][n_cand[dst]].  Returns the chosen candidates."""
    n = len(n_cand)
    offs, flat = [], []
    for m in edge_costs:
        offs.append(len(flat))
        for row in m:
            flat += [float(v) for v in row]
    choice = (ctypes.c_int32 * max(n, 1))()
    rc = _host().msb_propagate_strategies(n, _arr(ctypes.c_int32, n_cand), _arr(ctypes.c_int32, fixed), len(edges),
                                          _arr(ctypes.c_int32, [e[0] for e in edges]),
                                          _arr(ctypes.c_int32, [e[1] for e in edges]), _arr(ctypes.c_int64, offs),
                                          _arr(ctypes.c_double, flat), choice)
    if rc < 0:
        raise ValueError("invalid propagation request")
    return [choice[i] for i in range(n)]


def elimination_search(n_cand, op_costs, edges, edge_costs, fixed=None, max_table=4_000_000):
    """Exact minimum-cost strategy assignment on a general operator graph by node elimination (native).  Returns
    (choices, cost) or (None, None) when an intermediate table would exceed ``max_table`` entries."""
    n = len(n_cand)
    offs, flat = [], []
    for m in edge_costs:
        offs.append(len(flat))
        for row in m:
            flat += [float(v) for v in row]
    flat_op = [float(v) for c in op_costs for v in c]
    choice = (ctypes.c_int32 * max(n, 1))()
    lib = _host()
    lib.msb_elimination_search.restype = ctypes.c_double
    cost = lib.msb_elimination_search(
        n, _arr(ctypes.c_int32, n_cand), _arr(ctypes.c_double, flat_op), len(edges),
        _arr(ctypes.c_int32, [e[0] for e in edges]), _arr(ctypes.c_int32, [e[1] for e in edges]),
        _arr(ctypes.c_int64, offs), _arr(ctypes.c_double, flat),
        _arr(ctypes.c_int32, fixed if fixed is not None else [-1] * n), ctypes.c_longlong(max_table), choice)
    if cost < 0:
        return None, None
    return [choice[i] for i in range(n)], cost
