"""Cost model of the strategy search and its context (``set_cost_model_context``).

A candidate strategy of an operator costs

    alpha * computation  +  beta * communication                      (reference: auto_parallel/costmodel.h)

* computation  - bytes a rank reads and writes for the operator on its slices (the operators are memory- or
  tensor-core bound on slices of equal FLOPs per byte, so slice bytes rank candidates the way time does; a MatMul
  adds its FLOPs divided by the machine balance);
* communication - bytes of the forward collective (AllReduce counts twice: reduce-scatter + all-gather) plus what
  its backward mirror moves (the gradient all-reduce of every replicated parameter), passed through the
  reference's small-message correction: below ``costmodel_communi_threshold`` bytes a transfer costs
  ``costmodel_communi_const``, above it ``bytes + costmodel_communi_bias``;
* memory        - parameter slice + outputs kept for backward; the search must keep the sum over operators within
  ``device_memory_capacity``: ``fit_memory`` re-runs a search with a growing price on memory until it does
  (the reference carries (memory, cost) lists through its eliminations: dp_algo_costmodel.cc).

``fully_use_devices`` (algo parameter) drops candidates that leave devices idle.
Parity: ccsrc/frontend/parallel/auto_parallel/operator_costmodel.cc, costmodel_context.h:29-48,
python/mindspore/parallel/_cost_model_context.py:533-640, algo_parameter_config.py.
"""
from __future__ import annotations

_DEFAULTS = {
    "device_memory_capacity": 180.0 * 1024 ** 3,      # one B200
    "costmodel_alpha": 1.0,
    "costmodel_beta": 8.7,            # HBM bytes per NVLink byte: measured 6.55 TB/s copy rate / 0.75 TB/s link rate
    "costmodel_gamma": 0.001,
    "costmodel_communi_threshold": 2048.0,
    "costmodel_communi_const": 3072.0,
    "costmodel_communi_bias": 1024.0,
    "run_phase": 0,
    "multi_subgraphs": False,
    "costmodel_allreduce_fusion_algorithm": 0,
    "costmodel_allreduce_fusion_times": 0,
    "costmodel_allreduce_fusion_tail_percent": 0.1,
    "costmodel_allreduce_fusion_tail_time": 0.1,
    "costmodel_allreduce_fusion_allreduce_inherent_time": 0.1,
    "costmodel_allreduce_fusion_allreduce_bandwidth": 0.1,
    "costmodel_allreduce_fusion_computation_time_parameter": 0.1,
}
_ctx = dict(_DEFAULTS)
MACHINE_BALANCE = 210.0      # bf16 FLOPs per HBM byte at the measured rates (1.38 PFLOP/s sustained / 6.55 TB/s)


def set_cost_model_context(**kwargs):
    for k, v in kwargs.items():
        if k not in _DEFAULTS:
            raise ValueError("Set context keyword %s is not recognized!" % k)
        want = type(_DEFAULTS[k])
        if want is float and isinstance(v, int) and not isinstance(v, bool):
            v = float(v)
        if not isinstance(v, want):
            raise TypeError("For 'set_cost_model_context', '%s' must be %s, but got %s" % (k, want.__name__,
                                                                                           type(v).__name__))
        if k == "device_memory_capacity" and v <= 0:
            raise ValueError("device_memory_capacity must be positive")
        if k == "run_phase" and v not in (0, 1):
            raise ValueError("run_phase must be 0 (training) or 1 (inference)")
        _ctx[k] = v


def get_cost_model_context(attr_key):
    if attr_key not in _ctx:
        raise ValueError("Get context keyword %s is not recognized!" % attr_key)
    return _ctx[attr_key]


def reset_cost_model_context():
    _ctx.clear()
    _ctx.update(_DEFAULTS)


def comm_bytes_cost(nbytes):
    if nbytes <= 0:
        return 0.0
    if nbytes < _ctx["costmodel_communi_threshold"]:
        return _ctx["costmodel_communi_const"]
    return nbytes + _ctx["costmodel_communi_bias"]


def _numel(shape):
    n = 1
    for d in shape:
        n *= int(d)
    return n


def candidate_cost(prim, info, param_inputs=(), elem_bytes=2):
    """(cost, memory bytes) of one strategy.  ``param_inputs``: indices of inputs that are Parameters."""
    ins, outs = info.input_layouts(), info.output_layouts()
    in_b = [_numel(l.slice_shape()) * elem_bytes for l in ins]
    out_b = [_numel(l.slice_shape()) * elem_bytes for l in outs]
    comp = float(sum(in_b) + sum(out_b))
    if prim.name in ("MatMul", "BatchMatMul") and len(ins) == 2:
        a, b = ins[0].slice_shape(), ins[1].slice_shape()
        k = a[-2] if prim.attrs.get("transpose_a") else a[-1]
        flops = 2.0 * _numel(outs[0].slice_shape()) * k
        if info.forward_comm is not None and info.forward_comm[0] == "ReduceScatter":
            flops *= info.dev_matrix[len(info.dev_matrix) - 1 - info.forward_comm[1][0]]   # output shown is already scattered
        comp += flops / MACHINE_BALANCE
    comm = 0.0
    fc = info.forward_comm
    if fc is not None:
        nb = out_b[0]
        comm += comm_bytes_cost(nb * (2.0 if fc[0].startswith("AllReduce") else 1.0))
    training = _ctx["run_phase"] == 0
    mem = float(sum(out_b)) if training else float(max(out_b, default=0))
    for i in param_inputs:
        if i >= len(ins):
            continue
        mem += in_b[i] * (1 + 8 if training else 1)       # bf16 weight + fp32 master, gradient and two moments
        if training and ins[i].repeat_num() > 1:
            comm += comm_bytes_cost(2.0 * in_b[i] * 2)    # mirror: fp32 gradient all-reduce over the replicas
    return _ctx["costmodel_alpha"] * comp + _ctx["costmodel_beta"] * comm, mem
