"""Cell / function level ``shard``: input and output layouts (and a parameter plan) are given for a whole callable;
the primitives inside pick their strategies up by propagation.

``shard(fn, in_strategy, out_strategy, parameter_plan)`` returns a callable that, under ``semi_auto_parallel`` /
``auto_parallel``:

1. slices the parameters named in ``parameter_plan`` (``{"path.to.weight": (rows, cols) | Layout}``) once, exactly
   like a primitive's strategy would;
2. puts every tensor argument into the layout its ``in_strategy`` entry asks for (an un-tagged argument is the
   full tensor on every rank and is cut; an argument that already carries a layout is redistributed; ``None``
   leaves the argument alone);
3. runs ``fn``: primitives that carry no strategy of their own follow the layouts of their inputs through their
   OperatorInfo (sharding propagation at execution time - the forward communication and the redistribution between
   two primitives that disagree are inserted by the dispatcher as for annotated primitives);
4. redistributes the results to ``out_strategy`` when one is given; otherwise they keep the propagated layouts.
   ``parallel.spmd.to_full`` gathers a result.

A strategy entry is a tuple of split counts (one per tensor dim) or a ``Layout`` with a tensor map.  ``device`` and
``level`` are accepted for API compatibility (there is one device kind here and propagation needs no search level).

Parity: mindspore/python/mindspore/parallel/shard.py:129-345 (Shard, shard), ccsrc/frontend/parallel/shard/shard.cc.
"""
from __future__ import annotations

import torch

from .. import context
from .layout import Layout, TensorLayout


def _to_layout(entry, shape, stage_devices):
    if entry is None:
        return None
    if isinstance(entry, Layout):
        if entry.tensor_map is None:
            raise ValueError("For 'Shard', a Layout entry needs its tensor map: layout(\"axis\", ...)")
        if len(entry.tensor_map) != len(shape):
            raise ValueError("For 'Shard', layout %s does not match a tensor of rank %d" % (entry.tensor_map, len(shape)))
        return TensorLayout(entry.device_matrix, entry.tensor_map, shape)
    if len(entry) != len(shape):
        raise ValueError("For 'Shard', strategy %s does not match a tensor of rank %d" % (entry, len(shape)))
    return TensorLayout.from_strategy(entry, shape, stage_devices)


class Shard:
    def __call__(self, fn, in_strategy, out_strategy=None, parameter_plan=None, device="Ascend", level=0):
        mode = context.get_auto_parallel_context("parallel_mode")
        if mode not in ("auto_parallel", "semi_auto_parallel"):
            raise AssertionError("Cell shard only supports auto parallel and semi auto parallel.")
        if not isinstance(in_strategy, tuple):
            raise TypeError("For 'Shard', the 'in_strategy' should be a tuple, but got %s" % type(in_strategy).__name__)
        if out_strategy is not None and not isinstance(out_strategy, tuple):
            raise TypeError("For 'Shard', the 'out_strategy' should be None or tuple, but got %s"
                            % type(out_strategy).__name__)
        for s in in_strategy:
            if s is not None and not isinstance(s, (tuple, Layout)):
                raise TypeError("For 'Shard', every element of 'in_strategy' must be tuple(int), Layout or None")
        if parameter_plan is not None:
            if not isinstance(parameter_plan, dict):
                raise TypeError("For 'Shard', the 'parameter_plan' should be a dict or None")
            for k, v in parameter_plan.items():
                if not isinstance(k, str) or not isinstance(v, (tuple, Layout)):
                    raise TypeError("For 'Shard', 'parameter_plan' maps str -> tuple/Layout")
        if not isinstance(level, int) or level not in (0, 1, 2):
            raise ValueError("For 'Shard', 'level' should be 0, 1 or 2")
        state = {"params_done": False}

        def plan_parameters():
            if state["params_done"] or not parameter_plan:
                state["params_done"] = True
                return
            from . import spmd
            named = {}
            if hasattr(fn, "parameters_and_names"):
                for name, p in fn.parameters_and_names():
                    named[name] = p
                    named.setdefault(p.name, p)
            for key, entry in parameter_plan.items():
                p = named.get(key)
                if p is None:
                    p = next((v for k, v in named.items() if k.endswith("." + key)), None)
                if p is None:
                    raise ValueError("For 'Shard', parameter_plan names %r, which %s does not have"
                                     % (key, type(fn).__name__))
                if p.param_layout is not None:
                    continue
                lay = _to_layout(entry, tuple(p.shape), spmd.stage_devices())
                p.init_data(lay, set_sliced=True)
                spmd.parameter_layouts[p.name] = lay
                spmd.set_layout(p, lay)
                if any(m != -1 for m in lay.tensor_map):
                    p.tp_sharded = True
            state["params_done"] = True

        def wrapped(*args, **kwargs):
            from ..common.tensor import as_tensor
            from . import spmd
            if not spmd.active():
                return fn(*args, **kwargs)
            plan_parameters()
            args = list(args)
            ti = 0
            for i, a in enumerate(args):
                if not isinstance(a, torch.Tensor):
                    continue
                entry = in_strategy[ti] if ti < len(in_strategy) else None
                ti += 1
                if entry is None:
                    continue
                lay = _to_layout(entry, spmd.full_shape(a), spmd.stage_devices())
                args[i] = spmd._prepare_input(a, lay)
            out = fn(*args, **kwargs)
            if out_strategy is None:
                return out
            outs = list(out) if isinstance(out, (tuple, list)) else [out]
            for i, o in enumerate(outs):
                if i >= len(out_strategy) or out_strategy[i] is None or not isinstance(o, torch.Tensor):
                    continue
                cur = spmd.get_layout(o)
                want = _to_layout(out_strategy[i], spmd.full_shape(o), spmd.stage_devices())
                if cur is None:
                    outs[i] = spmd._prepare_input(o, want)
                else:
                    outs[i] = spmd.set_layout(as_tensor(spmd._redistribute(o, cur, want)), want)
            return type(out)(outs) if isinstance(out, (tuple, list)) else outs[0]

        wrapped.in_strategy, wrapped.out_strategy, wrapped.parameter_plan = in_strategy, out_strategy, parameter_plan
        wrapped.shard_fn = fn
        if hasattr(fn, "_in_strategy"):
            fn._in_strategy, fn._out_strategy = in_strategy, out_strategy
            fn._parameter_plan = parameter_plan
        return wrapped


def shard(fn, in_strategy, out_strategy=None, parameter_plan=None, device="Ascend", level=0):
    return Shard()(fn, in_strategy, out_strategy, parameter_plan, device, level)
