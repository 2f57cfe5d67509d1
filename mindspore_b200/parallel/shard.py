"""Cell / function level ``shard``: attaches input/output strategies to a callable; the planner spreads them to
the primitives inside by sharding propagation.
Parity: mindspore/python/mindspore/parallel/shard.py:129-345 (Shard, shard)."""
from .. import context
from .layout import Layout


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
        target = fn

        def wrapped(*args, **kwargs):
            return target(*args, **kwargs)

        wrapped.in_strategy, wrapped.out_strategy, wrapped.parameter_plan = in_strategy, out_strategy, parameter_plan
        wrapped.shard_fn = fn
        if hasattr(fn, "_in_strategy"):
            fn._in_strategy, fn._out_strategy = in_strategy, out_strategy
            fn._parameter_plan = parameter_plan
        return wrapped


def shard(fn, in_strategy, out_strategy=None, parameter_plan=None, device="Ascend", level=0):
    return Shard()(fn, in_strategy, out_strategy, parameter_plan, device, level)
