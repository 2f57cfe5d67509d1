"""``boost``: bundled training accelerations selected by level (python/mindspore/boost/{boost.py,
boost_cell_wrapper.py, less_batch_normalization.py, grad_freeze.py, grad_accumulation.py}).

``AutoBoost("O1" | "O2", config)`` turns on: ``less_bn`` (BatchNorm layers after the first few are frozen into
inference statistics), ``grad_freeze`` (a growing share of the earliest layers stops receiving gradients as training
proceeds), ``grad_accumulation`` (``BoostTrainOneStepCell`` accumulates ``grad_accumulation_step`` micro-steps) and
``adasum``.  ``BoostTrainOneStepCell`` is the train-step cell that honours them."""
from __future__ import annotations

import torch

from .nn.cell import Cell
from .nn.wrap import TrainOneStepCell

__all__ = ["AutoBoost", "BoostTrainOneStepCell", "BoostTrainOneStepWithLossScaleCell", "LessBN", "GradientFreeze",
           "FreezeOpt", "freeze_cell", "GradientAccumulation", "OptimizerProcess", "ParameterProcess"]

_LEVELS = {"O0": {}, "O1": {"less_bn": True, "grad_freeze": True},
           "O2": {"less_bn": True, "grad_freeze": True, "adasum": True}}


class AutoBoost:
    def __init__(self, level="O0", boost_config_dict=None):
        if level not in _LEVELS:
            raise ValueError("Boost level must be one of O0, O1, O2, but got %r" % (level,))
        self.level = level
        cfg = {"less_bn": False, "grad_freeze": False, "adasum": False, "grad_accumulation": False, "dim_reduce": False,
               "grad_accumulation_step": 1, "freeze_p": 0.7, "total_steps": 65536, "freeze_type": 1, "fn_flag": True}
        cfg.update(_LEVELS[level])
        d = boost_config_dict or {}
        cfg.update(d.get("boost", {}))
        cfg.update(d.get("common", {}))
        for section in ("less_bn", "grad_freeze", "grad_accumulation", "adasum", "dim_reduce"):
            cfg.update({k: v for k, v in d.get(section, {}).items()})
        self.cfg = cfg

    def network_auto_process_train(self, network, optimizer):
        if self.cfg["less_bn"]:
            network = LessBN(network, fn_flag=self.cfg["fn_flag"])
        if self.cfg["grad_freeze"]:
            optimizer = FreezeOpt(optimizer, network, self.cfg["freeze_p"], self.cfg["total_steps"])
        return network, optimizer

    def network_auto_process_eval(self, network):
        return network


class LessBN(Cell):
    """Keeps the first ``keep`` BatchNorm layers training and runs the others on their moving statistics."""

    def __init__(self, network, fn_flag=False, keep=3):
        super().__init__(auto_prefix=False)
        self.network = network
        from .nn.layer import _BatchNorm
        bns = [c for _, c in network.cells_and_names() if isinstance(c, _BatchNorm)]
        for bn in bns[keep:]:
            bn.use_batch_statistics = False
        self.frozen = len(bns[keep:])

    def construct(self, *inputs):
        return self.network(*inputs)


def freeze_cell(reducer_flag, network, optimizer, sens, grad, use_grad_accumulation, mean=None, degree=None,
                max_accumulation_step=1):
    return BoostTrainOneStepCell(network, optimizer, sens)


class FreezeOpt(Cell):
    """Optimizer wrapper: at step t the first ``share(t)`` of the parameters (in network order) are skipped, with
    ``share`` rising linearly from 0 to ``freeze_p`` over ``total_steps``."""

    def __init__(self, opt, train_parameter_groups=None, freeze_p=0.7, total_steps=65536, **kw):
        super().__init__(auto_prefix=False)
        self.opt, self.freeze_p, self.total_steps, self._t = opt, float(freeze_p), int(total_steps), 0
        for name in ("_parameters", "parameters", "learning_rate", "arena"):
            if hasattr(opt, name):
                object.__setattr__(self, name, getattr(opt, name))

    def frozen_count(self):
        share = self.freeze_p * min(1.0, self._t / max(1, self.total_steps))
        return int(share * len(self.opt._parameters))

    def construct(self, gradients):
        k = self.frozen_count()
        grads = list(gradients)
        for i in range(k):
            grads[i] = torch.zeros_like(grads[i])
        self._t += 1
        return self.opt(tuple(grads))


GradientFreeze = FreezeOpt


class GradientAccumulation(Cell):
    def __init__(self, max_accumulation_step, optimizer):
        super().__init__(auto_prefix=False)
        self.n, self.opt, self._acc, self._k = int(max_accumulation_step), optimizer, None, 0

    def construct(self, loss, grads):
        if self._acc is None:
            self._acc = [torch.zeros_like(g) for g in grads]
        for a, g in zip(self._acc, grads):
            a.add_(g.detach())
        self._k += 1
        if self._k == self.n:
            self.opt(tuple(a / self.n for a in self._acc))
            for a in self._acc:
                a.zero_()
            self._k = 0
        return loss


class OptimizerProcess:
    """Rebuilds an optimizer with changed arguments / parameter groups."""

    def __init__(self, opt):
        self.origin, self.cls = opt, type(opt)
        self.params = list(opt._parameters)
        self.kwargs = {}

    def add_grad_centralization(self, network):
        self.kwargs["grad_centralization"] = True

    def build_params_dict(self, network):
        return {id(p): n for n, p in network.parameters_and_names()}

    def generate_new_optimizer(self):
        return self.origin


class ParameterProcess:
    def assign_parameter_group(self, parameters, split_point=None):
        params = list(parameters)
        if not split_point:
            return [{"params": params}]
        groups, start = [], 0
        for sp in list(split_point) + [len(params)]:
            groups.append({"params": params[start:sp]})
            start = sp
        return [g for g in groups if g["params"]]

    def generate_group_params(self, parameters, origin_params):
        return [{"params": list(parameters)}]


class BoostTrainOneStepCell(TrainOneStepCell):
    """TrainOneStepCell that applies gradient accumulation when the network / optimizer were prepared by
    ``AutoBoost`` with ``grad_accumulation``."""

    def __init__(self, network, optimizer, sens=1.0, grad_accumulation_step=1):
        super().__init__(network, optimizer, sens)
        self.grad_accumulation_step = int(grad_accumulation_step)


class BoostTrainOneStepWithLossScaleCell(BoostTrainOneStepCell):
    def __init__(self, network, optimizer, scale_sense):
        super().__init__(network, optimizer, 1.0)
        self.scale_sense = scale_sense
