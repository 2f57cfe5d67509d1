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

__all__ = ["AdaSum", "DimReduce", "GroupLossScaleManager", "AutoBoost", "BoostTrainOneStepCell", "BoostTrainOneStepWithLossScaleCell", "LessBN", "GradientFreeze",
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


class AdaSum(Cell):
    """Gradient combination by adaptive summation over the data-parallel ranks (boost/adasum.py): pairs of
    gradients are merged as ``(1 - a.b / 2|a|^2) a + (1 - a.b / 2|b|^2) b`` up a binary tree, which keeps the update
    size of one rank when gradients agree and adds them when they are orthogonal.  Thin front for the wrap cells of
    ``nn.optim_ext``: ``AdaSum(rank, device_number, group_number, parameter_tuple)(delta_weights, parameters,
    old_parameters)`` returns the merged weight deltas."""

    def __init__(self, rank, device_number, group_number, parameter_tuple):
        super().__init__()
        self.rank, self.device_number, self.group_number = rank, device_number, group_number
        self.parameter_tuple = parameter_tuple

    def construct(self, delta_weights, parameters=None, old_parameters=None):
        from .nn.optim_ext import _adasum_allreduce
        ranks = list(range(self.device_number))
        return tuple(_adasum_allreduce(d, ranks, self.rank) for d in delta_weights)


class DimReduce(Cell):
    """Second-order style update in a reduced gradient subspace (boost/dim_reduce.py): gradients are projected onto
    ``pca_mat`` (n_components x n_params), the step is taken in that subspace with a backtracking line search on the
    loss, and mapped back.  ``construct(loss, old_grad, weight, weight_clone, *inputs)`` returns the loss."""

    def __init__(self, network, optimizer, weight, pca_mat_local, n_components, rho, gamma, alpha, sigma, rank,
                 rank_size):
        super().__init__()
        self.network, self.optimizer, self.weight = network, optimizer, weight
        self.pca = torch.as_tensor(pca_mat_local).float()
        self.n_components, self.rho, self.gamma, self.alpha, self.sigma = n_components, rho, gamma, alpha, sigma
        self.rank, self.rank_size = rank, rank_size

    def construct(self, loss, old_grad, weight, weight_clone, *inputs):
        flat = torch.cat([g.reshape(-1).float() for g in old_grad])
        coeff = self.pca.to(flat.device) @ flat                         # gradient in the reduced basis
        step = self.pca.to(flat.device).t() @ coeff                     # back in parameter space
        lr, base = 1.0, float(loss)
        with torch.no_grad():
            snapshot = [w.detach().clone() for w in weight]
            for _ in range(8):                                          # backtracking line search (rho, sigma)
                off = 0
                for w, s0 in zip(weight, snapshot):
                    n = w.numel()
                    w.copy_(s0 - lr * step[off:off + n].reshape(w.shape).to(w.dtype))
                    off += n
                new = float(self.network(*inputs))
                if new <= base - self.sigma * lr * float(flat @ step):
                    break
                lr *= self.rho
        return loss


class GroupLossScaleManager(Cell):
    """Loss scales per layer group (boost/group_loss_scale_manager.py): ``loss_scale_groups`` lists parameter names
    per group; each group keeps its own dynamic scale, updated from that group's overflow status."""

    def __init__(self, init_loss_scale, loss_scale_groups):
        super().__init__()
        self.init_loss_scale = float(init_loss_scale)
        self.loss_scale_groups = [list(g) for g in loss_scale_groups]
        self.scales = [self.init_loss_scale for _ in self.loss_scale_groups]
        self.scale_factor, self.scale_window = 2.0, 1000
        self._good = [0 for _ in self.loss_scale_groups]

    def get_loss_scale(self):
        return self.init_loss_scale

    def get_loss_scale_status(self, loss_scale_number, init_loss_scale):
        return [init_loss_scale] * loss_scale_number

    def update_loss_scale_status(self, layer, update_ratio=1.0):
        return self.scales[layer] * update_ratio

    def update(self, overflow_by_group):
        """``overflow_by_group[i]`` true: halve group i's scale; ``scale_window`` clean steps: double it."""
        for i, ov in enumerate(overflow_by_group):
            if ov:
                self.scales[i] = max(1.0, self.scales[i] / self.scale_factor)
                self._good[i] = 0
            else:
                self._good[i] += 1
                if self._good[i] >= self.scale_window:
                    self.scales[i] *= self.scale_factor
                    self._good[i] = 0
        return list(self.scales)


def _accumulate(accumulation_step, grad_sum, grad):
    with torch.no_grad():
        grad_sum.as_subclass(torch.Tensor).add_(grad.detach().as_subclass(torch.Tensor).to(grad_sum.dtype)
                                                / float(accumulation_step))
    return True


def _clear(grad_sum, zero=None):
    with torch.no_grad():
        grad_sum.as_subclass(torch.Tensor).zero_()
    return True


class _PerTensor:
    """Applies a function to every tensor of the sequences it is mapped over (what ``HyperMap`` does with the
    reference's MultitypeFuncGraph objects of the same names)."""

    def __init__(self, name, fn):
        self.name, self.fn = name, fn

    def __call__(self, *args):
        return self.fn(*args)

    def register(self, *types):
        return lambda f: f


gradient_accumulation_op = _PerTensor("gradient_accumulation_op", _accumulate)
gradient_clear_op = _PerTensor("gradient_clear_op", _clear)


class CommonHeadLastFN(Cell):
    """Classifier head of the gradient-freezing networks: L2-normalised features times L2-normalised weight rows
    (a cosine classifier), scaled by a learnable-free multiplier.  Parity: boost/base.py (CommonHeadLastFN)."""

    def __init__(self, in_channels, out_channels, weight_init="normal", bias_init="zeros", has_bias=True):
        super().__init__()
        from .common.initializer import initializer
        from .common.parameter import Parameter
        self.weight = Parameter(initializer(weight_init, (out_channels, in_channels), torch.float32), name="weight")
        self.bias = Parameter(initializer(bias_init, (out_channels,), torch.float32), name="bias") if has_bias else None
        self.multiplier = 20.0

    def construct(self, x):
        from .common.tensor import as_tensor
        t = x.as_subclass(torch.Tensor)
        w = self.weight.as_subclass(torch.Tensor)
        out = torch.nn.functional.linear(torch.nn.functional.normalize(t, dim=1),
                                         torch.nn.functional.normalize(w, dim=1)) * self.multiplier
        if self.bias is not None:
            out = out + self.bias.as_subclass(torch.Tensor)
        return as_tensor(out)


__all__ += ["gradient_accumulation_op", "gradient_clear_op", "CommonHeadLastFN"]
