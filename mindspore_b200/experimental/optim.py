"""``experimental.optim``: optimizers with the ``param_groups`` interface (``Adadelta Adagrad Adam Adamax AdamW ASGD
NAdam RAdam RMSprop Rprop SGD``) and ``lr_scheduler``.  An optimizer is called with the gradients of its parameters
(``optimizer(grads)``), in the order of ``optimizer.parameters``; schedulers change ``param_groups[i]['lr']``.

The update rules are PyTorch's own (this namespace mirrors ``torch.optim`` in the reference too:
python/mindspore/experimental/optim/{optimizer.py, adam.py, ..., lr_scheduler.py})."""
from __future__ import annotations

import types

import torch

from ..nn.cell import Cell

__all__ = ["Optimizer", "Adadelta", "Adagrad", "Adam", "Adamax", "AdamW", "ASGD", "NAdam", "RAdam", "RMSprop", "Rprop",
           "SGD", "lr_scheduler"]


def _plain(t):
    return t.detach().as_subclass(torch.Tensor) if isinstance(t, torch.Tensor) else t


class Optimizer(Cell):
    _torch_cls = None

    def __init__(self, params, defaults=None, **kwargs):
        super().__init__(auto_prefix=False)
        groups = list(params)
        if not groups:
            raise ValueError("Optimizer got an empty parameter list.")
        if not isinstance(groups[0], dict):
            groups = [{"params": groups}]
        self._ms_params = [p for g in groups for p in g["params"]]
        torch_groups = []
        for g in groups:
            tg = {k: v for k, v in g.items() if k != "params"}
            # the torch optimizer updates the very storage of the framework's parameters
            tg["params"] = list(g["params"])
            torch_groups.append(tg)
        self._shadow = [p for g in torch_groups for p in g["params"]]
        self._opt = self._torch_cls(torch_groups, **kwargs)
        self.defaults = self._opt.defaults

    @property
    def parameters(self):
        return self._ms_params

    @property
    def param_groups(self):
        return self._opt.param_groups

    @property
    def lrs(self):
        return [g["lr"] for g in self._opt.param_groups]

    def add_param_group(self, param_group):
        self._ms_params += list(param_group["params"])
        self._opt.add_param_group(param_group)

    def state_dict(self):
        return self._opt.state_dict()

    def load_state_dict(self, sd):
        self._opt.load_state_dict(sd)

    def construct(self, gradients):
        for p, g in zip(self._shadow, gradients):
            p.grad = _plain(g).to(p.dtype) if g is not None else None
        self._opt.step()
        for p in self._shadow:
            p.grad = None
        return True

    def step(self, gradients):
        return self.construct(gradients)


def _make(name, torch_cls):
    cls = type(name, (Optimizer,), {"_torch_cls": torch_cls, "__doc__": "%s with torch.optim.%s semantics." % (name, name),
                                    "__init__": lambda self, params, *a, **kw: Optimizer.__init__(
                                        self, params, **_bind(torch_cls, a, kw))})
    return cls


def _bind(torch_cls, args, kwargs):
    import inspect
    names = [n for n in inspect.signature(torch_cls.__init__).parameters][2:]
    out = dict(zip(names, args))
    out.update(kwargs)
    for drop in ("foreach", "capturable", "differentiable", "fused"):
        out.pop(drop, None)
    return out


Adadelta = _make("Adadelta", torch.optim.Adadelta)
Adagrad = _make("Adagrad", torch.optim.Adagrad)
Adam = _make("Adam", torch.optim.Adam)
Adamax = _make("Adamax", torch.optim.Adamax)
AdamW = _make("AdamW", torch.optim.AdamW)
ASGD = _make("ASGD", torch.optim.ASGD)
NAdam = _make("NAdam", torch.optim.NAdam)
RAdam = _make("RAdam", torch.optim.RAdam)
RMSprop = _make("RMSprop", torch.optim.RMSprop)
Rprop = _make("Rprop", torch.optim.Rprop)
SGD = _make("SGD", torch.optim.SGD)


def _scheduler(name):
    base = getattr(torch.optim.lr_scheduler, name)

    class _S:
        __doc__ = "%s over an experimental.optim optimizer (torch.optim.lr_scheduler.%s semantics)." % (name, name)

        def __init__(self, optimizer, *args, **kwargs):
            inner = optimizer._opt if isinstance(optimizer, Optimizer) else optimizer
            if name in ("SequentialLR", "ChainedScheduler"):
                key = "schedulers"
                seq = kwargs.get(key) if key in kwargs else (args[0] if args else None)
                conv = [s._s if hasattr(s, "_s") else s for s in seq]
                if key in kwargs:
                    kwargs[key] = conv
                else:
                    args = (conv,) + tuple(args[1:])
                self._s = base(inner, *args, **kwargs) if name == "SequentialLR" else base(conv)
            else:
                self._s = base(inner, *args, **kwargs)
            self.optimizer = optimizer

        def step(self, *args, **kwargs):
            inner = self.optimizer._opt if isinstance(self.optimizer, Optimizer) else self.optimizer
            inner._opt_called = True                      # the optimizer is stepped through construct(), not step()
            return self._s.step(*args, **kwargs)

        def get_last_lr(self):
            return self._s.get_last_lr()

        def state_dict(self):
            return self._s.state_dict()

        def load_state_dict(self, sd):
            self._s.load_state_dict(sd)

    _S.__name__ = _S.__qualname__ = name
    return _S


lr_scheduler = types.ModuleType(__name__ + ".lr_scheduler")
lr_scheduler.__dict__.update({n: _scheduler(n) for n in (
    "StepLR", "LinearLR", "ExponentialLR", "PolynomialLR", "ChainedScheduler", "MultiplicativeLR", "ConstantLR",
    "SequentialLR", "ReduceLROnPlateau", "CyclicLR", "CosineAnnealingWarmRestarts", "CosineAnnealingLR", "LambdaLR",
    "MultiStepLR")})
lr_scheduler.LRScheduler = torch.optim.lr_scheduler.LRScheduler
lr_scheduler.__all__ = [n for n in vars(lr_scheduler) if not n.startswith("_")]
import sys as _sys  # noqa: E402

_sys.modules[lr_scheduler.__name__] = lr_scheduler        # `from ...experimental.optim.lr_scheduler import StepLR`
__path__ = []                                             # lets the import system look below this module
