"""``Parameter`` and ``ParameterTuple``.

A Parameter is a named leaf ``Tensor``.  Besides MindSpore's attributes it may carry a *layout*
(how the full logical tensor is sharded over the device matrix) assigned by the parallel planner;
``init_data(layout)`` then keeps only this rank's slice, as the reference does after compile.

Parity: mindspore/python/mindspore/common/parameter.py:122 (class), :246 (__init__), :498 (clone),
:574 (comm_fusion), :646 (parallel_optimizer_comm_recompute), :795 (set_data), :842/:910
(init_data), :974/:1008 (ParameterTuple.clone).
"""
from __future__ import annotations

import itertools

import numpy as np
import torch

from . import dtype as mstype
from .tensor import Tensor, _to_torch

_uid = itertools.count()


def sync_master(param, value=None):
    """A parameter packed into an optimizer arena has an fp32 master copy (whole, or one slice per rank under the
    sharded optimizer) from which every update rewrites the low-precision weights: whoever overwrites the
    parameter's value calls this so that the master follows."""
    arena = getattr(param, "arena", None)
    owner = getattr(arena, "owner", None) if arena is not None else None
    opt = owner() if owner is not None else None
    if opt is not None:
        opt.write_master(param, param if value is None else value)


class Parameter(Tensor):
    @staticmethod
    def __new__(cls, default_input, name=None, requires_grad=True, layerwise_parallel=False,
                parallel_optimizer=True, storage_format="", device=None):
        if isinstance(default_input, (int, float, bool, np.ndarray, list, tuple)):
            t = _to_torch(default_input)
        elif isinstance(default_input, torch.Tensor):
            t = default_input.detach().as_subclass(torch.Tensor)
        else:
            raise TypeError("Parameter's default_input must be Tensor, int, float, numpy.ndarray or list, got %s"
                            % type(default_input))
        if device is None:
            from .. import context
            dev = context.device()
            if dev.type == "cuda" and t.device != dev:
                t = t.to(dev)
        elif t.device != torch.device(device):
            t = t.to(device)
        rg = bool(requires_grad) and (t.is_floating_point() or t.is_complex())
        obj = torch.Tensor._make_subclass(cls, t, rg)
        obj._ms_name = name if name is not None else "Parameter"
        obj._ms_requires_grad = bool(requires_grad)
        obj.layerwise_parallel = layerwise_parallel
        obj.parallel_optimizer = parallel_optimizer
        obj.storage_format = storage_format
        obj._comm_fusion = 1
        obj._parallel_optimizer_comm_recompute = False
        obj._sliced = False
        obj.is_init = False
        obj._uid = next(_uid)
        obj.param_layout = None          # parallel.TensorLayout of the full tensor, set by the planner
        obj.full_shape = None      # logical shape before slicing
        obj.opt_shard_group = None
        obj.is_in_shard = False
        obj._pipeline_stage_list = []
        obj.const_arg = False
        return obj

    def __init__(self, *args, **kwargs):
        pass

    @classmethod
    def __torch_function__(cls, func, types, args=(), kwargs=None):
        # results of arithmetic on a Parameter are plain Tensors, never Parameters
        if kwargs is None:
            kwargs = {}
        with torch._C.DisableTorchFunctionSubclass():
            ret = func(*args, **kwargs)
            if func in torch.overrides.get_default_nowrap_functions():
                return ret
            return torch._tensor._convert(ret, Tensor)

    def __repr__(self):
        return "Parameter (name=%s, shape=%s, dtype=%s, requires_grad=%s)" % (
            self.name, tuple(self.shape), self.dtype, self._ms_requires_grad)

    __str__ = __repr__

    def __deepcopy__(self, memo):
        out = self.clone_param()
        memo[id(self)] = out
        return out

    def __reduce_ex__(self, proto):
        return (_rebuild_parameter, (self.asnumpy(), self.dtype, self.name, self._ms_requires_grad))

    # ------------------------------------------------------------------ identity
    @property
    def name(self):
        return self._ms_name

    @name.setter
    def name(self, value):
        if value is not None and not isinstance(value, str):
            raise ValueError("The type of the Parameter's name should be 'string' or 'None', got %s" % type(value))
        self._ms_name = value if value else "Parameter"

    @property
    def param_info(self):
        return self

    @property
    def inited_param(self):
        return self

    @property
    def unique(self):
        return getattr(self, "_unique", False)

    @unique.setter
    def unique(self, v):
        self._unique = v

    @property
    def cache_shape(self):
        """Shape of the cache-enabled (embedding-cache) form of this parameter, if any."""
        return self.__dict__.get("_cache_shape", ())

    @cache_shape.setter
    def cache_shape(self, value):
        if not isinstance(value, (tuple, list)):
            raise TypeError("'cache_shape' must be a tuple or list, but got %s" % type(value))
        self.__dict__["_cache_shape"] = tuple(value)

    @property
    def key(self):
        """Unique key of the parameter (process-wide)."""
        return self.__dict__.setdefault("_key", id(self))

    @key.setter
    def key(self, value):
        self.__dict__["_key"] = int(value)

    def set_param_fl(self, push_to_server=False, pull_from_server=False, requires_aggr=True):
        """Federated-learning flags: whether the value is pushed to / pulled from a server and aggregated."""
        self.__dict__["push_weight_to_server"] = bool(push_to_server)
        self.__dict__["pull_weight_from_server"] = bool(pull_from_server)
        self.__dict__["requires_aggr"] = bool(requires_aggr)

    @property
    def sliced(self):
        return self._sliced

    @sliced.setter
    def sliced(self, v):
        self._sliced = bool(v)

    @property
    def comm_fusion(self):
        return self._comm_fusion

    @comm_fusion.setter
    def comm_fusion(self, v):
        if not isinstance(v, int) or v < 0:
            raise ValueError("comm_fusion must be a non-negative int, got %r" % (v,))
        self._comm_fusion = v

    @property
    def parallel_optimizer_comm_recompute(self):
        return self._parallel_optimizer_comm_recompute

    @parallel_optimizer_comm_recompute.setter
    def parallel_optimizer_comm_recompute(self, v):
        self._parallel_optimizer_comm_recompute = bool(v)

    @property
    def is_param_ps(self):
        return getattr(self, "_is_param_ps", False)

    def set_param_ps(self, init_in_server=False):
        """Marks the parameter as living on the parameter server (``parallel.ps``)."""
        self._is_param_ps = True
        self._init_in_server = bool(init_in_server)

    def add_pipeline_stage(self, stage):
        if not isinstance(stage, int) or stage < 0:
            raise TypeError("`stage` must be a non-negative int")
        if stage not in self._pipeline_stage_list:
            self._pipeline_stage_list.append(stage)

    @property
    def cache_enable(self):
        return False

    # ------------------------------------------------------------------ data
    def value(self):
        return self.detach().as_subclass(Tensor)

    def set_data(self, data, slice_shape=False):
        new = _to_torch(data, device=self.device) if not isinstance(data, torch.Tensor) else \
            data.detach().as_subclass(torch.Tensor).to(self.device)
        if tuple(new.shape) != tuple(self.shape) and not slice_shape and not self._sliced and new.numel() != 0 \
                and self.numel() != 0 and self.full_shape is None:
            raise ValueError("Can not change the shape of Parameter %s: %s -> %s (pass slice_shape=True)"
                             % (self.name, tuple(self.shape), tuple(new.shape)))
        with torch.no_grad():
            if tuple(new.shape) == tuple(self.shape) and new.dtype == self.dtype:
                torch.Tensor.copy_(self, new)
                sync_master(self, new)
            else:
                _swap_storage(self, new)
        return self

    def init_data(self, layout=None, set_sliced=False):
        """Keeps only this rank's slice when a layout is given (reference: parameter.py:910)."""
        if layout is not None and not self._sliced:
            from ..parallel.layout import slice_for_rank
            from .. import context
            rank = context.get_auto_parallel_context("global_rank")
            self.full_shape = tuple(self.shape)
            sl = slice_for_rank(self.detach().as_subclass(torch.Tensor), layout, rank)
            self.set_data(sl.clone(), slice_shape=True)
            self.param_layout = layout
            if set_sliced:
                self._sliced = True
        self.is_init = True
        return self

    def clone_param(self, init="same"):
        t = self.detach().as_subclass(torch.Tensor).clone()
        if init != "same":
            from .initializer import initializer
            t = initializer(init, tuple(self.shape), self.dtype).as_subclass(torch.Tensor).to(self.device)
        p = Parameter(t, name=self.name, requires_grad=self._ms_requires_grad,
                      layerwise_parallel=self.layerwise_parallel, parallel_optimizer=self.parallel_optimizer,
                      device=self.device)
        p.param_layout = self.param_layout
        p.full_shape = self.full_shape
        p._sliced = self._sliced
        p.cloned_from = self
        return p

    def clone(self, init="same", **kwargs):  # MindSpore's Parameter.clone returns a Parameter
        if kwargs or not (isinstance(init, (str, int, float)) or hasattr(init, "_initialize")):
            return torch.Tensor.clone(self, **kwargs)  # torch-internal call with memory_format etc.
        return self.clone_param(init)

    def copy(self):
        return self.clone_param()


def _swap_storage(param, new):
    """Rebinds the parameter to a tensor of another shape/dtype (slicing by layout, dtype casts)."""
    param.data = new.to(param.device).contiguous()


def _rebuild_parameter(arr, dtype, name, requires_grad):
    return Parameter(Tensor(arr, dtype=dtype), name=name, requires_grad=requires_grad)


class ParameterTuple(tuple):
    """Tuple of Parameters with unique names; ``clone(prefix, init)`` makes optimizer state."""

    def __new__(cls, iterable):
        data = tuple(iterable)
        names = set()
        for p in data:
            if not isinstance(p, Parameter):
                raise TypeError("ParameterTuple input should be `Parameter` collection, got %s" % type(p))
            if p.name in names:
                raise ValueError("The value %s has the same name '%s' with a previous Parameter" % (p, p.name))
            names.add(p.name)
        return tuple.__new__(ParameterTuple, data)

    def clone(self, prefix, init="same"):
        if not isinstance(prefix, str) or not prefix:
            raise ValueError("The prefix must be a non-empty str")
        new = []
        for p in self:
            c = p.clone_param(init)
            c.name = prefix + "." + p.name
            new.append(c)
        return ParameterTuple(new)

    def __parameter_tuple__(self):
        return True
