"""``Primitive``: the unit of computation shared by eager mode, graph tracing and auto-parallel.

A Primitive instance carries attributes (``add_prim_attr``), a shard strategy (``shard``), a pipeline
stage and a recompute flag.  Calling it either executes ``_run`` immediately on torch tensors
(PyNative) or, while a graph is being traced, records one IR node whose target is the instance
itself - so the parallel planner sees primitive names and strategies exactly as user code set them.

Parity: mindspore/python/mindspore/ops/primitive.py:35 (Primitive), :68 add_prim_attr, :161-216
(strategy checks), :238 set_stage, :257 shard, :437 recompute, :635 PrimitiveWithInfer,
:737 prim_attr_register, :859 constexpr.
"""
from __future__ import annotations

import functools
import inspect

import torch

from ..common.tensor import Tensor
from ..context import _AutoParallelContext

_parallel_ctx = _AutoParallelContext()
_SHARDED_MODES = ("semi_auto_parallel", "auto_parallel")

# set by graph.tracer while a trace is in flight: callable(prim, args, kwargs) -> proxy or NotImplemented
_trace_hook = None


def _set_trace_hook(hook):
    global _trace_hook
    _trace_hook = hook


def _wrap_out(out):
    if isinstance(out, torch.Tensor):
        return out if isinstance(out, Tensor) else out.as_subclass(Tensor)
    if isinstance(out, tuple):
        return tuple(_wrap_out(o) for o in out)
    if isinstance(out, list):
        return [_wrap_out(o) for o in out]
    return out


class Primitive:
    def __init__(self, name):
        self.name = name
        self.__name__ = name        # graph nodes take their label from the target's __name__
        self.attrs = {}
        self.init_attrs = {"name": name}
        self._update_parameter = False
        self.in_strategy = None
        self.out_strategy = None
        self.in_layout = None
        self.out_layout = None
        self.stage = None
        self.recompute_flag = None

    # ------------------------------------------------------------------ attributes
    def add_prim_attr(self, name, value):
        self.__dict__[name] = value
        self.attrs[name] = value
        return self

    def del_prim_attr(self, name):
        if name in self.__dict__ and name in self.attrs:
            del self.__dict__[name]
            del self.attrs[name]
        return self

    def _add_prim_arg(self, name, value):
        self.__dict__[name] = value
        self.init_attrs[name] = value
        self.attrs[name] = value

    def set_prim_instance_name(self, instance_name):
        self.instance_name = instance_name
        return self

    def set_stage(self, stage):
        if not isinstance(stage, int) or stage < 0:
            raise TypeError("stage must be a non-negative int")
        self.stage = stage
        self.add_prim_attr("stage", stage)
        return self

    def set_device(self, device_target):
        self.add_prim_attr("primitive_target", device_target)
        return self

    def place(self, role, rank_id):
        self.add_prim_attr("ms_role", role)
        self.add_prim_attr("rank_id", rank_id)
        return self

    def recompute(self, mode=True):
        if not isinstance(mode, bool):
            raise TypeError("recompute mode must be bool")
        self.recompute_flag = mode
        self.add_prim_attr("recompute", mode)
        return self

    def init_prim_io_names(self, inputs, outputs):
        self.add_prim_attr("input_names", list(inputs))
        self.add_prim_attr("output_names", list(outputs))

    # ------------------------------------------------------------------ shard strategies
    @staticmethod
    def _check_strategy(strategy, label):
        from ..parallel.layout import Layout
        if strategy is None:
            return None, False
        if not isinstance(strategy, tuple):
            raise TypeError("%s must be tuple type, but got %s" % (label, type(strategy)))
        is_layout = None
        for s in strategy:
            this = isinstance(s, Layout)
            if is_layout is None:
                is_layout = this
            elif is_layout != this:
                raise TypeError("%s elements must all be tuple(int) or all be Layout" % label)
            if not this:
                if not isinstance(s, tuple):
                    raise TypeError("The element of %s must be tuple/Layout type, but got %s" % (label, type(s)))
                for d in s:
                    if not isinstance(d, int) or isinstance(d, bool):
                        raise TypeError("The %s value must be int, but got %s" % (label, type(d)))
                    if d < 1:
                        raise ValueError("The %s value must be positive, but got %d" % (label, d))
        return strategy, bool(is_layout)

    def shard(self, in_strategy=None, out_strategy=None):
        from .. import context
        mode = context.get_auto_parallel_context("parallel_mode")
        in_s, in_is_layout = self._check_strategy(in_strategy, "in_strategy")
        out_s, out_is_layout = self._check_strategy(out_strategy, "out_strategy")
        if in_s is None and out_s is not None:
            raise ValueError("The out_strategy of %s is %s, need to set in_strategy, but got none" % (self.name, out_s))
        if in_s is not None and out_s is not None and in_is_layout != out_is_layout:
            raise ValueError("in_strategy and out_strategy must both be tuples of int or both be Layouts")
        if mode not in (context.ParallelMode.AUTO_PARALLEL, context.ParallelMode.SEMI_AUTO_PARALLEL):
            from ..utils.log import logger
            logger.warning("The shard strategy %s of %s is valid only when parallel_mode is semi_auto_parallel "
                           "or auto_parallel (current: %s)", in_strategy, self.name, mode)
        if in_is_layout:
            self.in_layout = in_s
            self.out_layout = out_s
            self.add_prim_attr("in_layout", tuple(l.to_dict() for l in in_s))
            if out_s is not None:
                self.add_prim_attr("out_layout", tuple(l.to_dict() for l in out_s))
            self.in_strategy = self.out_strategy = None
        else:
            self.in_strategy = in_s
            self.out_strategy = out_s
            self.add_prim_attr("in_strategy", in_s)
            self.add_prim_attr("out_strategy", out_s)
        return self

    # ------------------------------------------------------------------ execution
    def _run(self, *args, **kwargs):
        raise NotImplementedError("Primitive %s has no implementation" % self.name)

    def __call__(self, *args, **kwargs):
        if _trace_hook is not None:
            out = _trace_hook(self, args, kwargs)
            if out is not NotImplemented:
                return out
        return _wrap_out(self._execute(*args, **kwargs))

    def _execute(self, *args, **kwargs):
        """``_run`` under the current parallel mode: with a shard strategy (or sharded inputs) in
        semi_auto_parallel / auto_parallel mode the call goes through the SPMD dispatcher."""
        if _parallel_ctx._v["parallel_mode"] in _SHARDED_MODES and type(self).__module__[-8:] != "comm_ops":
            from ..parallel import spmd
            if spmd.needs_dispatch(self, args):
                out = spmd.dispatch(self, args, kwargs)
                if out is not NotImplemented:
                    return out
        return self._run(*args, **kwargs)

    def __repr__(self):
        extra = ", ".join("%s=%r" % (k, v) for k, v in self.init_attrs.items() if k != "name")
        return "Prim[%s]%s" % (self.name, "<" + extra + ">" if extra else "")

    def __getstate__(self):
        return self.__dict__

    def __setstate__(self, d):
        self.__dict__.update(d)

    def infer(self, *args, **kwargs):
        """The abstract result (shape with symbolic dimensions, dtype) for abstract or placeholder inputs, without
        running a kernel.  Parity (role): the InferShape / InferType pair of every primitive in core/ops."""
        from ..graph.abstract import infer
        return infer(self, *args, **kwargs)

    def check_elim(self, *args):
        return (False, None)

    @property
    def update_parameter(self):
        return self._update_parameter

    def set_const_prim(self, is_const_prim):
        self.const_prim = is_const_prim


class PrimitiveWithInfer(Primitive):
    """A primitive that answers shape / dtype questions before it runs.  The defaults evaluate the primitive on
    storage-less tensors (``graph/abstract.py``); a subclass may override ``infer_shape`` / ``infer_dtype`` /
    ``infer_value`` and ``__infer__`` then uses those.  Parity: ops/primitive.py PrimitiveWithInfer."""

    def infer_shape(self, *shapes):
        """Output shape(s) for input shapes (lists; -1 marks a dynamic dimension, which stays -1 where it flows)."""
        from ..graph.abstract import AbstractTensor
        out = self.infer(*[AbstractTensor([None if d == -1 else d for d in s], torch.float32) for s in shapes])
        return _shapes_of(out)

    def infer_dtype(self, *dtypes):
        """Output dtype(s) for input dtypes; the primitive is tried on inputs of rank 0 to 4."""
        from ..graph.abstract import AbstractTensor, InferenceError
        err = None
        for rank in range(5):
            try:
                out = self.infer(*[AbstractTensor([2] * rank, d) for d in dtypes])
                return _dtypes_of(out)
            except InferenceError as e:
                err = e
        raise err

    def infer_value(self, *args):
        return None

    def __infer__(self, *inputs):
        """``inputs``: dicts with ``shape`` / ``dtype`` / ``value``; returns the same form for the output."""
        from ..graph.abstract import AbstractTensor
        own = type(self)
        if own.infer_shape is not PrimitiveWithInfer.infer_shape or own.infer_dtype is not PrimitiveWithInfer.infer_dtype:
            shape = self.infer_shape(*[i["shape"] for i in inputs])
            dtype = self.infer_dtype(*[i["dtype"] for i in inputs])
            return {"shape": shape, "dtype": dtype, "value": self.infer_value(*[i.get("value") for i in inputs])}
        out = self.infer(*[AbstractTensor([None if d == -1 else d for d in i["shape"]], i["dtype"]) for i in inputs])
        return {"shape": _shapes_of(out), "dtype": _dtypes_of(out), "value": None}


def _shapes_of(a):
    from ..graph.abstract import AbstractSequence, AbstractTensor
    if isinstance(a, AbstractTensor):
        return a.shape_list
    if isinstance(a, AbstractSequence):
        return a.kind(_shapes_of(e) for e in a.elements)
    return None


def _dtypes_of(a):
    from ..graph.abstract import AbstractScalar, AbstractSequence, AbstractTensor
    if isinstance(a, AbstractTensor):
        return a.dtype
    if isinstance(a, AbstractSequence):
        return a.kind(_dtypes_of(e) for e in a.elements)
    if isinstance(a, AbstractScalar):
        return a.type
    return None


class PrimitiveWithCheck(Primitive):
    def check_shape(self, *args):
        pass

    def check_dtype(self, *args):
        pass


def prim_attr_register(fn):
    """Decorator for ``__init__``: records constructor arguments as primitive attributes."""

    @functools.wraps(fn)
    def deco(self, *args, **kwargs):
        class_name = self.__class__.__name__
        if getattr(self, "_prim_inited", False) is False:
            Primitive.__init__(self, class_name)
            self._prim_inited = True
        bound = inspect.signature(fn).bind(self, *args, **kwargs)
        bound.apply_defaults()
        for name, value in list(bound.arguments.items())[1:]:
            self._add_prim_arg(name, value)
        fn(self, *args, **kwargs)

    deco.decorated_func = fn
    return deco


def prim_arg_register(fn):
    return prim_attr_register(fn)


def constexpr(fn=None, get_instance=True, name=None, reuse_result=True, check=True):
    """Marks ``fn`` as evaluated on constants at trace time; in this runtime that is a plain call."""

    def deco(f):
        @functools.wraps(f)
        def wrapper(*args, **kwargs):
            return f(*args, **kwargs)

        wrapper.__constexpr__ = True
        return wrapper

    if fn is not None:
        return deco(fn)
    return deco


def _primexpr(fn=None, **kw):
    return constexpr(fn, **kw)
