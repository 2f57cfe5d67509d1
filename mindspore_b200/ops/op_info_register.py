"""Operator registration records for ``ops.Custom`` (python/mindspore/ops/op_info_register.py): builders that collect
the inputs, outputs, attributes and supported dtype / format combinations of a custom operator into the dictionary
``Custom(reg_info=...)`` consumes, and the ``DataType`` table of (dtype, format) pairs."""
from __future__ import annotations

import functools


class _DataTypeMeta(type):
    """``DataType.F16_Default`` style names resolve to (dtype, format) pairs: <dtype code>_<format>."""

    _DTYPES = {"None": "", "BOOL": "bool", "I8": "int8", "I16": "int16", "I32": "int32", "I64": "int64", "U8": "uint8",
               "U16": "uint16", "U32": "uint32", "U64": "uint64", "F16": "float16", "F32": "float32", "F64": "float64",
               "BF16": "bfloat16", "C64": "complex64", "C128": "complex128"}

    def __getattr__(cls, name):
        code, _, fmt = name.partition("_")
        if code in cls._DTYPES and fmt:
            return (cls._DTYPES[code], "DefaultFormat" if fmt == "Default" else fmt)
        raise AttributeError(name)


class DataType(metaclass=_DataTypeMeta):
    """(dtype, format) pairs for ``dtype_format``: ``DataType.F32_Default``, ``DataType.F16_NCHW``, ..."""


class RegOp:
    def __init__(self, op_name=""):
        if not isinstance(op_name, str):
            raise ValueError("op name value must be string")
        self.op_name = op_name
        self.inputs, self.outputs, self.attr_, self.dtype_format_ = [], [], [], []
        self.fusion_type_ = ""
        self.target_ = None

    def _io(self, kind, index, name, param_type, **kwargs):
        if index is not None and (not isinstance(index, int) or index < 0):
            raise TypeError("%s index must be a non-negative int, got %r" % (kind, index))
        rec = {"index": index, "name": name, "param_type": param_type}
        rec.update(kwargs)
        return rec

    def input(self, index=None, name=None, param_type="required", **kwargs):
        self.inputs.append(self._io("input", index, name, param_type, **kwargs))
        return self

    def output(self, index=None, name=None, param_type="required", **kwargs):
        self.outputs.append(self._io("output", index, name, param_type, **kwargs))
        return self

    def attr(self, name=None, param_type=None, value_type=None, default_value=None, **kwargs):
        rec = {"name": name, "param_type": param_type, "type": value_type, "default_value": default_value}
        rec.update(kwargs)
        self.attr_.append(rec)
        return self

    def dtype_format(self, *args):
        if len(args) != len(self.inputs) + len(self.outputs):
            raise ValueError("dtype_format needs one (dtype, format) pair per input and output: %d given, %d expected"
                             % (len(args), len(self.inputs) + len(self.outputs)))
        for a in args:
            if not isinstance(a, tuple) or len(a) != 2:
                raise ValueError("dtype and format value must be a tuple of two, got %r" % (a,))
        self.dtype_format_.append(tuple(args))
        return self

    def target(self, target=None):
        self.target_ = target
        return self

    def get_op_info(self):
        info = {"op_name": self.op_name, "inputs": self.inputs, "outputs": self.outputs, "attr": self.attr_,
                "dtype_format": self.dtype_format_, "fusion_type": self.fusion_type_}
        if self.target_ is not None:
            info["target"] = self.target_
        return info


class CustomRegOp(RegOp):
    def __init__(self, op_name="Custom"):
        super().__init__(op_name)


class CpuRegOp(RegOp):
    pass


class AkgGpuRegOp(RegOp):
    def __init__(self, op_name=""):
        super().__init__(op_name)
        self.target_ = "GPU"


class AkgAscendRegOp(RegOp):
    pass


class AiCPURegOp(RegOp):
    pass


class TBERegOp(RegOp):
    pass


_registered = {}


def op_info_register(op_info):
    """Decorator that records an operator's registration next to its implementation function."""
    def deco(fn):
        info = op_info if isinstance(op_info, dict) else op_info.get_op_info() if hasattr(op_info, "get_op_info") \
            else {"raw": op_info}
        _registered[info.get("op_name", getattr(fn, "__name__", "op"))] = info

        @functools.wraps(fn)
        def wrapped(*args, **kwargs):
            return fn(*args, **kwargs)
        wrapped.reg_info = info
        return wrapped
    return deco


def custom_info_register(*reg_info):
    """Attaches registration records to the function of an ``ops.Custom`` operator (read back as ``fn.reg_info``)."""
    def deco(fn):
        infos = [r if isinstance(r, dict) else r.get_op_info() for r in reg_info]

        @functools.wraps(fn)
        def wrapped(*args, **kwargs):
            return fn(*args, **kwargs)
        wrapped.reg_info = tuple(infos)
        return wrapped
    return deco


class _VmImplRegistry:
    """Python fallbacks of primitives by class (ops/vm_impl_registry.py): ``register(PrimClass)(fn)``; ``get``
    returns the fallback of a primitive instance or class, or None."""

    def __init__(self):
        self._impl = {}

    def register(self, prim):
        def deco(fn):
            self._impl[prim if isinstance(prim, type) else type(prim)] = fn
            return fn
        return deco

    def get(self, prim, default=None):
        cls = prim if isinstance(prim, type) else type(prim)
        for c in cls.__mro__:
            if c in self._impl:
                return self._impl[c]
        return default


vm_impl_registry = _VmImplRegistry()


def get_vm_impl_fn(prim):
    """The registered Python fallback of ``prim``; without one, the primitive's own eager implementation."""
    fn = vm_impl_registry.get(prim)
    if fn is not None:
        return fn
    run = getattr(prim, "_run", None)
    return run if callable(run) else None
