"""Data types.  MindSpore's dtype objects map one-to-one onto ``torch.dtype`` singletons, so
``mindspore_b200.float32 is torch.float32`` and tensors need no dtype translation layer.

Parity: mindspore/python/mindspore/common/dtype.py (type objects, ``dtype_to_nptype``,
``pytype_to_dtype``, ``get_py_obj_dtype``) and the checkpoint type strings of
mindspore/python/mindspore/train/serialization.py:78-85.
"""
from __future__ import annotations

import numpy as np
import torch

float16 = half = torch.float16
float32 = single = float_ = torch.float32
float64 = double = torch.float64
bfloat16 = torch.bfloat16
int8 = byte = torch.int8
int16 = short = torch.int16
int32 = intc = torch.int32
int64 = intp = int_ = torch.int64
uint8 = ubyte = torch.uint8
uint16 = getattr(torch, "uint16", torch.int16)
uint32 = getattr(torch, "uint32", torch.int32)
uint64 = getattr(torch, "uint64", torch.int64)
ushort, uintc, uintp, uint = uint16, uint32, uint64, uint64          # C-style aliases (common/dtype.py:69-73)
qint4x2 = torch.int8                                                  # two 4-bit values per byte: stored as bytes


class TensorType:
    """``TensorType(element_type)``: the type of a tensor whose elements have ``element_type``."""

    def __init__(self, element_type=None):
        self._element_type = element_type

    def element_type(self):
        return self._element_type

    def __eq__(self, other):
        return isinstance(other, TensorType) and other._element_type == self._element_type

    def __hash__(self):
        return hash(("TensorType", self._element_type))

    def __repr__(self):
        return "Tensor[%s]" % (dtype_to_pytype(self._element_type).__name__ if False else self._element_type)


tensor_type = TensorType


class Int:
    """Integer type descriptor with a bit width, e.g. ``Int(32)``; compares equal to the matching dtype."""

    _BY_BITS = {}

    def __init__(self, nbits=64):
        self.nbits = int(nbits)

    def __eq__(self, other):
        if isinstance(other, Int):
            return other.nbits == self.nbits
        return other is Int._BY_BITS.get(self.nbits)

    def __hash__(self):
        return hash(("Int", self.nbits))

    def __repr__(self):
        return "Int%d" % self.nbits
bool_ = torch.bool
complex64 = torch.complex64
complex128 = torch.complex128

number_type = (int8, int16, int32, int64, uint8, float16, float32, float64, bfloat16, complex64, complex128)
int_type = (int8, int16, int32, int64)
uint_type = (uint8,)
float_type = (float16, float32, float64, bfloat16)

Type = torch.dtype


class _Marker:
    """Non-tensor type markers (``mstype.tensor_type``, ``mstype.tuple_`` ...) used in signatures."""

    def __init__(self, name):
        self._name = name

    def __repr__(self):
        return self._name


tensor_type = tensor = _Marker("Tensor")
tuple_ = _Marker("Tuple")
list_ = _Marker("List")
string = _Marker("String")
type_none = _Marker("None")
function = _Marker("Function")
number = _Marker("Number")

_NP = {
    float16: np.float16, float32: np.float32, float64: np.float64, int8: np.int8, int16: np.int16,
    int32: np.int32, int64: np.int64, uint8: np.uint8, bool_: np.bool_, complex64: np.complex64,
    complex128: np.complex128,
}

# checkpoint / MindIR type strings (serialization.py:78-85)
_CKPT_NAME = {
    uint8: "UInt8", int8: "Int8", int16: "Int16", int32: "Int32", int64: "Int64", float16: "Float16",
    float32: "Float32", float64: "Float64", bool_: "Bool", bfloat16: "BFloat16",
}
_CKPT_NAME_REV = {v: k for k, v in _CKPT_NAME.items()}
_CKPT_NAME_REV.update({"UInt16": torch.int16, "UInt32": torch.int32, "UInt64": torch.int64})


def dtype_to_nptype(t):
    """bf16 has no NumPy type: it is surfaced as float32 (values preserved exactly)."""
    if t == bfloat16:
        return np.float32
    return _NP[t]


def nptype_to_dtype(npt):
    npt = np.dtype(npt)
    for k, v in _NP.items():
        if np.dtype(v) == npt:
            return k
    if npt == np.uint16:
        return int32
    if npt == np.uint32 or npt == np.uint64:
        return int64
    raise TypeError("unsupported numpy dtype %s" % npt)


def pytype_to_dtype(obj):
    if isinstance(obj, torch.dtype):
        return obj
    if obj is bool:
        return bool_
    if obj is int:
        return int64
    if obj is float:
        return float32
    if obj is complex:
        return complex64
    if isinstance(obj, type) and issubclass(obj, np.generic):
        return nptype_to_dtype(obj)
    raise NotImplementedError("no dtype for python type %r" % (obj,))


def get_py_obj_dtype(obj):
    if isinstance(obj, torch.Tensor):
        return obj.dtype
    return pytype_to_dtype(type(obj))


def dtype_to_pytype(t):
    if t == bool_:
        return bool
    if t in int_type or t in uint_type:
        return int
    if t in float_type:
        return float
    if t in (complex64, complex128):
        return complex
    raise NotImplementedError(str(t))


def ckpt_type_name(t) -> str:
    return _CKPT_NAME[t]


def ckpt_type_from_name(name: str):
    return _CKPT_NAME_REV[name]


def type_size_in_bytes(t) -> int:
    return torch.empty((), dtype=t).element_size()


def is_floating(t) -> bool:
    return t in float_type

Int._BY_BITS.update({8: int8, 16: int16, 32: int32, 64: int64})


import enum as _enum


class QuantDtype(_enum.Enum):
    """Integer widths for quantisation: INT1 .. INT16 (values 0 .. 15) and UINT1 .. UINT16 (100 .. 115).
    Parity: python/mindspore/common/dtype.py:353."""
    locals().update({"INT%d" % b: b - 1 for b in range(1, 17)})
    locals().update({"UINT%d" % b: 99 + b for b in range(1, 17)})

    def __str__(self):
        return self.name

    @staticmethod
    def is_signed(dtype):
        return dtype.value < 100

    @staticmethod
    def switch_signed(dtype):
        return QuantDtype(dtype.value + 100) if dtype.value < 100 else QuantDtype(dtype.value - 100)

    @property
    def num_bits(self):
        return self.value % 100 + 1

    def value_range(self):
        b = self.num_bits
        return (-(1 << (b - 1)), (1 << (b - 1)) - 1) if self.value < 100 else (0, (1 << b) - 1)
