"""ctypes bindings of the two in-tree native libraries.

``cuda()`` returns the sm_100a kernel library, ``host()`` the C++ host runtime
(layout algebra, search, schedulers, codecs).  Both are built on first use if
missing (see :mod:`mindspore_b200._native.build`).  A kernel entry point that
reports a non-zero code raises :class:`NativeError` carrying the library's
message, so a missing or failing extension is never silent.
"""
from __future__ import annotations

import ctypes
import os
import threading

from . import build as _build

_lock = threading.Lock()
_cuda = None
_host = None


class NativeError(RuntimeError):
    pass


def _load(path, builder):
    if not os.path.exists(path) or os.environ.get("MSB200_REBUILD") == "1":
        builder(verbose=True)
    try:
        return ctypes.CDLL(path)
    except OSError:
        builder(verbose=True)
        return ctypes.CDLL(path)


def host():
    """The host C++ library (always available: needs only g++)."""
    global _host
    if _host is None:
        with _lock:
            if _host is None:
                _host = _load(_build.HOST_LIB, _build.build_host)
    return _host


_P = ctypes.c_void_p
_I = ctypes.c_int
_L = ctypes.c_longlong
_F = ctypes.c_float

_CUDA_SIGNATURES = {
    "msb_last_error": (ctypes.c_char_p, []),
    "msb_read_status": (_I, [_I]),
    "msb_gemm_bf16": (_I, [_P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _L, _L, _L, _L, _L, _L, _I, _I, _F, _I, _P]),
    "msb_gemm_bf16_pair": (_I, [_P, _P, _P, _P, _I, _I, _I, _I, _I, _L, _L, _L, _I, _I, _F, _I, _P, _P]),
    "msb_rmsnorm_fwd": (_I, [_P, _P, _P, _P, _P, _P, _L, _I, _F, _P]),
    "msb_rmsnorm_bwd": (_I, [_P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _L, _I, _P]),
    "msb_layernorm_fwd": (_I, [_P, _P, _P, _P, _P, _P, _L, _I, _F, _P]),
    "msb_layernorm_bwd": (_I, [_P, _P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _L, _I, _P]),
    "msb_rope": (_I, [_P, _P, _P, _P, _L, _I, _I, _L, _I, _I, _P]),
    "msb_swiglu_fwd": (_I, [_P, _P, _L, _I, _P]),
    "msb_swiglu_bwd": (_I, [_P, _P, _P, _L, _I, _P]),
    "msb_gelu": (_I, [_P, _P, _P, _P, _L, _I, _I, _P]),
    "msb_ce_stats": (_I, [_P, _P, _P, _L, _I, _L, _I, _I, _P]),
    "msb_ce_grad": (_I, [_P, _P, _P, _P, _P, _P, _L, _I, _L, _I, _I, _I, _I, _P]),
    "msb_adamw": (_I, [_P, _P, _P, _P, _I, _P, _L, _P, _P, _P]),
    "msb_momentum": (_I, [_P, _P, _P, _I, _P, _L, _P, _P, _P]),
    "msb_sumsq_finite": (_I, [_P, _I, _L, _P, _P, _P]),
    "msb_finalize_grad_scale": (_I, [_P, _P, _F, _F, _P, _P, _P, _P]),
    "msb_embedding_fwd": (_I, [_P, _P, _P, _L, _I, _I, _I, _P]),
    "msb_embedding_bwd": (_I, [_P, _P, _P, _L, _I, _I, _I, _P]),
    "msb_cast_f32_to_bf16": (_I, [_P, _P, _L, _F, _P]),
    "msb_cast_bf16_to_f32": (_I, [_P, _P, _L, _F, _I, _P]),
    "msb_add_bf16": (_I, [_P, _P, _P, _L, _P]),
}


def _apply_signature(lib, name, restype, argtypes):
    """Sets the ctypes signature of ``name`` and of its fp16 build (``name_fp16``, or ``..._fp16`` for a name that
    spells ``bf16``), which takes the same arguments."""
    for n in {name, name + "_fp16", name.replace("bf16", "fp16")}:
        if hasattr(lib, n):
            fn = getattr(lib, n)
            fn.restype, fn.argtypes = restype, argtypes


def register_cuda_signature(name, restype, argtypes):
    """Lets later modules (attention, conv, fused collectives) declare their entry points."""
    _CUDA_SIGNATURES[name] = (restype, argtypes)
    if _cuda is not None:
        _apply_signature(_cuda, name, restype, argtypes)


def cuda():
    """The sm_100a kernel library.  Raises if it cannot be built or loaded."""
    global _cuda
    if _cuda is None:
        with _lock:
            if _cuda is None:
                lib = _load(_build.CUDA_LIB, _build.build_cuda)
                for name, (res, args) in _CUDA_SIGNATURES.items():
                    _apply_signature(lib, name, res, args)
                _cuda = lib
    return _cuda


def check(rc, what="kernel"):
    if rc != 0:
        msg = cuda().msb_last_error()
        raise NativeError("%s failed (code %d): %s" % (what, rc, msg.decode() if msg else "?"))


def device_status(clear=True) -> int:
    """Reads the device status word: non-zero means a kernel abandoned a bounded wait."""
    return int(cuda().msb_read_status(1 if clear else 0))


launch_count = 0  # number of kernel launcher calls made through mindspore_b200.ops.kernels
