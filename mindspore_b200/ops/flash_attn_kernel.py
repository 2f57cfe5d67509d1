"""Python side of the tcgen05 FlashAttention kernels (``csrc/cuda/flash_attn_sm100.cu``)."""
import ctypes
import math

import torch

from .. import _native
from . import kernels as K
from .kernels import _count, _p, _stream

_P, _I, _L, _F = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float
_native.register_cuda_signature("msb_flash_attn_fwd", _I, [_P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _L, _L, _L, _L, _I, _F, _P])
_native.register_cuda_signature("msb_flash_attn_bwd", _I, [_P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I,
                                                            _L, _L, _L, _L, _L, _I, _F, _P])


_native.register_cuda_signature("msb_flash_attn_bwd_strided", _I, [_P] * 10 + [_I] * 5 + [_L] * 7 + [_I, _F, _P])


def has_strided_bwd():
    return hasattr(_native.cuda(), "msb_flash_attn_bwd_strided")


def bwd_into(do, q, k, v, o, lse, causal, scale, dq, dk, dv, grad_pitch):
    """Backward with dq / dk / dv written into caller-provided column blocks (token pitch ``grad_pitch``)."""
    B, S, H, D = q.shape
    Hk = k.shape[2]
    do = do.contiguous()
    delta = torch.empty((B, H, S), dtype=torch.float32, device=q.device)
    rc = K._fn("msb_flash_attn_bwd_strided", q)(
        _p(q), _p(k), _p(v), _p(o), _p(do), _p(lse), _p(delta), _p(dq), _p(dk), _p(dv), B, S, H, Hk, D,
        _token_major(q), _token_major(k), _token_major(v), H * D, H * D, grad_pitch, grad_pitch, int(causal),
        float(scale), _stream())
    _native.check(rc, "flash_attn_bwd_strided")
    _count(3)


def available():
    return torch.cuda.is_available() and hasattr(_native.cuda(), "msb_flash_attn_fwd")


def _token_major(t):
    """[B, S, H, D] view with unit stride in D, heads D apart and batches S*pitch apart -> token pitch, else None."""
    B, S, H, D = t.shape
    if t.stride(3) != 1 or t.stride(2) != D:
        return None
    pitch = t.stride(1)
    if B > 1 and t.stride(0) != S * pitch:
        return None
    if pitch % 8 or t.data_ptr() % 16:
        return None
    return pitch


def supports(q, k, v):
    if not (q.is_cuda and q.dtype in (torch.bfloat16, torch.float16) and k.dtype == q.dtype and v.dtype == q.dtype):
        return False
    B, S, H, D = q.shape
    return D == 128 and S % 128 == 0 and k.shape[1] == S and H % k.shape[2] == 0 and k.shape[3] == 128


def fwd(q, k, v, causal, scale):
    B, S, H, D = q.shape
    Hk = k.shape[2]
    qp, kp, vp = _token_major(q), _token_major(k), _token_major(v)
    if qp is None:
        q = q.contiguous()
        qp = H * D
    if kp is None:
        k = k.contiguous()
        kp = Hk * D
    if vp is None:
        v = v.contiguous()
        vp = Hk * D
    o = torch.empty((B, S, H, D), dtype=q.dtype, device=q.device)
    lse = torch.empty((B, H, S), dtype=torch.float32, device=q.device)
    rc = K._fn("msb_flash_attn_fwd", q)(_p(q), _p(k), _p(v), _p(o), _p(lse), B, S, H, Hk, D, qp, kp, vp, H * D,
                                           int(causal), float(scale), _stream())
    _native.check(rc, "flash_attn_fwd")
    _count()
    return o, lse, q, k, v


def bwd(do, q, k, v, o, lse, causal, scale):
    lib = _native.cuda()
    B, S, H, D = q.shape
    Hk = k.shape[2]
    if not hasattr(lib, "msb_flash_attn_bwd") or Hk != H:
        return _bwd_reference(do, q, k, v, causal, scale)
    do = do.contiguous()
    qp, kp = _token_major(q), _token_major(k)
    dq = torch.empty((B, S, H, D), dtype=q.dtype, device=q.device)
    dk = torch.empty((B, S, Hk, D), dtype=q.dtype, device=q.device)
    dv = torch.empty((B, S, Hk, D), dtype=q.dtype, device=q.device)
    delta = torch.empty((B, H, S), dtype=torch.float32, device=q.device)
    rc = K._fn("msb_flash_attn_bwd", q)(_p(q), _p(k), _p(v), _p(o), _p(do), _p(lse), _p(delta), _p(dq), _p(dk), _p(dv), B, S, H,
                                Hk, D, qp, kp, _token_major(v), H * D, H * D, int(causal), float(scale), _stream())
    _native.check(rc, "flash_attn_bwd")
    _count(3)
    return dq, dk, dv


def _bwd_reference(do, q, k, v, causal, scale):
    """Recompute-and-differentiate path used where the backward kernel does not apply (e.g. grouped kv heads)."""
    from .attention import reference_attention
    with torch.enable_grad():
        qq, kk, vv = (t.detach().requires_grad_(True) for t in (q, k, v))
        out = reference_attention(qq, kk, vv, causal, scale)
        return torch.autograd.grad(out, (qq, kk, vv), do)


class _FlashFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, causal, scale):
        o, lse, q2, k2, v2 = fwd(q, k, v, causal, scale)
        ctx.save_for_backward(q2, k2, v2, o, lse)
        ctx.causal, ctx.scale = causal, scale
        return o

    @staticmethod
    def backward(ctx, do):
        q, k, v, o, lse = ctx.saved_tensors
        dq, dk, dv = bwd(do, q, k, v, o, lse, ctx.causal, ctx.scale)
        return dq, dk, dv, None, None


def flash_attention(q, k, v, causal=True, scale=None):
    scale = scale if scale is not None else 1.0 / math.sqrt(q.shape[-1])
    return _FlashFn.apply(q, k, v, bool(causal), float(scale))
