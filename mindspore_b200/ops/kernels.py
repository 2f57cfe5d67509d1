"""Tensor-level entry points of the hand-written sm_100a kernels.

Every function takes ``torch`` CUDA tensors, launches on the current stream and
returns tensors; nothing here falls back to a library kernel - if the native
library is missing or a launcher rejects its arguments, a ``NativeError`` is
raised.  Layer code (``nn``), the graph executor and the parallel runtime all
call these, so the set of functions in this file is the GPU op inventory.
"""
from __future__ import annotations

import ctypes
import os

import torch

from .. import _native

bf16 = torch.bfloat16
f16 = torch.float16
f32 = torch.float32


def _fn(name, t):
    """The entry point for t's element type: the fp16 builds of the 16-bit kernels carry the suffix _fp16."""
    return getattr(_native.cuda(), name + "_fp16" if t.dtype == f16 else name)


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _p(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else None


def _count(n=1):
    _native.launch_count += n


# --------------------------------------------------------------------------------------- GEMM
_PAIR_GEMM = os.environ.get("MSB200_GEMM_PAIR", "1") == "1"


def _pair_gemm_ok(M, N, K, batch, out, o2, accumulate, bn_hint, dtype=bf16):
    """The CTA-pair kernel (256 x 256 tiles on two SMs) takes un-batched problems whose output meets the TMA
    alignment rules and that fill the machine with 256-wide tiles."""
    if not _PAIR_GEMM or batch != 1 or bn_hint not in (0, 512) or dtype != bf16:
        return False
    es = out.element_size()
    if out.data_ptr() % 16 or (o2.stride(0) * es) % 16 or (accumulate and out.dtype != f32):
        return False
    tiles = ((M + 255) // 256) * ((N + 255) // 256)
    if accumulate and K >= 2048:
        return M >= 512 and N >= 512 and tiles >= 16      # split-K fills the machine with fewer output tiles
    return M >= 512 and N >= 512 and tiles >= 64


def gemm(a, b, *, a_mn=False, b_mn=False, out=None, out_dtype=None, accumulate=False, bias=None,
         alpha=1.0, bn_hint=0):
    """``C (+)= alpha * A @ B^T (+ bias)`` on tcgen05 tensor cores.

    ``a`` holds the logical ``[.., M, K]`` operand, stored either as ``[.., M, K]``
    (``a_mn=False``) or transposed as ``[.., K, M]`` (``a_mn=True``); likewise ``b``
    holds logical ``[.., N, K]`` stored ``[.., N, K]`` or ``[.., K, N]``.  Rows must be
    contiguous; row pitch may exceed the row length (views of wider buffers are fine).
    """
    assert a.dtype == b.dtype and a.dtype in (bf16, f16), "gemm operands must both be bf16 or both fp16"
    assert bias is None or bias.dtype == a.dtype
    if out_dtype is None:
        out_dtype = a.dtype
    assert a.dim() == b.dim() and a.dim() in (2, 3)
    batched = a.dim() == 3
    if batched:
        batch = a.shape[0]
        assert b.shape[0] == batch
        a2, b2 = a[0], b[0]
    else:
        batch = 1
        a2, b2 = a, b
    assert a2.stride(1) == 1 and b2.stride(1) == 1, "innermost dim must be contiguous"
    if a_mn:
        K, M = a2.shape
    else:
        M, K = a2.shape
    if b_mn:
        Kb, N = b2.shape
    else:
        N, Kb = b2.shape
    assert K == Kb, "reduction dims differ: %d vs %d" % (K, Kb)
    lda, ldb = a2.stride(0), b2.stride(0)
    abs_ = a.stride(0) if batched else 0
    bbs_ = b.stride(0) if batched else 0
    if out is None:
        shape = (batch, M, N) if batched else (M, N)
        out = torch.empty(shape, dtype=out_dtype, device=a.device)
        assert not accumulate
    o2 = out[0] if batched else out
    assert o2.stride(1) == 1 and o2.shape == (M, N) and out.dtype in (a.dtype, f32)
    if _pair_gemm_ok(M, N, K, batch, out, o2, accumulate, bn_hint, a.dtype):
        rc = _native.cuda().msb_gemm_bf16_pair(_p(a), _p(b), _p(out), _p(bias), M, N, K, int(a_mn), int(b_mn), lda, ldb,
                                               o2.stride(0), int(out.dtype == f32), int(accumulate), float(alpha), 2,
                                               None, _stream())
        _native.check(rc, "gemm_pair")
        _count()
        return out
    rc = (_native.cuda().msb_gemm_fp16 if a.dtype == f16 else _native.cuda().msb_gemm_bf16)(
        _p(a), _p(b), _p(out), _p(bias), M, N, K, batch, int(a_mn), int(b_mn), lda, ldb, o2.stride(0),
        abs_, bbs_, out.stride(0) if batched else 0, int(out.dtype == f32), int(accumulate), float(alpha),
        int(bn_hint), _stream())
    _native.check(rc, "gemm")
    _count()
    return out


def linear_fwd(x, w, bias=None, out=None):
    """y[M,N] = x[M,K] @ w[N,K]^T (+ bias)."""
    return gemm(x, w, bias=bias, out=out)


def linear_dgrad(dy, w, out=None, accumulate=False):
    """dx[M,K] = dy[M,N] @ w[N,K]."""
    return gemm(dy, w, b_mn=True, out=out, accumulate=accumulate)


def linear_wgrad(dy, x, out=None, accumulate=False, out_dtype=f32):
    """dw[N,K] (+)= dy[M,N]^T @ x[M,K]; fp32 output accumulates micro-batches without a separate pass."""
    return gemm(dy, x, a_mn=True, b_mn=True, out=out, accumulate=accumulate, out_dtype=out_dtype)


# --------------------------------------------------------------------------------------- norms
_scratch = {}


def _acc_scratch(device, H, with_bias=False):
    """Scratch for the two-stage weight-gradient reduction of the norm backward kernels: one fp32 partial row of H
    per CTA (the size comes from the library, which knows its grid)."""
    lib = _native.cuda()
    lib.msb_norm_bwd_scratch_elems.restype = ctypes.c_longlong
    n = int(lib.msb_norm_bwd_scratch_elems(int(H), int(with_bias)))
    key = (device, "acc")
    buf = _scratch.get(key)
    if buf is None or buf.numel() < n:
        buf = torch.empty(n, dtype=f32, device=device)
        _scratch[key] = buf
    return buf


def rmsnorm_fwd(x, w, eps, residual=None):
    """Returns (y, rstd, xsum): y = rmsnorm(x + residual) * w; xsum is the summed stream (or x itself)."""
    H = x.shape[-1]
    rows = x.numel() // H
    y = torch.empty_like(x)
    rstd = torch.empty(rows, dtype=f32, device=x.device)
    xsum = torch.empty_like(x) if residual is not None else None
    rc = _fn("msb_rmsnorm_fwd", x)(_p(x), _p(residual), _p(w), _p(y), _p(xsum), _p(rstd), rows, H, float(eps),
                                        _stream())
    _native.check(rc, "rmsnorm_fwd")
    _count()
    return y, rstd, (xsum if xsum is not None else x)


def rmsnorm_bwd(dy, x, w, rstd, dresidual=None, dw_out=None, accumulate=False):
    """Returns (dx, dw).  dx includes ``dresidual`` when given; dw goes to ``dw_out`` (bf16/fp32) if given."""
    H = x.shape[-1]
    rows = x.numel() // H
    dx = torch.empty_like(x)
    acc = _acc_scratch(x.device, H)
    if dw_out is None:
        dw_out = torch.empty(H, dtype=w.dtype, device=x.device)
        accumulate = False
    rc = _fn("msb_rmsnorm_bwd", x)(_p(dy), _p(x), _p(w), _p(rstd), _p(dresidual), _p(dx), _p(acc), _p(dw_out),
                                        int(dw_out.dtype == f32), int(accumulate), rows, H, _stream())
    _native.check(rc, "rmsnorm_bwd")
    _count(2)
    return dx, dw_out


def layernorm_fwd(x, w, b, eps):
    H = x.shape[-1]
    rows = x.numel() // H
    y = torch.empty_like(x)
    mean = torch.empty(rows, dtype=f32, device=x.device)
    rstd = torch.empty(rows, dtype=f32, device=x.device)
    rc = _fn("msb_layernorm_fwd", x)(_p(x), _p(w), _p(b), _p(y), _p(mean), _p(rstd), rows, H, float(eps),
                                          _stream())
    _native.check(rc, "layernorm_fwd")
    _count()
    return y, mean, rstd


def layernorm_bwd(dy, x, w, mean, rstd, dw_out=None, db_out=None, accumulate=False, has_bias=True):
    H = x.shape[-1]
    rows = x.numel() // H
    dx = torch.empty_like(x)
    acc = _acc_scratch(x.device, H, with_bias=True)
    if dw_out is None:
        dw_out = torch.empty(H, dtype=w.dtype, device=x.device)
        db_out = torch.empty(H, dtype=w.dtype, device=x.device) if has_bias else None
        accumulate = False
    rc = _fn("msb_layernorm_bwd", x)(_p(dy), _p(x), _p(w), _p(mean), _p(rstd), _p(dx), _p(acc), _p(dw_out),
                                          _p(db_out), int(dw_out.dtype == f32), int(accumulate), rows, H, _stream())
    _native.check(rc, "layernorm_bwd")
    _count(3)
    return dx, dw_out, db_out


# --------------------------------------------------------------------------------------- RoPE / activations
def rope_(x, cos, sin, heads, head_dim, seq, positions=None, backward=False):
    """In-place rotate-half RoPE on x viewed as [tokens, heads*head_dim] with row pitch x.stride(-2)."""
    x2 = x.reshape(-1, x.shape[-1]) if x.is_contiguous() else x
    assert x2.dim() == 2 and x2.stride(1) == 1
    tokens = x2.shape[0]
    rc = _fn("msb_rope", x2)(_p(x2), _p(cos), _p(sin), _p(positions), tokens, heads, head_dim, x2.stride(0), seq,
                                 int(backward), _stream())
    _native.check(rc, "rope")
    _count()
    return x


def swiglu_fwd(gu):
    F = gu.shape[-1] // 2
    rows = gu.numel() // (2 * F)
    out = torch.empty(gu.shape[:-1] + (F,), dtype=gu.dtype, device=gu.device)
    _native.check(_fn("msb_swiglu_fwd", gu)(_p(gu), _p(out), rows, F, _stream()), "swiglu_fwd")
    _count()
    return out


def swiglu_bwd(gu, dout):
    F = gu.shape[-1] // 2
    rows = gu.numel() // (2 * F)
    dgu = torch.empty_like(gu)
    _native.check(_fn("msb_swiglu_bwd", gu)(_p(gu), _p(dout), _p(dgu), rows, F, _stream()), "swiglu_bwd")
    _count()
    return dgu


def gelu_fwd(x, bias=None):
    N = x.shape[-1]
    y = torch.empty_like(x)
    _native.check(_fn("msb_gelu", x)(_p(x), _p(bias), None, _p(y), x.numel() // N, N, 0, _stream()), "gelu")
    _count()
    return y


def gelu_bwd(x, dy, bias=None):
    N = x.shape[-1]
    dx = torch.empty_like(x)
    _native.check(_fn("msb_gelu", x)(_p(x), _p(bias), _p(dy), _p(dx), x.numel() // N, N, 1, _stream()), "gelu")
    _count()
    return dx


# --------------------------------------------------------------------------------------- cross entropy
def ce_stats(logits, labels, vocab_start=0):
    V = logits.shape[-1]
    rows = logits.numel() // V
    l2 = logits.reshape(rows, V)
    stats = torch.empty(rows, 3, dtype=f32, device=logits.device)
    rc = _native.cuda().msb_ce_stats(_p(l2), _p(labels), _p(stats), rows, V, l2.stride(0), vocab_start,
                                     int(logits.dtype == f32), _stream())
    _native.check(rc, "ce_stats")
    _count()
    return stats


def ce_loss_grad(logits, labels, stats, grad_scale, vocab_start=0, ignore_index=-100, dlogits=None,
                 want_grad=True):
    """Per-row loss and (optionally) in-place-able dlogits = (softmax - onehot) * grad_scale[0]."""
    V = logits.shape[-1]
    rows = logits.numel() // V
    l2 = logits.reshape(rows, V)
    loss = torch.empty(rows, dtype=f32, device=logits.device)
    if want_grad and dlogits is None:
        dlogits = torch.empty_like(l2)
    rc = _native.cuda().msb_ce_grad(_p(l2), _p(labels), _p(stats), _p(loss), _p(dlogits) if want_grad else None,
                                    _p(grad_scale), rows, V, l2.stride(0), vocab_start, ignore_index, 1,
                                    int(logits.dtype == f32), _stream())
    _native.check(rc, "ce_grad")
    _count()
    return loss, dlogits


# --------------------------------------------------------------------------------------- optimizers
def _adamw_host(master, m, v, grad, param_lp, hyper, skip):
    """Same arithmetic in torch, for arenas that live in host memory."""
    if skip is not None and int(skip) != 0:
        return
    lr, b1, b2, eps, wd, bc1, bc2, gs = (float(x) for x in hyper[:8])
    g = grad.float() * gs
    m.mul_(b1).add_(g, alpha=1 - b1)
    v.mul_(b2).addcmul_(g, g, value=1 - b2)
    master.mul_(1 - lr * wd).sub_((lr / bc1) * m / (v.sqrt() / (bc2 ** 0.5) + eps))
    if param_lp is not None:
        param_lp.copy_(master)


def adamw_step(master, m, v, grad, param_lp, hyper, skip=None):
    if not master.is_cuda:
        return _adamw_host(master, m, v, grad, param_lp, hyper, skip)
    rc = _native.cuda().msb_adamw(_p(master), _p(m), _p(v), _p(grad), int(grad.dtype == f32), _p(param_lp),
                                  master.numel(), _p(hyper), _p(skip), _stream())
    _native.check(rc, "adamw")
    _count()


def momentum_step(master, accum, grad, param_lp, hyper, skip=None):
    rc = _native.cuda().msb_momentum(_p(master), _p(accum), _p(grad), int(grad.dtype == f32), _p(param_lp),
                                     master.numel(), _p(hyper), _p(skip), _stream())
    _native.check(rc, "momentum")
    _count()


def sumsq_finite(x, out, nonfinite):
    if not x.is_cuda:
        xf = x.float()
        out += (xf * xf).sum()
        if not bool(torch.isfinite(xf).all()):
            nonfinite.fill_(1)
        return
    rc = _native.cuda().msb_sumsq_finite(_p(x), int(x.dtype == f32), x.numel(), _p(out), _p(nonfinite), _stream())
    _native.check(rc, "sumsq_finite")
    _count()


def finalize_grad_scale(sumsq, nonfinite, inv_loss_scale, max_norm, hyper_scale, skip, norm_out=None):
    if not sumsq.is_cuda:
        norm = float(sumsq.reshape(-1)[0]) ** 0.5 * inv_loss_scale
        s = inv_loss_scale * (min(1.0, max_norm / (norm + 1e-6)) if max_norm > 0 else 1.0)
        hyper_scale.fill_(s)
        if skip is not None:
            skip.copy_(nonfinite.reshape(skip.shape))
        if norm_out is not None:
            norm_out.fill_(norm)
        return
    rc = _native.cuda().msb_finalize_grad_scale(_p(sumsq), _p(nonfinite), float(inv_loss_scale), float(max_norm),
                                                _p(hyper_scale), _p(skip), _p(norm_out), _stream())
    _native.check(rc, "finalize_grad_scale")
    _count()


# --------------------------------------------------------------------------------------- embedding / casts
def embedding_fwd(table, ids, vocab_start=0):
    H = table.shape[1]
    out = torch.empty(ids.shape + (H,), dtype=table.dtype, device=table.device)
    rc = _native.cuda().msb_embedding_fwd(_p(table), _p(ids), _p(out), ids.numel(), H, table.shape[0], vocab_start,
                                          _stream())
    _native.check(rc, "embedding_fwd")
    _count()
    return out


def embedding_bwd(dout, ids, dtable_f32, vocab_start=0):
    H = dtable_f32.shape[1]
    rc = _native.cuda().msb_embedding_bwd(_p(dout), _p(ids), _p(dtable_f32), ids.numel(), H, dtable_f32.shape[0],
                                          vocab_start, _stream())
    _native.check(rc, "embedding_bwd")
    _count()


def cast_f32_to_bf16(src, dst, scale=1.0):
    _native.check(_native.cuda().msb_cast_f32_to_bf16(_p(src), _p(dst), src.numel(), float(scale), _stream()), "cast")
    _count()
    return dst


def cast_bf16_to_f32(src, dst, scale=1.0, accumulate=False):
    _native.check(_native.cuda().msb_cast_bf16_to_f32(_p(src), _p(dst), src.numel(), float(scale), int(accumulate),
                                                      _stream()), "cast")
    _count()
    return dst


def add_bf16(a, b, out=None):
    if out is None:
        out = torch.empty_like(a)
    _native.check(_native.cuda().msb_add_bf16(_p(a), _p(b), _p(out), a.numel(), _stream()), "add")
    _count()
    return out
