"""Autograd-aware hot ops backed by the sm_100a kernels (CUDA bf16, and fp16 for the GEMM, norm, activation, RoPE and
attention kernels) with a PyTorch reference path for CPU tensors and other dtypes, so the same model code runs in CPU tests and on the GPU.

Each op is a ``torch.autograd.Function`` whose forward and backward call ``ops.kernels``; weight
gradients are accumulated straight into ``param.main_grad`` (fp32 arena view) when a parameter
has one, which folds micro-batch gradient accumulation into the wgrad GEMM epilogue.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F

from . import kernels as K


def _use_kernel(*tensors, fp16_ok=False):
    """All tensors on a GPU and of one 16-bit type the kernels take: bf16 everywhere, fp16 where the op has an fp16
    build (GEMM, norms, RoPE, SwiGLU, GELU)."""
    ts = [t for t in tensors if t is not None]
    if not ts or not all(t.is_cuda for t in ts):
        return False
    dt = ts[0].dtype
    if dt != torch.bfloat16 and not (fp16_ok and dt == torch.float16):
        return False
    return all(t.dtype == dt for t in ts)


def _plain(t):
    return t.as_subclass(torch.Tensor) if t is not None and type(t) is not torch.Tensor else t


def _producer(param):
    from ..nn.optim import note_grad_producer
    note_grad_producer(param)


def _written(param):
    from ..nn.optim import notify_grad_written
    notify_grad_written(param)


# ------------------------------------------------------------------------------------------ Linear
class _LinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, bias):
        x2 = x.reshape(-1, x.shape[-1])
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        y = K.linear_fwd(x2, w, bias)
        ctx.save_for_backward(x2, w)
        ctx.has_bias = bias is not None
        ctx.x_shape = x.shape
        ctx.w_ref = w
        return y.view(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, w = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            dx = K.linear_dgrad(dy2, w).view(ctx.x_shape)
        if ctx.needs_input_grad[1]:
            mg = getattr(ctx.w_ref, "main_grad", None)
            if mg is not None:
                K.linear_wgrad(dy2, x2, out=mg, accumulate=True)
                ctx.w_ref.grad_ready = True
                from ..nn.optim import notify_grad_written
                notify_grad_written(ctx.w_ref)
            else:
                dw = K.linear_wgrad(dy2, x2, out_dtype=dy2.dtype)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = dy2.float().sum(0).to(dy2.dtype)
        return dx, dw, db


def linear(x, w, bias=None):
    """y = x @ w^T + bias with w stored [out, in]."""
    if _use_kernel(x, w, bias, fp16_ok=True) and x.shape[-1] % 8 == 0 and w.shape[0] % 8 == 0:
        _producer(w)
        return _LinearFn.apply(x, w, bias)
    return F.linear(x, w, bias)


class _MatMulFn(torch.autograd.Function):
    """General 2-D/3-D 16-bit matmul with transpose flags (MatMul / BatchMatMul primitives).  A 2-D second operand
    that owns an fp32 gradient accumulator (``main_grad``, a parameter of an arena optimizer) gets its gradient added
    there by the wgrad GEMM's epilogue, like ``linear``: no 16-bit ``.grad`` tensor, no separate accumulation pass per
    micro-batch."""

    @staticmethod
    def forward(ctx, a, b, ta, tb):
        # logical C = op(a) @ op(b); kernel wants A=[M,K] (or stored [K,M]) and B as [N,K] (or stored [K,N])
        ctx.save_for_backward(a, b)
        ctx.ta, ctx.tb = ta, tb
        ctx.b_ref = b
        return K.gemm(a, b, a_mn=ta, b_mn=not tb)

    @staticmethod
    def backward(ctx, dc):
        a, b = ctx.saved_tensors
        ta, tb = ctx.ta, ctx.tb
        dc = dc.contiguous()
        da = db = None
        if ctx.needs_input_grad[0]:
            if not ta:   # da[M,K] = dc[M,N] @ op(b)^T ; B' logical [K_out, N_red]: b stored [K,N] is K-major
                da = K.gemm(dc, b, b_mn=tb)
            else:        # a stored [K,M]: da[K,M] = op(b) @ dc^T -> A' logical [K_out, N_red], B' = dc [M, N_red]
                da = K.gemm(b, dc, a_mn=tb)
        if ctx.needs_input_grad[1]:
            mg = getattr(ctx.b_ref, "main_grad", None)
            acc = mg is not None and b.dim() == 2 and tuple(mg.shape) == tuple(b.shape)
            kw = dict(out=mg, accumulate=True) if acc else {}
            if not tb:   # b stored [K,N]: db[K,N] = op(a)^T @ dc -> A logical [K, M(red)], B logical [N, M(red)]
                db = K.gemm(a, dc, a_mn=not ta, b_mn=True, **kw)
            else:        # b stored [N,K]: db[N,K] = dc^T @ op(a) -> A logical [N, M(red)], B logical [K, M(red)]
                db = K.gemm(dc, a, a_mn=True, b_mn=not ta, **kw)
            if acc:
                db = None
                ctx.b_ref.grad_ready = True
                _written(ctx.b_ref)
        return da, db, None, None


def matmul(a, b, transpose_a=False, transpose_b=False):
    if _use_kernel(a, b, fp16_ok=True) and a.dim() == b.dim() and a.dim() in (2, 3) and a.is_contiguous() and b.is_contiguous() \
            and all(s % 8 == 0 for s in a.shape[-2:]) and all(s % 8 == 0 for s in b.shape[-2:]):
        if b.dim() == 2 and getattr(b, "main_grad", None) is not None:
            _producer(b)
        return _MatMulFn.apply(a, b, bool(transpose_a), bool(transpose_b))
    aa = a.transpose(-1, -2) if transpose_a else a
    bb = b.transpose(-1, -2) if transpose_b else b
    return torch.matmul(aa, bb)


# ------------------------------------------------------------------------------------------ norms
class _RmsNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, eps, residual):
        y, rstd, xsum = K.rmsnorm_fwd(x.contiguous(), w, eps, residual.contiguous() if residual is not None else None)
        ctx.save_for_backward(xsum, w, rstd)
        ctx.w_ref = w
        ctx.has_res = residual is not None
        rstd_out = rstd.view_as(rstd)
        ctx.mark_non_differentiable(rstd_out)
        if residual is not None:
            return y, xsum, rstd_out
        dummy = x.new_empty(0)
        ctx.mark_non_differentiable(dummy)
        return y, dummy, rstd_out

    @staticmethod
    def backward(ctx, dy, dxsum, _drstd):
        xsum, w, rstd = ctx.saved_tensors
        mg = getattr(ctx.w_ref, "main_grad", None)
        dres = dxsum.contiguous() if (ctx.has_res and dxsum is not None) else None
        dx, dw = K.rmsnorm_bwd(dy.contiguous(), xsum, w, rstd, dresidual=dres, dw_out=mg, accumulate=mg is not None)
        if mg is not None:
            dw = None
            _written(ctx.w_ref)
        if ctx.has_res:
            return dx, dw, None, dx
        return dx, dw, None, None


def rms_norm(x, w, eps=1e-6, residual=None, with_rstd=False):
    """Returns (y, stream) where stream = x + residual (or x).  y = stream * rsqrt(mean(stream^2)+eps) * w.
    ``with_rstd`` appends the per-row reciprocal RMS (fp32, shape [..., 1])."""
    if _use_kernel(x, w, residual, fp16_ok=True) and x.shape[-1] % 8 == 0 and x.shape[-1] <= 16384:
        _producer(w)
        y, stream, rstd = _RmsNormFn.apply(x, w, eps, residual)
        stream = stream if residual is not None else x
        return (y, stream, rstd.reshape(*x.shape[:-1], 1)) if with_rstd else (y, stream)
    stream = x if residual is None else x + residual
    xf = stream.float()
    rstd = torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    y = (xf * rstd).to(x.dtype) * w
    return (y, stream, rstd) if with_rstd else (y, stream)


class _LayerNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, b, eps):
        y, mean, rstd = K.layernorm_fwd(x.contiguous(), w, b, eps)
        ctx.save_for_backward(x, w, mean, rstd)
        ctx.w_ref, ctx.b_ref = w, b
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w, mean, rstd = ctx.saved_tensors
        mgw = getattr(ctx.w_ref, "main_grad", None)
        mgb = getattr(ctx.b_ref, "main_grad", None) if ctx.b_ref is not None else None
        if mgw is not None and (ctx.b_ref is None or mgb is not None):
            dx, _, _ = K.layernorm_bwd(dy.contiguous(), x.contiguous(), w, mean, rstd, dw_out=mgw, db_out=mgb,
                                       accumulate=True)
            _written(ctx.w_ref)
            if ctx.b_ref is not None:
                _written(ctx.b_ref)
            return dx, None, None, None
        dx, dw, db = K.layernorm_bwd(dy.contiguous(), x.contiguous(), w, mean, rstd, has_bias=ctx.b_ref is not None)
        return dx, dw, db, None


def layer_norm(x, w, b, eps=1e-5):
    if _use_kernel(x, w, b, fp16_ok=True) and x.shape[-1] % 8 == 0 and x.shape[-1] <= 16384:
        _producer(w)
        if b is not None:
            _producer(b)
        return _LayerNormFn.apply(x, w, b, eps)
    return F.layer_norm(x, (x.shape[-1],), w, b, eps)


# ------------------------------------------------------------------------------------------ activations
class _SwiGLUFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gu):
        ctx.save_for_backward(gu)
        return K.swiglu_fwd(gu)

    @staticmethod
    def backward(ctx, dout):
        (gu,) = ctx.saved_tensors
        return K.swiglu_bwd(gu, dout.contiguous())


def swiglu(gu):
    """silu(gu[..., :F]) * gu[..., F:]"""
    if _use_kernel(gu, fp16_ok=True) and gu.is_contiguous() and (gu.shape[-1] // 2) % 8 == 0:
        return _SwiGLUFn.apply(gu)
    f = gu.shape[-1] // 2
    return F.silu(gu[..., :f]) * gu[..., f:]


class _GeluFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, bias):
        ctx.save_for_backward(x, bias)
        ctx.b_ref = bias
        return K.gelu_fwd(x, bias)

    @staticmethod
    def backward(ctx, dy):
        x, bias = ctx.saved_tensors
        dx = K.gelu_bwd(x, dy.contiguous(), bias)
        db = None
        if bias is not None and ctx.needs_input_grad[1]:
            db = dx.reshape(-1, dx.shape[-1]).float().sum(0).to(dx.dtype)
        return dx, db


def gelu_tanh(x, bias=None):
    if _use_kernel(x, bias, fp16_ok=True) and x.is_contiguous() and x.shape[-1] % 8 == 0:
        return _GeluFn.apply(x, bias)
    return F.gelu(x if bias is None else x + bias, approximate="tanh")


# ------------------------------------------------------------------------------------------ RoPE
class _RopeFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, cos, sin, heads, head_dim, seq):
        ctx.save_for_backward(cos, sin)
        ctx.meta = (heads, head_dim, seq)
        out = x.clone()
        K.rope_(out, cos, sin, heads, head_dim, seq)
        return out

    @staticmethod
    def backward(ctx, dy):
        cos, sin = ctx.saved_tensors
        heads, head_dim, seq = ctx.meta
        dx = dy.clone()
        K.rope_(dx, cos, sin, heads, head_dim, seq, backward=True)
        return dx, None, None, None, None, None


def rope_tables(seq, head_dim, theta=10000.0, device="cpu"):
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, device=device, dtype=torch.float32) / head_dim))
    fr = torch.outer(torch.arange(seq, device=device, dtype=torch.float32), inv)
    return fr.cos().contiguous(), fr.sin().contiguous()


def rope(x, cos, sin, heads, head_dim, seq):
    """Rotate-half RoPE on x[..., seq, heads*head_dim] (token-major); cos/sin fp32 [seq, head_dim/2]."""
    if _use_kernel(x, fp16_ok=True) and x.is_contiguous() and head_dim % 16 == 0:
        return _RopeFn.apply(x, cos, sin, heads, head_dim, seq)
    shp = x.shape
    xv = x.reshape(-1, seq, heads, head_dim).float()
    c = cos[None, :, None, :]
    s = sin[None, :, None, :]
    a, b = xv[..., : head_dim // 2], xv[..., head_dim // 2:]
    out = torch.cat([a * c - b * s, b * c + a * s], -1)
    return out.to(x.dtype).reshape(shp)


# ------------------------------------------------------------------------------------------ cross entropy
class _SoftmaxCEFn(torch.autograd.Function):
    """Mean cross entropy over non-ignored rows; gradient written in one pass (softmax - onehot)."""

    @staticmethod
    def forward(ctx, logits, labels, ignore_index):
        labels = labels.reshape(-1).to(torch.int32)
        stats = K.ce_stats(logits, labels)
        loss_rows, _ = K.ce_loss_grad(logits, labels, stats, None, ignore_index=ignore_index, want_grad=False)
        nvalid = (labels != ignore_index).sum().clamp(min=1).float()
        ctx.save_for_backward(logits, labels, stats, nvalid)
        ctx.ignore_index = ignore_index
        return loss_rows.sum() / nvalid

    @staticmethod
    def backward(ctx, dloss):
        logits, labels, stats, nvalid = ctx.saved_tensors
        scale = (dloss.float() / nvalid).reshape(1).contiguous()
        _, dl = K.ce_loss_grad(logits, labels, stats, scale, ignore_index=ctx.ignore_index, want_grad=True)
        return dl.view(logits.shape), None, None


def softmax_cross_entropy(logits, labels, ignore_index=-100):
    """Mean token cross entropy.  logits [..., V] (bf16 or fp32, CUDA) and integer labels [...]."""
    if logits.is_cuda and logits.dtype in (torch.bfloat16, torch.float32) and logits.is_contiguous():
        return _SoftmaxCEFn.apply(logits, labels, ignore_index)
    return F.cross_entropy(logits.reshape(-1, logits.shape[-1]).float(), labels.reshape(-1).long(),
                           ignore_index=ignore_index)


# ------------------------------------------------------------------------------------------ embedding
class _EmbeddingFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, table, ids, vocab_start):
        ids32 = ids.to(torch.int32).contiguous()
        ctx.save_for_backward(ids32)
        ctx.t_ref = table
        ctx.vocab_start = vocab_start
        return K.embedding_fwd(table, ids32, vocab_start)

    @staticmethod
    def backward(ctx, dout):
        (ids32,) = ctx.saved_tensors
        t = ctx.t_ref
        mg = getattr(t, "main_grad", None)
        if mg is not None:
            K.embedding_bwd(dout.contiguous(), ids32, mg.view(t.shape), ctx.vocab_start)
            _written(t)
            return None, None, None
        acc = torch.zeros(t.shape, dtype=torch.float32, device=t.device)
        K.embedding_bwd(dout.contiguous(), ids32, acc, ctx.vocab_start)
        return acc.to(t.dtype), None, None


def embedding(table, ids, vocab_start=0):
    if _use_kernel(table) and table.shape[1] % 8 == 0:
        _producer(table)
        return _EmbeddingFn.apply(table, ids, vocab_start)
    idx = ids.long() - vocab_start
    mask = (idx >= 0) & (idx < table.shape[0])
    return F.embedding(idx.clamp(0, table.shape[0] - 1), table) * mask.unsqueeze(-1).to(table.dtype)


# ------------------------------------------------------------------------------------------ attention
def flash_attention(q, k, v, causal=True, scale=None):
    """Scaled-dot-product attention on [B, S, H, D] tensors (kv heads may divide q heads)."""
    from . import attention as _attn
    return _attn.flash_attention(q, k, v, causal=causal, scale=scale)


# ------------------------------------------------------------------------------------------ packed QKV attention
class _QkvRopeAttnFn(torch.autograd.Function):
    """RoPE + causal attention straight on the packed output of a fused QKV projection.

    ``qkv`` [tokens, (H + 2 Hk) * D] is rotated in place (q and k column blocks), the attention kernel reads q, k, v
    as strided views of it, and the backward kernels write dq, dk, dv into the column blocks of one packed gradient,
    which is then un-rotated in place: no slicing copies, no concatenation."""

    @staticmethod
    def forward(ctx, qkv, cos, sin, batch, seq, heads, kv_heads, d, causal, scale):
        from . import flash_attn_kernel as FK
        hd, kd = heads * d, kv_heads * d
        K.rope_(qkv[:, :hd + kd], cos, sin, heads + kv_heads, d, seq)
        q = qkv[:, :hd].view(batch, seq, heads, d)
        k = qkv[:, hd:hd + kd].view(batch, seq, kv_heads, d)
        v = qkv[:, hd + kd:].view(batch, seq, kv_heads, d)
        o, lse, _, _, _ = FK.fwd(q, k, v, causal, scale)
        ctx.save_for_backward(qkv, o, lse, cos, sin)
        ctx.meta = (batch, seq, heads, kv_heads, d, causal, scale)
        return o

    @staticmethod
    def backward(ctx, do):
        from . import flash_attn_kernel as FK
        qkv, o, lse, cos, sin = ctx.saved_tensors
        batch, seq, heads, kv_heads, d, causal, scale = ctx.meta
        hd, kd = heads * d, kv_heads * d
        q = qkv[:, :hd].view(batch, seq, heads, d)
        k = qkv[:, hd:hd + kd].view(batch, seq, kv_heads, d)
        v = qkv[:, hd + kd:].view(batch, seq, kv_heads, d)
        dqkv = torch.empty_like(qkv)
        FK.bwd_into(do, q, k, v, o, lse, causal, scale, dqkv[:, :hd], dqkv[:, hd:hd + kd], dqkv[:, hd + kd:],
                    qkv.shape[1])
        K.rope_(dqkv[:, :hd + kd], cos, sin, heads + kv_heads, d, seq, backward=True)
        return dqkv, None, None, None, None, None, None, None, None, None


def qkv_rope_attention(qkv, cos, sin, batch, seq, heads, kv_heads, head_dim, causal=True, scale=None):
    """Attention output [batch, seq, heads, head_dim] from the packed projection ``qkv`` [batch*seq, (H+2Hk)*D]
    (q heads, then k heads, then v heads).  ``qkv`` is consumed: the kernel path rotates it in place."""
    import math
    from . import flash_attn_kernel as FK
    scale = scale if scale is not None else 1.0 / math.sqrt(head_dim)
    hd, kd = heads * head_dim, kv_heads * head_dim
    if (_use_kernel(qkv, fp16_ok=True) and qkv.is_contiguous() and head_dim == 128
            and seq % 128 == 0 and heads == kv_heads and FK.available() and FK.has_strided_bwd()):
        return _QkvRopeAttnFn.apply(qkv, cos, sin, batch, seq, heads, kv_heads, head_dim, bool(causal), float(scale))
    qk = rope(qkv[:, :hd + kd].contiguous(), cos, sin, heads + kv_heads, head_dim, seq)
    q = qk[:, :hd].reshape(batch, seq, heads, head_dim)
    k = qk[:, hd:].reshape(batch, seq, kv_heads, head_dim)
    v = qkv[:, hd + kd:].reshape(batch, seq, kv_heads, head_dim)
    return flash_attention(q, k, v, causal=causal, scale=scale)
