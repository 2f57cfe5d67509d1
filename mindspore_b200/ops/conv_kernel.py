"""Convolution + BatchNorm + ReLU on the sm_100a kernels (``csrc/cuda/conv_sm100.cu``, ``bn_pool.cu``).

Tensors keep the NCHW *shape* of the public API but live in channels-last memory, so every kernel sees NHWC.  The
fused unit is ``conv_bn_act``: implicit-GEMM convolution whose epilogue also accumulates the BatchNorm statistics,
a finalize kernel, and one elementwise pass ``relu(x * scale + shift (+ residual))``; backward is two passes for
BatchNorm (reduce, apply) followed by the data-gradient and weight-gradient implicit GEMMs.

Parity: what the reference gets from cuDNN through Conv2D / Conv2DBackpropInput / Conv2DBackpropFilter
(plugin/device/gpu/kernel/nn/conv2d_gpu_kernel.h and the two grad kernels), BatchNorm(+Grad) with fused activation
(batch_norm_gpu_kernel.cc:62, batch_norm_grad_gpu_kernel.cc), MaxPool / AvgPool (pooling_gpu_kernel.h)."""
from __future__ import annotations

import ctypes

import torch

from .. import _native
from . import kernels as K
from .kernels import _count, _p, _stream

_P, _I, _L, _F = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float
_native.register_cuda_signature("msb_conv_fwd", _I, [_P, _P, _P, _P] + [_I] * 13 + [_L, _L, _I, _P])
_native.register_cuda_signature("msb_conv_wgrad", _I, [_P, _P, _P] + [_I] * 12 + [_L, _L, _I, _P])
_native.register_cuda_signature("msb_im2col_nhwc", _I, [_P, _P] + [_I] * 12 + [_P])
_native.register_cuda_signature("msb_channel_stats", _I, [_P, _P, _L, _I, _P])
_native.register_cuda_signature("msb_bn_finalize", _I, [_P] * 9 + [_I, _F, _F, _F, _I, _P])
_native.register_cuda_signature("msb_bn_apply", _I, [_P, _P, _P, _P, _P, _L, _I, _I, _P])
_native.register_cuda_signature("msb_bn_bwd_reduce", _I, [_P, _P, _P, _P, _P, _P, _L, _I, _I, _P])
_native.register_cuda_signature("msb_bn_bwd_apply", _I, [_P] * 10 + [_L, _I, _I, _P])
_native.register_cuda_signature("msb_maxpool3x3s2", _I, [_P, _P, _P, _P, _I, _I, _I, _I, _I, _P])
_native.register_cuda_signature("msb_global_avgpool", _I, [_P, _P, _I, _I, _I, _I, _P])

CL = torch.channels_last


def _notify(param):
    from ..nn.optim import notify_grad_written
    notify_grad_written(param)


def _producer(*params):
    from ..nn.optim import note_grad_producer
    for p in params:
        if p is not None:
            note_grad_producer(p)


def available():
    return torch.cuda.is_available() and _native.cuda() is not None


def supports(x, w, group=1, dilation=(1, 1)):
    return (available() and x.is_cuda and x.dtype in (torch.bfloat16, torch.float16) and x.dim() == 4 and group == 1
            and tuple(dilation) == (1, 1) and w.shape[0] % 8 == 0 and w.shape[2] * w.shape[3] <= 49)


def _nhwc(x):
    """The same NCHW-shaped tensor in channels-last memory (no copy when it already is)."""
    return x if x.is_contiguous(memory_format=CL) else x.contiguous(memory_format=CL)


def _empty(n, c, h, w, device, dtype=torch.bfloat16):
    return torch.empty((n, c, h, w), dtype=dtype, device=device, memory_format=CL)


def _out_size(h, k, stride, pad_lo, pad_hi):
    return (h + pad_lo + pad_hi - k) // stride + 1


def _w_krsc(w):
    """[Cout, Cin, R, S] parameter -> [Cout, R, S, Cin] contiguous (what the kernels index)."""
    return w.permute(0, 2, 3, 1).contiguous()


# ------------------------------------------------------------------------------------------------ raw launches
def conv_fwd_raw(x, w_krsc, stride, pad_h, pad_w, ho, wo, stats=None, flip=False):
    """x NHWC-memory [N, Cin, H, W]; w_krsc [Cout, R, S, Cin] -> y [N, Cout, ho, wo] (channels-last)."""
    n, cin, h, w_ = x.shape
    cout, r, s, _ = w_krsc.shape
    y = _empty(n, cout, ho, wo, x.device, x.dtype)
    rc = K._fn("msb_conv_fwd", x)(_p(x), _p(w_krsc), _p(y), _p(stats), n, h, w_, cin, cout, r, s, stride, pad_h,
                                     pad_w, int(flip), ho, wo, cin, cout, 0, _stream())
    _native.check(rc, "conv_fwd")
    _count()
    return y


def conv_wgrad_raw(x, dy, r, s, stride, pad_h, pad_w):
    """dW [Cout, R, S, Cin] fp32 from x [N, Cin, H, W] and dy [N, Cout, Ho, Wo] (both channels-last)."""
    n, cin, h, w_ = x.shape
    _, cout, ho, wo = dy.shape
    dw = torch.empty((cout, r, s, cin), dtype=torch.float32, device=x.device)
    rc = K._fn("msb_conv_wgrad", x)(_p(x), _p(dy), _p(dw), n, h, w_, cin, cout, r, s, stride, pad_h, pad_w, ho, wo,
                                       cin, cout, 0, _stream())
    _native.check(rc, "conv_wgrad")
    _count(2)
    return dw


def _im2col(x, r, s, stride, pad_h, pad_w, ho, wo):
    n, cin, h, w_ = x.shape
    kpad = (r * s * cin + 63) // 64 * 64
    col = torch.empty((n * ho * wo, kpad), dtype=x.dtype, device=x.device)
    rc = K._fn("msb_im2col_nhwc", x)(_p(x), _p(col), n, h, w_, cin, r, s, stride, pad_h, pad_w, ho, wo, kpad,
                                        _stream())
    _native.check(rc, "im2col")
    _count()
    return col, kpad


def _split_k(rows):
    b = 1
    while b < 256 and rows % (b * 2) == 0 and rows // (b * 2) >= 4096:
        b *= 2
    return b


class _ConvFn(torch.autograd.Function):
    """Convolution alone (weights [Cout, Cin, R, S], symmetric padding); returns y and, when asked, the fp32
    [2*Cout] sum / sum-of-squares of y."""

    @staticmethod
    def forward(ctx, x, w, stride, pad_h, pad_w, want_stats):
        x = _nhwc(x)
        n, cin, h, w_ = x.shape
        cout, _, r, s = w.shape
        ho, wo = _out_size(h, r, stride, pad_h, pad_h), _out_size(w_, s, stride, pad_w, pad_w)
        wk = _w_krsc(w)
        stats = torch.zeros(2 * cout, dtype=torch.float32, device=x.device) if want_stats else None
        ctx.small = cin % 64 != 0
        if ctx.small:
            col, kpad = _im2col(x, r, s, stride, pad_h, pad_w, ho, wo)
            wmat = torch.zeros((cout, kpad), dtype=x.dtype, device=x.device)
            wmat[:, :r * s * cin] = wk.reshape(cout, -1)
            y2 = K.gemm(col, wmat)                                       # [pixels, Cout]
            y = y2.view(n, ho, wo, cout).permute(0, 3, 1, 2)
            if want_stats:
                _native.check(K._fn("msb_channel_stats", y2)(_p(y2), _p(stats), y2.shape[0], cout, _stream()),
                              "channel_stats")
                _count()
        else:
            y = conv_fwd_raw(x, wk, stride, pad_h, pad_w, ho, wo, stats)
        ctx.save_for_backward(x, w)
        ctx.col = (col, kpad) if ctx.small else None      # the patch matrix is kept for the weight gradient
        ctx.geom = (stride, pad_h, pad_w, ho, wo)
        if want_stats:
            ctx.mark_non_differentiable(stats)
            return y, stats
        return y, None

    @staticmethod
    def backward(ctx, dy, _dstats):
        x, w = ctx.saved_tensors
        stride, pad_h, pad_w, ho, wo = ctx.geom
        n, cin, h, w_ = x.shape
        cout, _, r, s = w.shape
        dy = _nhwc(dy)
        dx = dw = None
        if ctx.needs_input_grad[1]:
            if ctx.small:
                col, kpad = ctx.col
                rows = col.shape[0]
                b = _split_k(rows)
                dy2 = dy.permute(0, 2, 3, 1).reshape(b, rows // b, cout)
                part = K.gemm(dy2, col.view(b, rows // b, kpad), a_mn=True, b_mn=True, out_dtype=torch.float32)
                dwk = part.sum(0)[:, :r * s * cin].reshape(cout, r, s, cin)
            else:
                dwk = conv_wgrad_raw(x, dy, r, s, stride, pad_h, pad_w)
            dw = dwk.permute(0, 3, 1, 2)
            mg = getattr(w, "main_grad", None)
            if mg is not None:
                mg.add_(dw)
                dw = None
                _notify(w)
            else:
                dw = dw.to(w.dtype)
        if ctx.needs_input_grad[0]:
            if ctx.small:
                raise NotImplementedError("data gradient of a convolution with fewer than 64 input channels on the "
                                          "kernel path (only a first layer, whose input needs no gradient, is "
                                          "expected)")
            wt = w.permute(1, 2, 3, 0).contiguous()                      # [Cin, R, S, Cout]
            if cout % 64:                                                # the box loads take 64 channels at a time
                extra = 64 - cout % 64
                wt = torch.nn.functional.pad(wt, (0, extra))
                dy = _nhwc(torch.nn.functional.pad(dy, (0, 0, 0, 0, 0, extra)))
                cout += extra
            if stride == 1:
                dx = conv_fwd_raw(dy, wt, 1, pad_h, pad_w, h, w_, None, flip=True)
            elif r == 1 and s == 1:
                sub = conv_fwd_raw(dy, wt, 1, 0, 0, ho, wo, None, flip=True)
                dx = _empty(n, cin, h, w_, dy.device, dy.dtype).zero_()
                dx[:, :, 0:2 * ho:2, 0:2 * wo:2] = sub
            else:
                hz, wz = max(h, 2 * (ho - 1) + 1), max(w_, 2 * (wo - 1) + 1)
                dyz = _empty(n, cout, hz, wz, dy.device, dy.dtype).zero_()
                dyz[:, :, 0:2 * ho:2, 0:2 * wo:2] = dy
                dx = conv_fwd_raw(dyz, wt, 1, pad_h, pad_w, h, w_, None, flip=True)
        return dx, dw, None, None, None, None


def conv2d(x, w, stride, pads, dilation=(1, 1), bias=None):
    """Entry used by ``ops.conv.conv2d``: pads = (top, bottom, left, right)."""
    top, bottom, left, right = pads
    sh, sw = stride
    if sh != sw or sh not in (1, 2) or top != bottom or left != right:
        x = torch.nn.functional.pad(x, (left, right, top, bottom))
        return torch.nn.functional.conv2d(x, w, bias, stride, 0, dilation)
    _producer(w)
    y, _ = _ConvFn.apply(x, w.to(x.dtype) if w.dtype != x.dtype else w, sh, top, left, False)
    if bias is not None:
        y = y + bias.view(1, -1, 1, 1)
    return y


# ------------------------------------------------------------------------------------------------ BatchNorm (+ ReLU)
class _BnActFn(torch.autograd.Function):
    """y = relu(bn(x) (+ residual)) in training mode from precomputed channel sums of x.

    Inputs: x (conv output, channels-last bf16), stats fp32 [2C] (sum, sum of squares over N*H*W), gamma, beta
    (fp32 [C]), residual or None.  ``moving`` = (moving_mean, moving_var, momentum) is updated in place."""

    @staticmethod
    def forward(ctx, x, stats, gamma, beta, residual, relu, eps, moving):
        n, c, h, w = x.shape
        rows = n * h * w
        dev = x.device
        scale = torch.empty(c, dtype=torch.float32, device=dev)
        shift = torch.empty(c, dtype=torch.float32, device=dev)
        mean = torch.empty(c, dtype=torch.float32, device=dev)
        rstd = torch.empty(c, dtype=torch.float32, device=dev)
        mm, mv, momentum = moving
        g32, b32 = gamma.float().contiguous(), beta.float().contiguous()
        lib = _native.cuda()
        _native.check(lib.msb_bn_finalize(_p(stats), _p(g32), _p(b32), _p(mm), _p(mv), _p(scale), _p(shift), _p(mean),
                                          _p(rstd), c, float(rows), float(momentum), float(eps), 1, _stream()),
                      "bn_finalize")
        y = torch.empty_like(x, memory_format=CL)
        res = _nhwc(residual) if residual is not None else None
        _native.check(K._fn("msb_bn_apply", x)(_p(x), _p(scale), _p(shift), _p(res), _p(y), rows, c, int(relu), _stream()),
                      "bn_apply")
        _count(2)
        ctx.save_for_backward(x, y, g32, mean, rstd)
        ctx.relu, ctx.has_res = relu, residual is not None
        ctx.gamma_ref, ctx.beta_ref = gamma, beta
        return y

    @staticmethod
    def backward(ctx, dy):
        x, y, g32, mean, rstd = ctx.saved_tensors
        n, c, h, w = x.shape
        rows = n * h * w
        dy = _nhwc(dy)
        sums = torch.zeros(2 * c, dtype=torch.float32, device=x.device)
        lib = _native.cuda()
        _native.check(K._fn("msb_bn_bwd_reduce", x)(_p(dy), _p(x), _p(y), _p(mean), _p(rstd), _p(sums), rows, c,
                                            int(ctx.relu), _stream()), "bn_bwd_reduce")
        dx = torch.empty_like(x, memory_format=CL)
        dres = torch.empty_like(x, memory_format=CL) if ctx.has_res else None
        coef = torch.empty(3 * c, dtype=torch.float32, device=x.device)
        _native.check(K._fn("msb_bn_bwd_apply", x)(_p(dy), _p(x), _p(y), _p(g32), _p(mean), _p(rstd), _p(sums), _p(coef),
                                           _p(dx), _p(dres), rows, c, int(ctx.relu), _stream()), "bn_bwd_apply")
        _count(3)
        dgamma, dbeta = sums[c:], sums[:c]
        out_g = out_b = None
        for ref, g, slot in ((ctx.gamma_ref, dgamma, 0), (ctx.beta_ref, dbeta, 1)):
            mg = getattr(ref, "main_grad", None)
            if mg is not None:
                mg.add_(g)
                _notify(ref)
            elif slot == 0:
                out_g = g.to(ref.dtype)
            else:
                out_b = g.to(ref.dtype)
        return dx, None, out_g, out_b, dres, None, None, None


def conv_bn_act(x, w, gamma, beta, moving_mean, moving_var, stride=1, pad=0, relu=True, residual=None, eps=1e-5,
                momentum=0.9):
    """Training-mode Conv2d -> BatchNorm2d -> (+ residual) -> ReLU on the kernel path.  ``momentum`` is the weight
    of the old moving statistics (nn.BatchNorm2d convention)."""
    wb = w if w.dtype == x.dtype else w.to(x.dtype)
    _producer(wb, gamma, beta)
    y, stats = _ConvFn.apply(x, wb, stride, pad, pad, True)
    return _BnActFn.apply(y, stats, gamma, beta, residual, relu, eps, (moving_mean, moving_var, momentum))


def bn_act_inference(x, gamma, beta, moving_mean, moving_var, relu=True, residual=None, eps=1e-5):
    x = _nhwc(x)
    n, c, h, w = x.shape
    dev = x.device
    scale = torch.empty(c, dtype=torch.float32, device=dev)
    shift = torch.empty(c, dtype=torch.float32, device=dev)
    lib = _native.cuda()
    _native.check(lib.msb_bn_finalize(None, _p(gamma.float().contiguous()), _p(beta.float().contiguous()),
                                      _p(moving_mean), _p(moving_var), _p(scale), _p(shift), None, None, c, 1.0, 0.0,
                                      float(eps), 0, _stream()), "bn_finalize")
    y = torch.empty_like(x, memory_format=CL)
    res = _nhwc(residual) if residual is not None else None
    _native.check(K._fn("msb_bn_apply", x)(_p(x), _p(scale), _p(shift), _p(res), _p(y), n * h * w, c, int(relu), _stream()),
                  "bn_apply")
    _count(2)
    return y


# ------------------------------------------------------------------------------------------------ pooling
class _MaxPool3x3s2Fn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        x = _nhwc(x)
        n, c, h, w = x.shape
        ho, wo = (h - 1) // 2 + 1, (w - 1) // 2 + 1
        y = _empty(n, c, ho, wo, x.device)
        idx = torch.empty(n * ho * wo * c, dtype=torch.uint8, device=x.device)
        _native.check(K._fn("msb_maxpool3x3s2", x)(_p(x), None, _p(y), _p(idx), n, h, w, c, 0, _stream()),
                      "maxpool")
        _count()
        ctx.save_for_backward(idx)
        ctx.shape = (n, c, h, w)
        return y

    @staticmethod
    def backward(ctx, dy):
        (idx,) = ctx.saved_tensors
        n, c, h, w = ctx.shape
        dx = _empty(n, c, h, w, dy.device, dy.dtype)
        _native.check(K._fn("msb_maxpool3x3s2", dy)(None, _p(_nhwc(dy)), _p(dx), _p(idx), n, h, w, c, 1, _stream()),
                      "maxpool_bwd")
        _count()
        return dx


class _GlobalAvgPoolFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        x = _nhwc(x)
        n, c, h, w = x.shape
        y = torch.empty((n, c), dtype=x.dtype, device=x.device)
        _native.check(K._fn("msb_global_avgpool", x)(_p(x), _p(y), n, h * w, c, 0, _stream()), "avgpool")
        _count()
        ctx.shape = (n, c, h, w)
        return y

    @staticmethod
    def backward(ctx, dy):
        n, c, h, w = ctx.shape
        dx = _empty(n, c, h, w, dy.device, dy.dtype)
        _native.check(K._fn("msb_global_avgpool", dy)(_p(dy.contiguous()), _p(dx), n, h * w, c, 1, _stream()),
                      "avgpool_bwd")
        _count()
        return dx


def maxpool3x3s2(x):
    return _MaxPool3x3s2Fn.apply(x)


def global_avgpool(x):
    return _GlobalAvgPoolFn.apply(x)


def batch_norm_train(x, gamma, beta, moving_mean, moving_var, keep, eps, relu=False, residual=None):
    """Stand-alone training-mode BatchNorm2d (statistics by a reduction kernel instead of a convolution epilogue).
    ``keep`` is the weight of the old moving statistics."""
    x = _nhwc(x)
    n, c, h, w = x.shape
    stats = torch.zeros(2 * c, dtype=torch.float32, device=x.device)
    _native.check(K._fn("msb_channel_stats", x)(_p(x), _p(stats), n * h * w, c, _stream()), "channel_stats")
    _count()
    mm = moving_mean.detach().as_subclass(torch.Tensor)
    mv = moving_var.detach().as_subclass(torch.Tensor)
    _producer(gamma, beta)
    return _BnActFn.apply(x, stats, gamma, beta, residual, relu, eps, (mm, mv, keep))
