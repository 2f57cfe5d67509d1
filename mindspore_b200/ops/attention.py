"""Attention entry point.  CUDA bf16 inputs with head_dim 128 or 64 run the tcgen05 FlashAttention kernels
(``csrc/cuda/flash_attn_sm100.cu``); everything else (CPU tests, fp32, odd head sizes) evaluates
the same math with PyTorch.

Parity: the FlashAttentionScore primitive (mindspore/core/ops/ops_def/flash_attention_score_op.yaml),
which has no GPU kernel in the reference.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F

_impl = None


def _kernel_impl():
    global _impl
    if _impl is None:
        try:
            from . import flash_attn_kernel as fk
            _impl = fk if fk.available() else False
        except ImportError:
            _impl = False
    return _impl


def reference_attention(q, k, v, causal=True, scale=None):
    """[B, S, H, D] -> [B, S, H, D]; fp32 softmax; kv heads are repeated to match q heads."""
    B, S, H, D = q.shape
    Hk = k.shape[2]
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    qt, kt, vt = (t.permute(0, 2, 1, 3) for t in (q, k, v))
    if Hk != H:
        kt = kt.repeat_interleave(H // Hk, dim=1)
        vt = vt.repeat_interleave(H // Hk, dim=1)
    out = F.scaled_dot_product_attention(qt, kt, vt, is_causal=causal, scale=scale)
    return out.permute(0, 2, 1, 3).contiguous()


def flash_attention(q, k, v, causal=True, scale=None):
    impl = _kernel_impl()
    if impl and impl.supports(q, k, v):
        return impl.flash_attention(q, k, v, causal, scale)
    return reference_attention(q, k, v, causal, scale)
