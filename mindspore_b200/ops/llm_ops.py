"""Fused decoder primitives: the units a Llama / GPT block is written in when every op between two MatMuls is one
kernel.  Each has a distributed OperatorInfo (``parallel/operator_info.py``), so a block built from them plus
``MatMul.shard(...)`` runs under ``semi_auto_parallel`` exactly like the reference's composition of small ops.

* ``AddRmsNorm(epsilon)``       : (x, residual, gamma) -> (rms_norm(x + residual) * gamma, x + residual); the
  residual stream is carried unnormalised, the add is part of the norm kernel (forward and backward).
* ``SwiGLU(groups)``            : silu(gate) * up on a packed ``[.., 2F]`` projection.
* ``RotaryFlashAttention(...)`` : RoPE + causal FlashAttention straight on the packed QKV projection
  ``[tokens, (H + 2 Hk) * D]``; q / k / v are read as strided views, the gradient is written packed.

``groups`` describes the packing of the last dim.  With ``groups = g`` the packed dim is ``g`` consecutive blocks,
block i holding ``[gate_i, up_i]`` (or ``[q_i, k_i, v_i]``) of the i-th 1/g of the features (heads).  A model-parallel
layer sets ``groups = mp`` and splits that dim ``mp`` ways: every rank then owns exactly one block - its own gate /
up columns or its own heads - and runs the kernel with ``groups = 1`` on it.

The reference composes these from Split / Mul / SiLU / ApplyRotaryPosEmb / FlashAttentionScore / Add / RmsNorm
(ops_def/{rms_norm,apply_rotary_pos_emb,flash_attention_score,silu}_op.yaml); those primitives exist here too.
"""
from __future__ import annotations

import math

import torch

from . import fused
from .primitive import Primitive, prim_attr_register

__all__ = ["AddRmsNorm", "SwiGLU", "RotaryFlashAttention"]


class AddRmsNorm(Primitive):
    @prim_attr_register
    def __init__(self, epsilon=1e-6):
        self.init_prim_io_names(["x1", "x2", "gamma"], ["y", "x"])

    def _run(self, x1, x2, gamma):
        return fused.rms_norm(x1, gamma, self.epsilon, x2)


class SwiGLU(Primitive):
    @prim_attr_register
    def __init__(self, groups=1):
        if not isinstance(groups, int) or groups < 1:
            raise ValueError("For 'SwiGLU', 'groups' must be a positive int, but got %r" % (groups,))

    def _run(self, gu):
        g = self.groups
        if g == 1:
            return fused.swiglu(gu)
        if gu.shape[-1] % (2 * g):
            raise ValueError("For 'SwiGLU', the last dim %d must be divisible by 2 * groups (%d)" % (gu.shape[-1], 2 * g))
        f = gu.shape[-1] // (2 * g)
        v = gu.reshape(*gu.shape[:-1], g, 2, f)
        return (torch.nn.functional.silu(v[..., 0, :]) * v[..., 1, :]).reshape(*gu.shape[:-1], g * f)


class RotaryFlashAttention(Primitive):
    """qkv [batch * seq, (H + 2 Hk) * D], cos / sin fp32 [seq, D / 2] -> attention output [batch * seq, H * D]."""

    @prim_attr_register
    def __init__(self, head_num, kv_head_num, head_dim, groups=1, causal=True, scale_value=None):
        if head_num % groups or kv_head_num % groups:
            raise ValueError("For 'RotaryFlashAttention', head_num %d and kv_head_num %d must be divisible by "
                             "groups %d" % (head_num, kv_head_num, groups))

    def _one(self, qkv, cos, sin, heads, kv_heads):
        seq, d = cos.shape[0], self.head_dim          # the tables cover exactly one sequence
        if qkv.shape[0] % seq:
            raise ValueError("For 'RotaryFlashAttention', %d tokens are not whole sequences of %d"
                             % (qkv.shape[0], seq))
        batch = qkv.shape[0] // seq
        scale = self.scale_value if self.scale_value is not None else 1.0 / math.sqrt(d)
        o = fused.qkv_rope_attention(qkv, cos, sin, batch, seq, heads, kv_heads, d, causal=self.causal, scale=scale)
        return o.reshape(batch * seq, heads * d)

    def _run(self, qkv, cos, sin):
        g = self.groups
        h, hk = self.head_num // g, self.kv_head_num // g
        if g == 1:
            return self._one(qkv, cos, sin, h, hk)
        blk = (h + 2 * hk) * self.head_dim
        return torch.cat([self._one(qkv[:, i * blk:(i + 1) * blk].contiguous(), cos, sin, h, hk) for i in range(g)], -1)
