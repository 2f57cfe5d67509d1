"""Long-sequence (context) parallel attention: the sequence is split over a communication group.

Two schemes, both differentiable:

* ``ulysses_attention`` - all-to-all turns the sequence split into a head split, every rank runs ordinary attention
  over the full sequence for ``heads / cp`` heads, and a second all-to-all restores the sequence split (the
  reference's ``FlashAttentionScore`` strategy that shards N instead of S after an AlltoAll redistribution).
* ``ring_attention`` - K/V blocks travel around the ring; each rank attends its queries to one block per step and
  merges the partial results by their log-sum-exp.  Backward walks the ring again: with the *global* LSE and output,
  the block-wise backward kernel yields exact partial dQ and the dK/dV of the visiting block, which are passed on
  with the block so that they arrive home after a full turn.  With causal masking, blocks from later ranks are
  skipped and the rank's own block uses the causal kernel (ccsrc/frontend/parallel/ops_info/
  flash_attention_score_info.cc:1134-1390 covers the reference's ring / load-balance expansion; kv send/recv there
  is NeighborExchange, here ``batch_isend_irecv`` on the group).

* ``ring_attention(..., load_balance=True)`` - the causal ring with the zigzag layout: the sequence is cut into
  ``2 cp`` chunks and rank r holds chunks r and ``2 cp - 1 - r`` (``zigzag_split`` / ``zigzag_merge`` convert).  Every
  ring step then costs every rank the same: its own block is one causal call, a block from an earlier rank is all
  local queries against the first half of the visiting keys, a block from a later rank is the second half of the
  local queries against all visiting keys - half a block pair each, instead of rank r working r + 1 steps and idling
  the rest (the reference's load-balanced ring, flash_attention_score_info.cc:1134-1390, and flash_sp.cc).

On CUDA bf16 with head dim 128 the per-block work is the tcgen05 FlashAttention forward / backward kernels; other
inputs use the fp32 torch formulation of the same block update."""
from __future__ import annotations

import math

import torch
import torch.distributed as dist

from ..communication import management as M
from ..ops import flash_attn_kernel as FK


# ------------------------------------------------------------------------------------------------ block kernels
def _block_fwd(q, k, v, causal, scale):
    """(out [B,S,H,D], lse [B,H,S] fp32) of one q-block x kv-block attention."""
    if FK.supports(q, k, v):
        o, lse, _, _, _ = FK.fwd(q, k, v, causal, scale)
        return o, lse
    s = torch.einsum("bqhd,bkhd->bhqk", q.float(), k.float()) * scale
    if causal:
        s = s.masked_fill(torch.ones(s.shape[-2:], dtype=torch.bool, device=s.device).triu(1), float("-inf"))
    lse = torch.logsumexp(s, -1)
    o = torch.einsum("bhqk,bkhd->bqhd", torch.exp(s - lse[..., None]), v.float())
    return o.to(q.dtype), lse


def _block_bwd(do, q, k, v, o, lse, causal, scale):
    """dq, dk, dv of one block given the *final* output ``o`` and log-sum-exp ``lse`` of the whole row."""
    if FK.supports(q, k, v):
        return FK.bwd(do, q, k, v, o, lse, causal, scale)
    s = torch.einsum("bqhd,bkhd->bhqk", q.float(), k.float()) * scale
    if causal:
        s = s.masked_fill(torch.ones(s.shape[-2:], dtype=torch.bool, device=s.device).triu(1), float("-inf"))
    p = torch.exp(s - lse[..., None])
    dv = torch.einsum("bhqk,bqhd->bkhd", p, do.float())
    dp = torch.einsum("bqhd,bkhd->bhqk", do.float(), v.float())
    delta = (do.float() * o.float()).sum(-1).permute(0, 2, 1)                 # [B,H,S]
    ds = p * (dp - delta[..., None]) * scale
    dq = torch.einsum("bhqk,bkhd->bqhd", ds, k.float())
    dk = torch.einsum("bhqk,bqhd->bkhd", ds, q.float())
    return dq.to(q.dtype), dk.to(k.dtype), dv.to(v.dtype)


def _ring_exchange(tensors, group, rank_in_group, world):
    """Sends ``tensors`` to the next rank of the ring and returns what arrives from the previous one."""
    nxt = group.ranks[(rank_in_group + 1) % world]
    prv = group.ranks[(rank_in_group - 1) % world]
    recv = [torch.empty_like(t) for t in tensors]
    ops = []
    for t, r in zip(tensors, recv):
        ops.append(dist.P2POp(dist.isend, t.contiguous(), nxt, group=group.pg))
        ops.append(dist.P2POp(dist.irecv, r, prv, group=group.pg))
    for w in dist.batch_isend_irecv(ops):
        w.wait()
    return recv


class _RingAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, gname, causal, scale):
        g = M._group(gname)
        world, me = g.size, g.ranks.index(M.get_rank())
        out = lse = None
        kb, vb = k.contiguous(), v.contiguous()
        for step in range(world):
            src = (me - step) % world                     # whose block is visiting
            if not causal or src <= me:
                o_i, lse_i = _block_fwd(q, kb, vb, causal and src == me, scale)
                if out is None:
                    out, lse = o_i.float(), lse_i
                else:
                    new = torch.logaddexp(lse, lse_i)
                    w_old = torch.exp(lse - new).permute(0, 2, 1)[..., None]
                    w_new = torch.exp(lse_i - new).permute(0, 2, 1)[..., None]
                    out = out * w_old + o_i.float() * w_new
                    lse = new
            if step + 1 < world:
                kb, vb = _ring_exchange([kb, vb], g, me, world)
        out = out.to(q.dtype)
        ctx.save_for_backward(q, k, v, out, lse)
        ctx.meta = (gname, causal, scale)
        return out

    @staticmethod
    def backward(ctx, do):
        q, k, v, out, lse = ctx.saved_tensors
        gname, causal, scale = ctx.meta
        g = M._group(gname)
        world, me = g.size, g.ranks.index(M.get_rank())
        do = do.contiguous()
        dq = torch.zeros_like(q, dtype=torch.float32)
        kb, vb = k.contiguous(), v.contiguous()
        dkb = torch.zeros_like(k, dtype=torch.float32)
        dvb = torch.zeros_like(v, dtype=torch.float32)
        for step in range(world):
            src = (me - step) % world
            if not causal or src <= me:
                dq_i, dk_i, dv_i = _block_bwd(do, q, kb, vb, out, lse.contiguous(), causal and src == me, scale)
                dq += dq_i.float()
                dkb += dk_i.float()
                dvb += dv_i.float()
            # the block and the gradients gathered for it move on together; after `world` moves they are home
            kb, vb, dkb, dvb = _ring_exchange([kb, vb, dkb, dvb], g, me, world)
        return dq.to(q.dtype), dkb.to(k.dtype), dvb.to(v.dtype), None, None, None


def _merge(out, lse, o_i, lse_i):
    """Folds a partial attention result (o_i, lse_i) into the running (out fp32 [B,S,H,D], lse [B,H,S])."""
    if out is None:
        return o_i.float(), lse_i
    new = torch.logaddexp(lse, lse_i)
    w_old = torch.exp(lse - new).permute(0, 2, 1)[..., None]
    w_new = torch.exp(lse_i - new).permute(0, 2, 1)[..., None]
    return out * w_old + o_i.float() * w_new, new


class _ZigzagRingAttention(torch.autograd.Function):
    """Causal ring attention on the zigzag layout: local rows = [chunk me ; chunk 2 cp - 1 - me]."""

    @staticmethod
    def forward(ctx, q, k, v, gname, scale):
        g = M._group(gname)
        world, me = g.size, g.ranks.index(M.get_rank())
        half = q.shape[1] // 2
        out_lo = lse_lo = out_hi = lse_hi = None           # running results of the early / late local chunk
        kb, vb = k.contiguous(), v.contiguous()
        for step in range(world):
            src = (me - step) % world
            if src == me:
                o_i, lse_i = _block_fwd(q, kb, vb, True, scale)
                out_lo, lse_lo = _merge(out_lo, lse_lo, o_i[:, :half], lse_i[..., :half])
                out_hi, lse_hi = _merge(out_hi, lse_hi, o_i[:, half:], lse_i[..., half:])
            elif src < me:      # the visitor's early chunk precedes both local chunks; its late chunk follows both
                o_i, lse_i = _block_fwd(q, kb[:, :half].contiguous(), vb[:, :half].contiguous(), False, scale)
                out_lo, lse_lo = _merge(out_lo, lse_lo, o_i[:, :half], lse_i[..., :half])
                out_hi, lse_hi = _merge(out_hi, lse_hi, o_i[:, half:], lse_i[..., half:])
            else:               # both visiting chunks precede the local late chunk and follow the local early chunk
                o_i, lse_i = _block_fwd(q[:, half:].contiguous(), kb, vb, False, scale)
                out_hi, lse_hi = _merge(out_hi, lse_hi, o_i, lse_i)
            if step + 1 < world:
                kb, vb = _ring_exchange([kb, vb], g, me, world)
        out = torch.cat([out_lo, out_hi], 1).to(q.dtype)
        lse = torch.cat([lse_lo, lse_hi], -1).contiguous()
        ctx.save_for_backward(q, k, v, out, lse)
        ctx.meta = (gname, scale)
        return out

    @staticmethod
    def backward(ctx, do):
        q, k, v, out, lse = ctx.saved_tensors
        gname, scale = ctx.meta
        g = M._group(gname)
        world, me = g.size, g.ranks.index(M.get_rank())
        half = q.shape[1] // 2
        do = do.contiguous()
        dq = torch.zeros_like(q, dtype=torch.float32)
        kb, vb = k.contiguous(), v.contiguous()
        dkb = torch.zeros_like(k, dtype=torch.float32)
        dvb = torch.zeros_like(v, dtype=torch.float32)
        q_hi, do_hi, out_hi = (t[:, half:].contiguous() for t in (q, do, out))
        lse_hi = lse[..., half:].contiguous()
        for step in range(world):
            src = (me - step) % world
            if src == me:
                dq_i, dk_i, dv_i = _block_bwd(do, q, kb, vb, out, lse, True, scale)
                dq += dq_i.float()
                dkb += dk_i.float()
                dvb += dv_i.float()
            elif src < me:
                dq_i, dk_i, dv_i = _block_bwd(do, q, kb[:, :half].contiguous(), vb[:, :half].contiguous(), out, lse,
                                              False, scale)
                dq += dq_i.float()
                dkb[:, :half] += dk_i.float()
                dvb[:, :half] += dv_i.float()
            else:
                dq_i, dk_i, dv_i = _block_bwd(do_hi, q_hi, kb, vb, out_hi, lse_hi, False, scale)
                dq[:, half:] += dq_i.float()
                dkb += dk_i.float()
                dvb += dv_i.float()
            kb, vb, dkb, dvb = _ring_exchange([kb, vb, dkb, dvb], g, me, world)
        return dq.to(q.dtype), dkb.to(k.dtype), dvb.to(v.dtype), None, None


def zigzag_split(x, world, rank, dim=1):
    """This rank's rows of a full sequence in the load-balanced layout: chunks ``rank`` and ``2 world - 1 - rank`` of
    ``2 world`` equal chunks along ``dim``."""
    chunks = x.chunk(2 * world, dim)
    return torch.cat([chunks[rank], chunks[2 * world - 1 - rank]], dim)


def zigzag_merge(parts, dim=1):
    """Inverse of ``zigzag_split``: ``parts[r]`` is rank r's tensor; returns the full sequence in natural order."""
    world = len(parts)
    chunks = [None] * (2 * world)
    for r, p in enumerate(parts):
        lo, hi = p.chunk(2, dim)
        chunks[r], chunks[2 * world - 1 - r] = lo, hi
    return torch.cat(chunks, dim)


def ring_attention(q, k, v, group, causal=True, scale=None, load_balance=False):
    """q, k, v: [B, S/cp, H, D], this rank's slice of the sequence: contiguous (rank order = sequence order), or with
    ``load_balance=True`` (causal only) the zigzag layout of ``zigzag_split``."""
    scale = scale if scale is not None else 1.0 / math.sqrt(q.shape[-1])
    g = M._group(group)
    if load_balance and not causal:
        raise ValueError("ring_attention: load_balance applies to causal attention (full attention is balanced)")
    if g.size == 1:
        from ..ops import fused
        return fused.flash_attention(q, k, v, causal=causal, scale=scale)
    if load_balance:
        if q.shape[1] % 2:
            raise ValueError("ring_attention: the local sequence length %d must be even for the zigzag layout"
                             % q.shape[1])
        return _ZigzagRingAttention.apply(q, k, v, g.name, scale)
    return _RingAttention.apply(q, k, v, g.name, causal, scale)


# ------------------------------------------------------------------------------------------------ Ulysses
class _SeqToHead(torch.autograd.Function):
    """[B, S/cp, H, D] -> [B, S, H/cp, D] (forward) and back (backward) with one all-to-all."""

    @staticmethod
    def forward(ctx, x, gname, inverse):
        ctx.meta = (gname, inverse)
        return _a2a(x, M._group(gname), inverse)

    @staticmethod
    def backward(ctx, dy):
        gname, inverse = ctx.meta
        return _a2a(dy.contiguous(), M._group(gname), not inverse), None, None


def _a2a(x, g, inverse):
    cp = g.size
    b, s, h, d = x.shape
    if not inverse:      # split heads, gather sequence
        send = x.reshape(b, s, cp, h // cp, d).permute(2, 0, 1, 3, 4).contiguous()      # [cp, B, s, h/cp, D]
        recv = torch.empty_like(send)
        dist.all_to_all_single(recv, send, group=g.pg)
        return recv.permute(1, 0, 2, 3, 4).reshape(b, cp * s, h // cp, d)
    send = x.reshape(b, cp, s // cp, h, d).permute(1, 0, 2, 3, 4).contiguous()           # [cp, B, S/cp, h, D]
    recv = torch.empty_like(send)
    dist.all_to_all_single(recv, send, group=g.pg)
    return recv.permute(1, 2, 0, 3, 4).reshape(b, s // cp, cp * h, d)


def ulysses_attention(q, k, v, group, causal=True, scale=None):
    """q, k, v: [B, S/cp, H, D] with H divisible by the group size."""
    from ..ops import fused
    g = M._group(group)
    if g.size == 1:
        return fused.flash_attention(q, k, v, causal=causal, scale=scale)
    if q.shape[2] % g.size:
        raise ValueError("ulysses_attention: %d heads are not divisible by the group size %d" % (q.shape[2], g.size))
    qh, kh, vh = (_SeqToHead.apply(t.contiguous(), g.name, False) for t in (q, k, v))
    o = fused.flash_attention(qh, kh, vh, causal=causal, scale=scale)
    return _SeqToHead.apply(o.contiguous(), g.name, True)
