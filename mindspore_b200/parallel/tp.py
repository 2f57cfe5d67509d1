"""Tensor (model) parallel building blocks with sequence parallelism.

Activations between tensor-parallel regions are sharded along the token dim (``[tokens/mp, hidden]``); a
column-parallel Dense starts with AllGather(tokens) and a row-parallel Dense ends with ReduceScatter(tokens) -
the strategy the reference expresses as ``matmul.shard(((dp, 1), (mp, 1)))`` followed by a row-parallel MatMul
whose ``out_strategy`` row-shards the output (ccsrc/frontend/parallel/ops_info/matmul_info.cc:333-337,394-398)
with LayerNorm sharded on the sequence dim.  Here the communication is explicit and differentiable
(AllGather <-> ReduceScatter), and each (collective, GEMM) pair is served by one fused NVLink kernel when the
symmetric-memory runtime is up (``parallel.fused_comm``): AllGather->MatMul pulls peer token shards inside the
GEMM loader, MatMul->ReduceScatter pushes partial tiles to their owner from the epilogue.

Parity: mindspore/python/mindspore/parallel/_transformer/layers.py:347 (_Linear), transformer.py:349
(FeedForward), :756 (MultiHeadAttention), loss.py:157 (vocab-parallel CrossEntropyLoss).
"""
from __future__ import annotations

import torch

from ..communication import comm_func as CF
from ..communication import management as M
from ..ops import fused
from ..ops import kernels as K
from . import fused_comm


class TPGroup:
    """Model-parallel group descriptor: name, size and this rank's index."""

    def __init__(self, name=None, size=None, rank=None):
        if name is None and M.GlobalComm.INITED:
            name = M.GlobalComm.WORLD_COMM_GROUP
        self.name = name
        self.size = size if size is not None else (M.get_group_size(name) if name else 1)
        self.rank = rank if rank is not None else (M.get_rank(name) if name and not M.is_simulation() else 0)

    @property
    def active(self):
        return self.size > 1


def gather_tokens(x, tp):
    """[T/mp, ...] -> [T, ...]; backward ReduceScatter."""
    if not tp.active:
        return x
    return CF.all_gather_autograd(x.contiguous(), tp.name)


def scatter_tokens_reduce(x, tp):
    """partial [T, ...] -> summed [T/mp, ...]; backward AllGather."""
    if not tp.active:
        return x
    return CF.reduce_scatter_autograd(x.contiguous(), "sum", tp.name)


class _ReduceFromTP(torch.autograd.Function):
    """AllReduce forward, identity backward: the partner of ``_CopyToTP`` (whose backward all-reduces).  Between
    the two, replicated activations carry the complete gradient on every rank."""

    @staticmethod
    def forward(ctx, x, gname):
        return CF._all_reduce_(x.clone(), "sum", M._group(gname))

    @staticmethod
    def backward(ctx, dy):
        return dy, None


def reduce_partial(x, tp):
    if not tp.active:
        return x
    return _ReduceFromTP.apply(x, tp.name)


class _CopyToTP(torch.autograd.Function):
    """Identity forward, AllReduce backward (input of a column-parallel op without sequence parallelism)."""

    @staticmethod
    def forward(ctx, x, gname):
        ctx.gname = gname
        return x.view_as(x)

    @staticmethod
    def backward(ctx, dy):
        return CF._all_reduce_(dy.clone(), "sum", M._group(ctx.gname)), None


def copy_to_tp(x, tp):
    return _CopyToTP.apply(x, tp.name) if tp.active else x


def column_parallel_linear(x_shard, w_shard, tp, bias=None, sequence_parallel=True):
    """x [T/mp, K] (token-sharded) or [T, K]; w_shard [N/mp, K] -> y [T, N/mp]."""
    if tp.active and sequence_parallel and fused_comm.available(M._group(tp.name)):
        return fused_comm.allgather_matmul(x_shard, w_shard, tp, bias)
    x = gather_tokens(x_shard, tp) if sequence_parallel else copy_to_tp(x_shard, tp)
    return fused.linear(x, w_shard, bias)


def row_parallel_linear(x, w_shard, tp, bias=None, sequence_parallel=True):
    """x [T, K/mp]; w_shard [N, K/mp] -> y [T/mp, N] (token-sharded) or [T, N]."""
    if tp.active and sequence_parallel and fused_comm.available(M._group(tp.name)):
        y = fused_comm.matmul_reduce_scatter(x, w_shard, tp)
    else:
        y = fused.linear(x, w_shard)
        y = scatter_tokens_reduce(y, tp) if sequence_parallel else reduce_partial(y, tp)
    if bias is not None:
        y = y + bias
    return y


def vocab_parallel_embedding(table_shard, ids, tp, sequence_parallel=True):
    """table_shard [V/mp, H]; ids [T] (full) -> [T/mp, H] (or [T, H])."""
    if not tp.active:
        return fused.embedding(table_shard, ids)
    part = fused.embedding(table_shard, ids, tp.rank * table_shard.shape[0])
    return scatter_tokens_reduce(part, tp) if sequence_parallel else reduce_partial(part, tp)


class _VocabParallelCE(torch.autograd.Function):
    """Mean cross entropy with logits sharded over the vocabulary: per-shard (max, sumexp, target) statistics
    are combined across the group, then each rank writes the gradient of its own shard in one pass."""

    @staticmethod
    def forward(ctx, logits, labels, gname, rank, ignore_index):
        g = M._group(gname)
        V = logits.shape[-1]
        rows = logits.numel() // V
        labels32 = labels.reshape(-1).to(torch.int32)
        start = rank * V
        if logits.is_cuda and logits.dtype in (torch.bfloat16, torch.float32):
            stats = K.ce_stats(logits, labels32, start)
        else:
            lf = logits.reshape(rows, V).float()
            m = torch.amax(lf, -1)
            s = torch.exp(lf - m[:, None]).sum(-1)
            loc = labels32.long() - start
            inr = (loc >= 0) & (loc < V)
            tgt = torch.where(inr, lf.gather(1, loc.clamp(0, V - 1)[:, None])[:, 0], torch.zeros_like(m))
            stats = torch.stack([m, s, tgt], -1)
        allst = CF._all_gather(stats.unsqueeze(0).contiguous(), g)          # [mp, rows, 3]
        gm = torch.amax(allst[..., 0], 0)
        gs = (allst[..., 1] * torch.exp(allst[..., 0] - gm)).sum(0)
        gt = allst[..., 2].sum(0)
        merged = torch.stack([gm, gs, gt], -1).contiguous()
        valid = labels32 != ignore_index
        nvalid = valid.sum().clamp(min=1).float()
        loss_rows = torch.where(valid, torch.log(gs) + gm - gt, torch.zeros_like(gm))
        ctx.save_for_backward(logits, labels32, merged, nvalid)
        ctx.meta = (start, ignore_index)
        return loss_rows.sum() / nvalid

    @staticmethod
    def backward(ctx, dloss):
        logits, labels32, merged, nvalid = ctx.saved_tensors
        start, ignore_index = ctx.meta
        scale = (dloss.float() / nvalid).reshape(1).contiguous()
        if logits.is_cuda and logits.dtype in (torch.bfloat16, torch.float32):
            _, dl = K.ce_loss_grad(logits, labels32, merged, scale, start, ignore_index)
            return dl.view(logits.shape), None, None, None, None
        V = logits.shape[-1]
        lf = logits.reshape(-1, V).float()
        p = torch.exp(lf - merged[:, 0:1]) / merged[:, 1:2]
        loc = labels32.long() - start
        inr = (loc >= 0) & (loc < V)
        p[torch.arange(p.shape[0], device=p.device)[inr], loc[inr]] -= 1
        p = p * (labels32 != ignore_index)[:, None] * scale
        return p.to(logits.dtype).view(logits.shape), None, None, None, None


def vocab_parallel_cross_entropy(logits_shard, labels, tp, ignore_index=-100):
    if not tp.active:
        return fused.softmax_cross_entropy(logits_shard, labels, ignore_index)
    return _VocabParallelCE.apply(logits_shard.contiguous(), labels, tp.name, tp.rank, ignore_index)
