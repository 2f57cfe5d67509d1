"""Functional collectives and their differentiable forms.

The plain functions follow ``mindspore.communication.comm_func`` (return new tensors, take a group name).
The ``*_autograd`` functions are ``torch.autograd.Function``s whose backward is the dual collective, the
rule table of mindspore/python/mindspore/ops/_grad_experimental/grad_comm_ops.py:39-672:
AllReduce<->AllReduce, AllGather<->ReduceScatter, AlltoAll<->AlltoAll, Send<->Receive, Broadcast->Reduce.

In simulation mode (``MS_SIMULATION_LEVEL``) every collective is evaluated locally with the shapes a real
run would produce (AllGather tiles the input, ReduceScatter keeps the first chunk ...), so one rank of a
large virtual cluster can execute on one device.

Parity: mindspore/python/mindspore/communication/comm_func.py:135-1140.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from ..common.tensor import Tensor
from ..ops.primitive import _wrap_out
from ..utils import recorder as _recorder
from . import management as M

_REDUCE = {"sum": dist.ReduceOp.SUM, "prod": dist.ReduceOp.PRODUCT, "max": dist.ReduceOp.MAX, "min": dist.ReduceOp.MIN}


class ReduceOp:
    SUM = "sum"
    MAX = "max"
    MIN = "min"
    PROD = "prod"


def _op(op):
    if op not in _REDUCE:
        raise ValueError("For collective ops, 'op' must be one of sum, prod, max, min, but got %r" % (op,))
    return _REDUCE[op]


def _plain(t):
    return t.detach().as_subclass(torch.Tensor) if isinstance(t, torch.Tensor) else t


def _single(g):
    return g.size == 1


# ------------------------------------------------------------------------------------ raw (non-differentiable)
def _rec(name, t, g):
    if _recorder.enabled():
        _recorder.record("collective", "%s %s" % (name, g.name), t.numel() * t.element_size(), g.size)


def _traced(fn, *args):
    """While a graph is being traced a raw collective is recorded as one node (target = the function below taking
    the group by *name*), so that a replay performs it; eagerly it just runs."""
    from ..graph import tracer
    if not tracer.is_tracing():
        return None
    from ..graph import jit
    return jit.leaf_call(fn, args, {})


def all_reduce_node(t, op, gname):
    return _all_reduce_(t, op, M._group(gname), _node=True)


def all_gather_node(t, gname):
    return _all_gather(t, M._group(gname), _node=True)


def reduce_scatter_node(t, op, gname):
    return _reduce_scatter(t, op, M._group(gname), _node=True)


def all_to_all_node(t, split_dim, concat_dim, gname):
    return _all_to_all(t, split_dim, concat_dim, M._group(gname), _node=True)


for _f in (all_reduce_node, all_gather_node, reduce_scatter_node, all_to_all_node):
    _f.is_collective = True


def _all_reduce_(t, op, g, _node=False):
    if not _node and isinstance(t, torch.Tensor) and not _single(g):
        out = _traced(all_reduce_node, t, op, g.name)
        if out is not None:
            return out
    if M.is_simulation() or _single(g):
        return t
    _rec("AllReduce", t, g)
    dist.all_reduce(t, _op(op), group=g.pg)
    return t


def _all_gather(t, g, _node=False):
    if not _node and not _single(g):
        out = _traced(all_gather_node, t, g.name)
        if out is not None:
            return out
    n = g.size
    out = torch.empty((n * t.shape[0],) + tuple(t.shape[1:]), dtype=t.dtype, device=t.device)
    if M.is_simulation() or _single(g):
        out.view(n, *t.shape).copy_(t.unsqueeze(0).expand(n, *t.shape))
        return out
    _rec("AllGather", t, g)
    dist.all_gather_into_tensor(out, t.contiguous(), group=g.pg)
    return out


def _reduce_scatter(t, op, g, _node=False):
    if not _node and not _single(g):
        out = _traced(reduce_scatter_node, t, op, g.name)
        if out is not None:
            return out
    n = g.size
    if t.shape[0] % n:
        raise ValueError("ReduceScatter needs dim 0 (%d) divisible by the group size (%d)" % (t.shape[0], n))
    out = torch.empty((t.shape[0] // n,) + tuple(t.shape[1:]), dtype=t.dtype, device=t.device)
    if M.is_simulation() or _single(g):
        r = 0 if M.is_simulation() else 0
        out.copy_(t[r * out.shape[0]:(r + 1) * out.shape[0]])
        return out
    _rec("ReduceScatter", t, g)
    dist.reduce_scatter_tensor(out, t.contiguous(), _op(op), group=g.pg)
    return out


def _all_to_all(t, split_dim, concat_dim, g, _node=False):
    if not _node and not _single(g):
        out = _traced(all_to_all_node, t, split_dim, concat_dim, g.name)
        if out is not None:
            return out
    n = g.size
    chunks = [c.contiguous() for c in torch.chunk(t, n, dim=split_dim)]
    if M.is_simulation() or _single(g):
        return torch.cat(chunks, dim=concat_dim)
    outs = [torch.empty_like(c) for c in chunks]
    _rec("AlltoAll", t, g)
    if g.pg is not None and dist.get_backend(g.pg) == "gloo":
        # gloo has no all_to_all: emulate with all_gather of the full tensor list
        gathered = [torch.empty_like(t) for _ in range(n)]
        dist.all_gather(gathered, t.contiguous(), group=g.pg)
        me = M.get_rank(g.name)
        outs = [torch.chunk(gathered[r], n, dim=split_dim)[me] for r in range(n)]
    else:
        dist.all_to_all(outs, chunks, group=g.pg)
    return torch.cat(outs, dim=concat_dim)


# ------------------------------------------------------------------------------------ differentiable forms
class _AllReduceFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, op, gname):
        ctx.op, ctx.gname = op, gname
        return _all_reduce_(x.clone(), op, M._group(gname))

    @staticmethod
    def backward(ctx, dy):
        if ctx.op != "sum":
            raise RuntimeError("gradient of AllReduce is defined for op=sum only")
        return _all_reduce_(dy.clone(), "sum", M._group(ctx.gname)), None, None


class _AllGatherFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, gname, mean):
        ctx.gname, ctx.mean = gname, mean
        return _all_gather(x, M._group(gname))

    @staticmethod
    def backward(ctx, dy):
        g = M._group(ctx.gname)
        dx = _reduce_scatter(dy.contiguous(), "sum", g)
        if ctx.mean:
            dx = dx / g.size
        return dx, None, None


class _ReduceScatterFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, op, gname):
        ctx.gname = gname
        return _reduce_scatter(x, op, M._group(gname))

    @staticmethod
    def backward(ctx, dy):
        return _all_gather(dy.contiguous(), M._group(ctx.gname)), None, None


class _AllToAllFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, split_dim, concat_dim, gname):
        ctx.meta = (split_dim, concat_dim, gname)
        return _all_to_all(x, split_dim, concat_dim, M._group(gname))

    @staticmethod
    def backward(ctx, dy):
        sd, cd, gname = ctx.meta
        return _all_to_all(dy.contiguous(), cd, sd, M._group(gname)), None, None, None


class _BroadcastFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, src, gname):
        ctx.meta = (src, gname)
        g = M._group(gname)
        out = x.clone()
        if not (M.is_simulation() or _single(g)):
            dist.broadcast(out, src, group=g.pg)
        return out

    @staticmethod
    def backward(ctx, dy):
        src, gname = ctx.meta
        g = M._group(gname)
        d = dy.clone()
        if not (M.is_simulation() or _single(g)):
            dist.reduce(d, src, group=g.pg)
            if M._state.rank != src:
                d = torch.zeros_like(d)
        return d, None, None


def all_reduce_autograd(x, op="sum", group=None):
    return _AllReduceFn.apply(x, op, M._group(group).name)


def all_gather_autograd(x, group=None, mean=False):
    return _AllGatherFn.apply(x, M._group(group).name, mean)


def reduce_scatter_autograd(x, op="sum", group=None):
    return _ReduceScatterFn.apply(x, op, M._group(group).name)


def all_to_all_autograd(x, split_dim, concat_dim, group=None):
    return _AllToAllFn.apply(x, split_dim, concat_dim, M._group(group).name)


def broadcast_autograd(x, src=0, group=None):
    return _BroadcastFn.apply(x, src, M._group(group).name)


# ------------------------------------------------------------------------------------ public functional API
def all_reduce(tensor, op=ReduceOp.SUM, group=None):
    if not isinstance(tensor, torch.Tensor):
        raise TypeError("For all_reduce, the input tensor must be tensor")
    return _wrap_out(all_reduce_autograd(tensor, op, group))


def all_gather_into_tensor(tensor, group=None):
    if not isinstance(tensor, torch.Tensor):
        raise TypeError("For all_gather_into_tensor, the input tensor must be tensor")
    return _wrap_out(all_gather_autograd(tensor, group))


def reduce_scatter_tensor(tensor, op=ReduceOp.SUM, group=None):
    if not isinstance(tensor, torch.Tensor):
        raise TypeError("For reduce_scatter_tensor, the input tensor must be tensor")
    return _wrap_out(reduce_scatter_autograd(tensor, op, group))


def reduce(tensor, dst, op=ReduceOp.SUM, group=None):
    g = M._group(group)
    out = _plain(tensor).clone()
    if not (M.is_simulation() or _single(g)):
        dist.reduce(out, M.get_world_rank_from_group_rank(g.name, dst) if g.name != M.GlobalComm.WORLD_COMM_GROUP
                    else dst, _op(op), group=g.pg)
    return _wrap_out(out)


def broadcast(tensor, src=0, group=None):
    return _wrap_out(broadcast_autograd(tensor, src, group))


def barrier(group=None):
    g = M._group(group)
    if not (M.is_simulation() or _single(g)):
        dist.barrier(group=g.pg)


def isend(tensor, dst=0, group=None, tag=0):
    g = M._group(group)
    if M.is_simulation():
        return None
    return dist.isend(_plain(tensor).contiguous(), dst, group=g.pg, tag=tag)


def irecv(tensor, src=0, group=None, tag=0):
    g = M._group(group)
    if M.is_simulation():
        return tensor
    out = _plain(tensor)
    w = dist.irecv(out, src, group=g.pg, tag=tag)
    w.wait()
    return _wrap_out(out)


class P2POp:
    def __init__(self, op, tensor, peer, group=None, tag=0, *, recv_dtype=None):
        self.op = op if isinstance(op, str) else getattr(op, "__name__", str(op))
        self.tensor, self.peer, self.group, self.tag = tensor, peer, group, tag


def batch_isend_irecv(p2p_op_list):
    if M.is_simulation():
        return tuple(o.tensor for o in p2p_op_list if o.op == "irecv")
    ops = []
    for o in p2p_op_list:
        g = M._group(o.group)
        fn = dist.isend if o.op == "isend" else dist.irecv
        ops.append(dist.P2POp(fn, _plain(o.tensor), o.peer, g.pg, o.tag))
    for w in dist.batch_isend_irecv(ops):
        w.wait()
    return tuple(_wrap_out(_plain(o.tensor)) for o in p2p_op_list if o.op == "irecv")


def scatter_tensor(tensor, src=0, group=None):
    g = M._group(group)
    n = g.size
    me = 0 if M.is_simulation() else M.get_rank(g.name)
    full = broadcast_autograd(tensor, src, g.name)
    return _wrap_out(torch.chunk(full, n, dim=0)[me].contiguous())


def gather_into_tensor(tensor, dst=0, group=None):
    g = M._group(group)
    out = _all_gather(_plain(tensor), g)
    return _wrap_out(out)


def all_to_all_single_with_output_shape(output_shape, tensor, output_split_sizes=None, input_split_sizes=None,
                                        group=None):
    g = M._group(group)
    t = _plain(tensor).contiguous()
    out = torch.empty(tuple(output_shape), dtype=t.dtype, device=t.device)
    if M.is_simulation() or _single(g):
        out.view(-1)[:t.numel()].copy_(t.view(-1)[:out.numel()])
        return _wrap_out(out)
    dist.all_to_all_single(out, t, output_split_sizes, input_split_sizes, group=g.pg)
    return _wrap_out(out)


def all_to_all_with_output_shape(output_shape_list, input_tensor_list, group=None):
    g = M._group(group)
    ins = [_plain(t).contiguous() for t in input_tensor_list]
    outs = [torch.empty(tuple(s), dtype=ins[0].dtype, device=ins[0].device) if not isinstance(s, torch.Tensor)
            else torch.empty_like(s) for s in output_shape_list]
    if M.is_simulation() or _single(g):
        for o, i in zip(outs, ins):
            o.copy_(i)
    else:
        dist.all_to_all(outs, ins, group=g.pg)
    return tuple(_wrap_out(o) for o in outs)
