"""Communication primitives, including the internal ones the parallel planner inserts.

Every primitive here differentiates into the dual collective of the reference's rule table
(mindspore/python/mindspore/ops/_grad_experimental/grad_comm_ops.py:39-672):

=====================  ============================================================
forward                backward
=====================  ============================================================
AllReduce(sum)         AllReduce(sum)
AllGather              ReduceScatter (x 1/N when mean_flag)
ReduceScatter          AllGather
AlltoAll               AlltoAll with split/concat dims swapped
Send / Receive         Receive / Send
_MirrorOperator        AllReduce of the gradient (x 1/dev_num when mean_flag)
_MirrorMicroStepOp     accumulate into the accumulator, AllReduce once per step
_MicroStepAllGather    ReduceScatter of the accumulated gradient
_VirtualDiv            gradient / divisor
_VirtualAssignAdd      AssignAdd into the gradient accumulator
=====================  ============================================================

Parity: mindspore/python/mindspore/ops/operations/comm_ops.py:29-1914.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from ..communication import comm_func as CF
from ..communication import management as M
from ..communication.comm_func import ReduceOp
from .primitive import Primitive, prim_attr_register


def _gname(group):
    return group if group is not None else M.GlobalComm.WORLD_COMM_GROUP


class _CommPrimitive(Primitive):
    def _init_group(self, group):
        self.group = _gname(group)
        self.add_prim_attr("group", self.group)
        self.add_prim_attr("fusion", 0)
        self.add_prim_attr("index", 0)
        self.add_prim_attr("no_eliminate", True)
        try:
            self.rank_size = M.get_group_size(self.group)
            self.rank = M.get_rank(self.group)
        except (RuntimeError, ValueError):
            self.rank_size, self.rank = 1, 0
        self.add_prim_attr("rank_size", self.rank_size)


class AllReduce(_CommPrimitive):
    def __init__(self, op=ReduceOp.SUM, group=None):
        super().__init__("AllReduce")
        if not isinstance(op, str):
            raise TypeError("For 'AllReduce', the 'op' must be str, but got %s" % type(op).__name__)
        if not isinstance(_gname(group), str):
            raise TypeError("For 'AllReduce', the 'group' must be str, but got %s" % type(group).__name__)
        self.op = op
        self.add_prim_attr("op", op)
        self._init_group(group)

    def _run(self, x):
        return CF.all_reduce_autograd(x, self.op, self.group)


class AllGather(_CommPrimitive):
    def __init__(self, group=None):
        super().__init__("AllGather")
        self._init_group(group)
        self.add_prim_attr("mean_flag", False)

    def _run(self, x):
        return CF.all_gather_autograd(x, self.group, bool(self.attrs.get("mean_flag", False)))


class ReduceScatter(_CommPrimitive):
    def __init__(self, op=ReduceOp.SUM, group=None):
        super().__init__("ReduceScatter")
        self.op = op
        self.add_prim_attr("op", op)
        self._init_group(group)

    def _run(self, x):
        return CF.reduce_scatter_autograd(x, self.op, self.group)


class Broadcast(_CommPrimitive):
    def __init__(self, root_rank, group=None):
        super().__init__("Broadcast")
        if not isinstance(root_rank, int):
            raise TypeError("For 'Broadcast', 'root_rank' must be int")
        self.root_rank = root_rank
        self.add_prim_attr("root_rank", root_rank)
        self._init_group(group)

    def _run(self, xs):
        single = isinstance(xs, torch.Tensor)
        outs = tuple(CF.broadcast_autograd(x, self.root_rank, self.group) for x in ((xs,) if single else xs))
        return outs[0] if single else outs


class Reduce(_CommPrimitive):
    def __init__(self, dest_rank, op=ReduceOp.SUM, group=None):
        super().__init__("Reduce")
        self.dest_rank, self.op = dest_rank, op
        self._init_group(group)

    def _run(self, x):
        return CF.reduce(x, self.dest_rank, self.op, self.group)


class AlltoAll(_CommPrimitive):
    def __init__(self, split_count, split_dim, concat_dim, group=None):
        super().__init__("AlltoAll")
        self._init_group(group)
        if not isinstance(split_count, int) or split_count < 1:
            raise TypeError("For 'AlltoAll', 'split_count' must be a positive int")
        self.split_count, self.split_dim, self.concat_dim = split_count, split_dim, concat_dim
        for k in ("split_count", "split_dim", "concat_dim"):
            self.add_prim_attr(k, getattr(self, k))

    def _run(self, x):
        if self.rank_size not in (1, self.split_count) and not M.is_simulation():
            raise ValueError("For 'AlltoAll', 'split_count' (%d) must equal the group size (%d)"
                             % (self.split_count, self.rank_size))
        if x.shape[self.split_dim] % self.split_count:
            raise ValueError("For 'AlltoAll', dim %d (%d) must be divisible by split_count %d"
                             % (self.split_dim, x.shape[self.split_dim], self.split_count))
        return CF.all_to_all_autograd(x, self.split_dim, self.concat_dim, self.group)


class AlltoAllV(_CommPrimitive):
    def __init__(self, group=None, block_size=1):
        super().__init__("AlltoAllV")
        self._init_group(group)
        self.block_size = block_size

    def _run(self, x, send_numel_list, recv_numel_list):
        out = CF.all_to_all_single_with_output_shape((sum(recv_numel_list),), x.reshape(-1), list(recv_numel_list),
                                                     list(send_numel_list), self.group)
        return out


class NeighborExchange(_CommPrimitive):
    def __init__(self, send_rank_ids, recv_rank_ids, recv_shapes, send_shapes, recv_type, group=None):
        super().__init__("NeighborExchange")
        self._init_group(group)
        self.send_rank_ids, self.recv_rank_ids = list(send_rank_ids), list(recv_rank_ids)
        self.recv_shapes, self.recv_type = recv_shapes, recv_type

    def _run(self, xs):
        ops = [CF.P2POp("isend", x, r, self.group) for x, r in zip(xs, self.send_rank_ids)]
        recv = [torch.empty(tuple(s), dtype=self.recv_type, device=xs[0].device if xs else None)
                for s in self.recv_shapes]
        ops += [CF.P2POp("irecv", t, r, self.group) for t, r in zip(recv, self.recv_rank_ids)]
        return CF.batch_isend_irecv(ops)


class NeighborExchangeV2(_CommPrimitive):
    """Halo exchange of an NCHW tensor with up to eight neighbours.  ``send_rank_ids`` / ``recv_rank_ids`` list the
    neighbour in the order top, top-right, right, bottom-right, bottom, bottom-left, left, top-left (-1: none);
    ``send_lens`` / ``recv_lens`` are [top, bottom, left, right] widths.  The output is the input padded with the
    received halos (ops/operations/comm_ops.py:994 in the reference; its GPU lowering is
    plugin/device/gpu/optimizer/neighbor_exchange_v2_fusion.cc)."""

    def __init__(self, send_rank_ids, send_lens, recv_rank_ids, recv_lens, data_format="NCHW", group=None):
        super().__init__("NeighborExchangeV2")
        self._init_group(group)
        self.send_rank_ids, self.recv_rank_ids = list(send_rank_ids), list(recv_rank_ids)
        self.send_lens, self.recv_lens = list(send_lens), list(recv_lens)
        if data_format != "NCHW":
            raise ValueError("For 'NeighborExchangeV2', only NCHW is supported, got %r" % data_format)

    @staticmethod
    def _region(direction, lens, H, W, inner):
        """(row slice, col slice) of the strip for ``direction``; ``inner`` selects the strip inside the tensor that
        is sent, otherwise the halo strip of the padded output that is received."""
        t, b, l, r = lens
        rows = {"top": slice(0, t), "bottom": slice(H - b, H), "mid": slice(0, H)}
        cols = {"left": slice(0, l), "right": slice(W - r, W), "mid": slice(0, W)}
        table = [("top", "mid"), ("top", "right"), ("mid", "right"), ("bottom", "right"), ("bottom", "mid"),
                 ("bottom", "left"), ("mid", "left"), ("top", "left")]
        rk, ck = table[direction]
        return rows[rk], cols[ck]

    def _run(self, x):
        N, C, H, W = x.shape
        st, sb, sl, sr = self.send_lens
        rt, rb, rl, rr = self.recv_lens
        out = torch.zeros(N, C, H + rt + rb, W + rl + rr, dtype=x.dtype, device=x.device)
        out[:, :, rt:rt + H, rl:rl + W] = x
        ops, recvs = [], []
        for d, peer in enumerate(self.send_rank_ids):
            if peer < 0:
                continue
            rs, cs = self._region(d, self.send_lens, H, W, True)
            ops.append(CF.P2POp("isend", x[:, :, rs, cs].contiguous(), peer, self.group))
        Hp, Wp = H + rt + rb, W + rl + rr
        for d, peer in enumerate(self.recv_rank_ids):
            if peer < 0:
                continue
            rows = {"top": slice(0, rt), "bottom": slice(Hp - rb, Hp), "mid": slice(rt, rt + H)}
            cols = {"left": slice(0, rl), "right": slice(Wp - rr, Wp), "mid": slice(rl, rl + W)}
            table = [("top", "mid"), ("top", "right"), ("mid", "right"), ("bottom", "right"), ("bottom", "mid"),
                     ("bottom", "left"), ("mid", "left"), ("top", "left")]
            rk, ck = table[d]
            buf = torch.empty_like(out[:, :, rows[rk], cols[ck]]).contiguous()
            recvs.append((rows[rk], cols[ck], buf))
            ops.append(CF.P2POp("irecv", buf, peer, self.group))
        if ops:
            CF.batch_isend_irecv(ops)
        for rs, cs, buf in recvs:
            out[:, :, rs, cs] = buf
        return out


class _AllSwap(_CommPrimitive):
    """All-to-all with per-peer element counts: ``send_size[i]`` elements of the flat input go to rank i and
    ``recv_size[i]`` elements arrive from rank i (ops/operations/comm_ops.py:741)."""

    def __init__(self, group=None):
        super().__init__("_AllSwap")
        self._init_group(group)

    def _run(self, x, send_size, recv_size):
        send = [int(v) for v in (send_size.tolist() if isinstance(send_size, torch.Tensor) else send_size)]
        recv = [int(v) for v in (recv_size.tolist() if isinstance(recv_size, torch.Tensor) else recv_size)]
        return CF.all_to_all_single_with_output_shape((sum(recv),) + tuple(x.shape[1:]), x, recv, send, self.group)


class CollectiveScatter(_CommPrimitive):
    def __init__(self, src_rank=0, group=None):
        super().__init__("CollectiveScatter")
        self.src_rank = src_rank
        self._init_group(group)

    def _run(self, x):
        return CF.scatter_tensor(x, self.src_rank, self.group)


class CollectiveGather(_CommPrimitive):
    def __init__(self, dest_rank=0, group=None):
        super().__init__("CollectiveGather")
        self.dest_rank = dest_rank
        self._init_group(group)

    def _run(self, x):
        return CF.gather_into_tensor(x, self.dest_rank, self.group)


class Barrier(_CommPrimitive):
    def __init__(self, group=None):
        super().__init__("Barrier")
        self._init_group(group)

    def _run(self):
        CF.barrier(self.group)


class _SendFn(torch.autograd.Function):
    """Send forward / Receive backward.  Returns a zero-size token so that autograd can reach the op."""

    @staticmethod
    def forward(ctx, x, dest, gname, tag):
        ctx.meta = (dest, gname, tag, x.shape, x.dtype, x.device)
        g = M._group(gname)
        if not M.is_simulation():
            dist.send(x.contiguous(), M.get_world_rank_from_group_rank(gname, dest) if g.size != M._state.world
                      else dest, group=g.pg, tag=tag)
        return x.new_zeros(())

    @staticmethod
    def backward(ctx, _d):
        dest, gname, tag, shape, dtype, device = ctx.meta
        g = M._group(gname)
        dx = torch.zeros(shape, dtype=dtype, device=device)
        if not M.is_simulation():
            dist.recv(dx, M.get_world_rank_from_group_rank(gname, dest) if g.size != M._state.world else dest,
                      group=g.pg, tag=tag)
        return dx, None, None, None


class _RecvFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, token, src, gname, tag, shape, dtype, device):
        ctx.meta = (src, gname, tag)
        g = M._group(gname)
        out = torch.zeros(shape, dtype=dtype, device=device)
        if not M.is_simulation():
            dist.recv(out, M.get_world_rank_from_group_rank(gname, src) if g.size != M._state.world else src,
                      group=g.pg, tag=tag)
        return out

    @staticmethod
    def backward(ctx, dy):
        src, gname, tag = ctx.meta
        g = M._group(gname)
        if not M.is_simulation():
            dist.send(dy.contiguous(), M.get_world_rank_from_group_rank(gname, src) if g.size != M._state.world
                      else src, group=g.pg, tag=tag)
        return dy.new_zeros(()), None, None, None, None, None, None


class Send(_CommPrimitive):
    def __init__(self, sr_tag, dest_rank, group=None, group_back=None):
        super().__init__("Send")
        self.sr_tag, self.dest_rank = sr_tag, dest_rank
        self._init_group(group)
        self.add_prim_attr("sr_tag", sr_tag)
        self.add_prim_attr("dest_rank", dest_rank)

    def _run(self, x):
        return _SendFn.apply(x, self.dest_rank, self.group, self.sr_tag)


class Receive(_CommPrimitive):
    def __init__(self, sr_tag, src_rank, shape, dtype, group=None, group_back=None):
        super().__init__("Receive")
        self.sr_tag, self.src_rank, self.shape, self.dtype = sr_tag, src_rank, tuple(shape), dtype
        self._init_group(group)
        self.add_prim_attr("sr_tag", sr_tag)
        self.add_prim_attr("src_rank", src_rank)

    def _run(self, token=None):
        from .. import context
        dev = context.device()
        if token is None:
            token = torch.zeros((), device=dev, requires_grad=torch.is_grad_enabled())
        return _RecvFn.apply(token, self.src_rank, self.group, self.sr_tag, self.shape, self.dtype, dev)


class BatchISendIRecv(_CommPrimitive):
    def __init__(self, op_types, remote_ranks, receive_shapes=None, receive_dtypes=None, group=None):
        super().__init__("BatchISendIRecv")
        self._init_group(group)
        self.op_types, self.remote_ranks = list(op_types), list(remote_ranks)
        self.receive_shapes, self.receive_dtypes = receive_shapes or [], receive_dtypes or []

    def _run(self, xs):
        ops, si, ri = [], 0, 0
        dev = xs[0].device if xs else None
        for t, r in zip(self.op_types, self.remote_ranks):
            if t == "isend":
                ops.append(CF.P2POp("isend", xs[si], r, self.group))
                si += 1
            else:
                buf = torch.empty(tuple(self.receive_shapes[ri]), dtype=self.receive_dtypes[ri], device=dev)
                ops.append(CF.P2POp("irecv", buf, r, self.group))
                ri += 1
        return CF.batch_isend_irecv(ops)


# ------------------------------------------------------------------------------------ planner-internal ops
class _MirrorFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, gname, dev_num, mean_flag):
        ctx.meta = (gname, dev_num, mean_flag)
        return x.view_as(x)

    @staticmethod
    def backward(ctx, dy):
        gname, dev_num, mean_flag = ctx.meta
        d = CF._all_reduce_(dy.clone(), "sum", M._group(gname))
        if mean_flag:
            d = d / dev_num
        return d, None, None, None


class _MirrorOperator(_CommPrimitive):
    """Identity on a replicated parameter; its gradient is all-reduced over the replica group."""

    def __init__(self, group=None, dev_num=None, mean_flag=None):
        super().__init__("_MirrorOperator")
        self._init_group(group)
        self.dev_num = dev_num if dev_num is not None else self.rank_size
        self.mean_flag = bool(mean_flag)
        self.add_prim_attr("dev_num", self.dev_num)
        self.add_prim_attr("mean_flag", self.mean_flag)

    def _run(self, x):
        return _MirrorFn.apply(x, self.group, self.dev_num, self.mean_flag)


class _MirrorMicroFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, accu, prim):
        ctx.prim, ctx.accu = prim, accu
        return x.view_as(x)

    @staticmethod
    def backward(ctx, dy):
        # accumulate; the step cell all-reduces the accumulator once per optimizer step
        with torch.no_grad():
            torch.Tensor.add_(ctx.accu, dy.to(ctx.accu.dtype))
        return torch.zeros_like(dy), None, None


class _MirrorMicroStepOperator(_MirrorOperator):
    def __init__(self, group=None, dev_num=None, mean_flag=None):
        super().__init__(group, dev_num, mean_flag)
        self.name = "_MirrorMicroStepOperator"

    def _run(self, x, accu):
        return _MirrorMicroFn.apply(x, accu, self)


_MirrorMiniStepOperator = _MirrorMicroStepOperator


class _MicroStepAllGather(AllGather):
    """AllGather of an optimizer-sharded weight under gradient accumulation: backward accumulates the full
    gradient and the ReduceScatter runs once per step on the accumulator (grad_comm_ops.py:308-345)."""

    def __init__(self, group=None, mean_flag=None):
        super().__init__(group)
        self.name = "_MicroStepAllGather"
        self.add_prim_attr("mean_flag", bool(mean_flag))

    def _run(self, x, accu=None):
        out = CF._all_gather(x.detach(), M._group(self.group))
        if accu is None or not torch.is_grad_enabled():
            return CF.all_gather_autograd(x, self.group, bool(self.attrs["mean_flag"]))
        return _MicroGatherFn.apply(x, out, accu)


_MiniStepAllGather = _MicroStepAllGather


class _MicroGatherFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, gathered, accu):
        ctx.accu = accu
        ctx.shape = x.shape
        return gathered

    @staticmethod
    def backward(ctx, dy):
        with torch.no_grad():
            torch.Tensor.add_(ctx.accu, dy.to(ctx.accu.dtype))
        return dy.new_zeros(ctx.shape), None, None


class _DivFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, divisor):
        ctx.divisor = divisor
        return x.view_as(x)

    @staticmethod
    def backward(ctx, dy):
        return dy / ctx.divisor, None


class _VirtualDiv(Primitive):
    def __init__(self, divisor=None):
        super().__init__("_VirtualDiv")
        self.divisor = divisor
        self.add_prim_attr("divisor", divisor)

    def _run(self, x):
        return _DivFn.apply(x, float(self.divisor))


class _VirtualAdd(Primitive):
    def __init__(self):
        super().__init__("_VirtualAdd")

    def _run(self, x, y):
        return x


class _VirtualDataset(Primitive):
    def __init__(self):
        super().__init__("_VirtualDataset")

    def _run(self, *args):
        return args[0] if len(args) == 1 else args


class _VirtualOutput(Primitive):
    def __init__(self):
        super().__init__("_VirtualOutput")

    def _run(self, x):
        return x


class _VirtualPipelineEnd(Primitive):
    def __init__(self):
        super().__init__("_VirtualPipelineEnd")

    def _run(self, x):
        return x


class _AccuFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, accu):
        ctx.accu = accu
        return x.view_as(x)

    @staticmethod
    def backward(ctx, dy):
        with torch.no_grad():
            torch.Tensor.add_(ctx.accu, dy.to(ctx.accu.dtype))
        return torch.zeros_like(dy), None


class _VirtualAssignAdd(Primitive):
    def __init__(self):
        super().__init__("_VirtualAssignAdd")

    def _run(self, x, accu):
        return _AccuFn.apply(x, accu)


class _VirtualAccuGrad(Primitive):
    def __init__(self):
        super().__init__("_VirtualAccuGrad")

    def _run(self, x, accu):
        return x


class _GetTensorSlice(Primitive):
    def __init__(self):
        super().__init__("_GetTensorSlice")

    def _run(self, x, dev_mat, tensor_map, slice_shape=None, rank=None):
        from ..parallel.layout import TensorLayout, slice_for_rank
        from .. import context
        layout = TensorLayout(tuple(dev_mat), tuple(tensor_map), tuple(x.shape))
        r = context.get_auto_parallel_context("global_rank") if rank is None else rank
        return slice_for_rank(x, layout, r)


class AShardIdentity(Primitive):
    def __init__(self):
        super().__init__("AShardIdentity")

    def _run(self, x):
        return x


class _HostAllGather(AllGather):
    pass


class _HostReduceScatter(ReduceScatter):
    pass


__all__ = ["ReduceOp", "AllReduce", "AllGather", "ReduceScatter", "Broadcast", "Reduce", "AlltoAll", "AlltoAllV",
           "NeighborExchange", "CollectiveScatter", "CollectiveGather", "Barrier", "Send", "Receive",
           "BatchISendIRecv", "_MirrorOperator", "_MirrorMicroStepOperator", "_MirrorMiniStepOperator",
           "_MicroStepAllGather", "_MiniStepAllGather", "_VirtualDiv", "_VirtualAdd", "_VirtualDataset",
           "_VirtualOutput", "_VirtualPipelineEnd", "_VirtualAssignAdd", "_VirtualAccuGrad", "_GetTensorSlice",
           "AShardIdentity", "_HostAllGather", "_HostReduceScatter"]
