"""Mixture of experts with expert parallelism.

Routing follows the reference's ``TopkRouter`` exactly (python/mindspore/parallel/_transformer/moe.py:604-693:
softmax, k rounds of arg-max with the kept choices masked, capacity ``ceil(k * tokens * factor / experts)``,
position by token order, load-balance loss per round, weights normalised over the rounds), but tokens are moved as
rows, not multiplied by one-hot dispatch / combine tensors:

* the router is one kernel per round (``csrc/cuda/moe.cu``) plus a backward kernel;
* dispatch stores each kept row straight into the owner rank's expert input buffer and combine pulls the expert
  outputs back and applies the weights - over NVLink peer memory when the expert-parallel group has a symmetric-
  memory context, which replaces the AlltoAll pair of the reference; the NCCL ``all_to_all`` form is the selectable
  baseline (and the gloo path on CPU);
* the expert FFN is a batched tcgen05 GEMM over ``[local experts, sources * capacity, hidden]``.

``MoE``, ``MoEConfig`` and ``calculate_expert_capacity`` keep the reference's names and arguments
(moe.py:42, :137, :143)."""
from __future__ import annotations

import ctypes
import math
import os

import torch

from .. import _native
from ..common.initializer import initializer
from ..common.parameter import Parameter
from ..nn.cell import Cell
from ..ops import fused
from ..ops.kernels import _count, _p, _stream

_P, _I, _F = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
_U64P = ctypes.POINTER(ctypes.c_ulonglong)
_native.register_cuda_signature("msb_moe_router_step", _I, [_P] * 10 + [_I] * 5 + [_P])
_native.register_cuda_signature("msb_moe_router_weights", _I, [_P, _P, _I, _I, _P])
_native.register_cuda_signature("msb_moe_router_bwd", _I, [_P] * 8 + [_I, _I, _I, _P])
_native.register_cuda_signature("msb_moe_scatter_rows", _I, [_P, _P, _P, _P, _U64P] + [_I] * 7 + [_P])
_native.register_cuda_signature("msb_moe_gather_rows", _I, [_U64P, _P, _P, _P, _P, _P, _P] + [_I] * 7 + [_P])


class MoEConfig:
    def __init__(self, expert_num=1, capacity_factor=1.1, aux_loss_factor=0.05, num_experts_chosen=1,
                 expert_group_size=None, group_wise_a2a=False, comp_comm_parallel=False, comp_comm_parallel_degree=2):
        for name, v in (("expert_num", expert_num), ("num_experts_chosen", num_experts_chosen),
                        ("comp_comm_parallel_degree", comp_comm_parallel_degree)):
            if not isinstance(v, int) or isinstance(v, bool) or v <= 0:
                raise TypeError("'%s' must be a positive int, but got %r" % (name, v))
        if capacity_factor < 1.0:
            raise ValueError("'capacity_factor' must be equal to or greater than 1.0, but got %s." % capacity_factor)
        if aux_loss_factor >= 1.0:
            raise ValueError("'aux_loss_factor' must be less than 1.0, but got %s." % aux_loss_factor)
        if num_experts_chosen > expert_num:
            raise ValueError("'num_experts_chosen' must not be larger than 'expert_num', but got %d."
                             % num_experts_chosen)
        self.expert_num, self.capacity_factor, self.aux_loss_factor = expert_num, capacity_factor, aux_loss_factor
        self.num_experts_chosen, self.expert_group_size = num_experts_chosen, expert_group_size
        self.group_wise_a2a, self.comp_comm_parallel = group_wise_a2a, comp_comm_parallel
        self.comp_comm_parallel_degree = comp_comm_parallel_degree


default_moe_config = MoEConfig()


def calculate_expert_capacity(k, tokens_per_group, capacity_factor, expert_dim):
    res = k * tokens_per_group * capacity_factor / expert_dim
    res_int = int(res)
    return res_int if res < 0 or res == res_int else res_int + 1


# ------------------------------------------------------------------------------------------------ router
def router_reference(logits, k, capacity):
    """The routing arithmetic in plain torch (differentiable): returns expert [T,k] int32, slot [T,k] int32
    (-1 = dropped), weight [T,k] fp32, load-balance loss (scalar)."""
    T, E = logits.shape
    prob = torch.softmax(logits.float(), dim=-1)
    accum_mask = torch.zeros_like(prob)
    fill = torch.zeros(E, dtype=torch.long, device=logits.device)
    loss = prob.new_zeros(())
    experts, slots, gates = [], [], []
    for _ in range(k):
        prob = prob * (1 - accum_mask)
        gate, idx = prob.max(dim=-1)
        mask = torch.nn.functional.one_hot(idx, E).to(prob.dtype)
        prob_normal = prob / (prob.sum(-1, keepdim=True) + 1e-9)
        loss = loss + (mask.mean(0) * prob_normal.mean(0)).mean() * E * E
        position = (torch.cumsum(mask, 0) - mask).long() + fill       # exclusive count in token order
        pos = position.gather(1, idx[:, None])[:, 0]
        keep = pos < capacity
        kept_mask = mask * keep[:, None].to(mask.dtype)
        accum_mask = accum_mask + kept_mask
        fill = fill + kept_mask.sum(0).long()
        experts.append(idx)
        slots.append(torch.where(keep, pos, torch.full_like(pos, -1)))
        gates.append(gate * keep.to(gate.dtype))
    gate = torch.stack(gates, 1)
    weight = gate / (gate.sum(-1, keepdim=True) + 1e-9) if k > 1 else gate
    return torch.stack(experts, 1).int(), torch.stack(slots, 1).int(), weight, loss


class _RouterFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, k, capacity):
        T, E = logits.shape
        dev = logits.device
        logits = logits.float().contiguous()
        expert = torch.empty((T, k), dtype=torch.int32, device=dev)
        slot = torch.empty((T, k), dtype=torch.int32, device=dev)
        gate = torch.empty((T, k), dtype=torch.float32, device=dev)
        weight = torch.empty((T, k), dtype=torch.float32, device=dev)
        fill = torch.zeros(E, dtype=torch.int32, device=dev)
        proxy = torch.zeros(E, dtype=torch.float32, device=dev)
        density = torch.empty((k, E), dtype=torch.float32, device=dev)
        loss = torch.zeros((), dtype=torch.float32, device=dev)
        blocks = (T + 255) // 256
        scan = torch.empty(blocks * E, dtype=torch.int64, device=dev)
        ticket = torch.empty(1, dtype=torch.int32, device=dev)
        lib = _native.cuda()
        for step in range(k):
            rc = lib.msb_moe_router_step(_p(logits), _p(expert), _p(slot), _p(gate), _p(fill), _p(proxy), _p(density),
                                         _p(loss), _p(scan), _p(ticket), T, E, k, step, capacity, _stream())
            _native.check(rc, "moe_router_step")
            _count(2)
        _native.check(lib.msb_moe_router_weights(_p(gate), _p(weight), T, k, _stream()), "moe_router_weights")
        _count()
        ctx.save_for_backward(logits, expert, slot, gate, density)
        ctx.mark_non_differentiable(expert, slot)
        return expert, slot, weight, loss

    @staticmethod
    def backward(ctx, _de, _ds, dweight, dloss):
        logits, expert, slot, gate, density = ctx.saved_tensors
        T, E = logits.shape
        k = expert.shape[1]
        dlogits = torch.empty_like(logits)
        dweight = dweight.float().contiguous() if dweight is not None else torch.zeros_like(gate)
        dloss = dloss.float().contiguous() if dloss is not None else None
        rc = _native.cuda().msb_moe_router_bwd(_p(logits), _p(expert), _p(slot), _p(gate), _p(dweight), _p(dloss),
                                               _p(density), _p(dlogits), T, E, k, _stream())
        _native.check(rc, "moe_router_bwd")
        _count()
        return dlogits, None, None


def route(logits, k, capacity):
    """expert, slot, weight, loss for router logits [T, E] (kernel on CUDA, torch elsewhere)."""
    if logits.is_cuda and _native.cuda() is not None and logits.shape[1] <= 256 and k <= 4:
        return _RouterFn.apply(logits, k, capacity)
    return router_reference(logits, k, capacity)


# ------------------------------------------------------------------------------------------------ token movement
def _ptr_array(ptrs):
    arr = (ctypes.c_ulonglong * 8)()
    for i, p in enumerate(ptrs):
        arr[i] = int(p)
    return arr


class _TorchTransport:
    """Rows moved with torch indexing; across ranks with ``all_to_all_single`` (NCCL or gloo).  The un-fused
    baseline of the kernel transport and the CPU path."""

    def __init__(self, experts, capacity, group=None):
        self.group = group                                   # communication.management._Group or None
        self.ep = group.size if group is not None else 1
        self.me = group.ranks.index(torch.distributed.get_rank()) if group is not None else 0
        self.E, self.EL, self.C = experts, experts // self.ep, capacity

    def _flat_index(self, expert, slot):
        """Row index into the send layout [ep_dst, EL, C] (kept choices only) + mask."""
        keep = slot >= 0
        idx = (expert.long() * self.C + slot.long().clamp(min=0))      # expert = dst_rank * EL + e_local
        return idx, keep

    def _exchange(self, buf):
        """[ep_dst, EL, C, H] on every rank -> [EL, ep_src, C, H]."""
        if self.ep == 1:
            return buf.permute(1, 0, 2, 3).contiguous()
        out = torch.empty_like(buf)
        torch.distributed.all_to_all_single(out, buf.contiguous(), group=self.group.pg)
        return out.permute(1, 0, 2, 3).contiguous()

    def _exchange_back(self, buf):
        """[EL, ep_src, C, H] -> [ep_owner, EL, C, H] back on the source ranks."""
        send = buf.permute(1, 0, 2, 3).contiguous()
        if self.ep == 1:
            return send
        out = torch.empty_like(send)
        torch.distributed.all_to_all_single(out, send, group=self.group.pg)
        return out

    def scatter(self, src, scale, expert, slot):
        T, H = src.shape
        idx, keep = self._flat_index(expert, slot)
        rows = src[:, None, :].expand(T, expert.shape[1], H)
        if scale is not None:
            rows = rows * scale[:, :, None].to(src.dtype)
        send = src.new_zeros((self.ep * self.EL * self.C, H))
        send.index_put_((idx[keep],), rows[keep].to(src.dtype))
        return self._exchange(send.view(self.ep, self.EL, self.C, H))

    def gather(self, buf, scale, expert, slot, g=None, want_out=True):
        H = buf.shape[-1]
        back = self._exchange_back(buf).reshape(-1, H)
        idx, keep = self._flat_index(expert, slot)
        rows = back[idx] * keep[:, :, None].to(back.dtype)                # [T, K, H]
        out = None
        if want_out:
            w = scale if scale is not None else keep.to(torch.float32)
            out = (rows.float() * w[:, :, None]).sum(1).to(buf.dtype)
        dots = (rows.float() * g[:, None, :].float()).sum(-1) if g is not None else None
        return out, dots


class _KernelTransport:
    """Rows moved by the scatter / gather kernels: peer stores into, and peer loads from, the owners' buffers in
    symmetric memory (or plain device memory when the group is a single rank)."""

    def __init__(self, experts, capacity, group=None, symm=None):
        self.symm = symm                                     # fused_comm.SymmContext or None (single rank)
        self.ep = symm.world if symm is not None else 1
        self.me = symm.rank if symm is not None else 0
        self.E, self.EL, self.C = experts, experts // self.ep, capacity

    def _buffer(self, tag, H, dtype, device):
        n = self.EL * self.ep * self.C * H
        if self.symm is None:
            buf = torch.empty(n, dtype=dtype, device=device)
            return buf, [buf.data_ptr()]
        raw, ptrs = self.symm.buffer(self.symm._next("moe_" + tag), n * 2)
        return raw[:n * 2].view(dtype), ptrs

    def _barrier(self):
        if self.symm is not None:
            self.symm.barrier(1)

    def scatter(self, src, scale, expert, slot):
        T, H = src.shape
        buf, ptrs = self._buffer("in", H, src.dtype, src.device)
        buf.zero_()
        self._barrier()                                      # every owner's buffer is clear
        rc = _native.cuda().msb_moe_scatter_rows(_p(src), _p(scale), _p(expert), _p(slot), _ptr_array(ptrs), T,
                                                 expert.shape[1], H, self.EL, self.ep, self.me, self.C, _stream())
        _native.check(rc, "moe_scatter_rows")
        _count()
        self._barrier()                                      # every source has stored its rows
        out = buf.view(self.EL, self.ep, self.C, H)
        # the symmetric buffer is recycled two operations later, but backward still needs these rows: hand out a copy
        return out.clone() if self.symm is not None else out

    def gather(self, buf, scale, expert, slot, g=None, want_out=True):
        T, K = expert.shape
        H = buf.shape[-1]
        if self.symm is not None:
            stage, ptrs = self._buffer("out", H, buf.dtype, buf.device)
            stage.view(buf.shape).copy_(buf)
            self._barrier()                                  # every owner has published its rows
        else:
            buf = buf.contiguous()
            ptrs = [buf.data_ptr()]
        out = torch.empty((T, H), dtype=buf.dtype, device=buf.device) if want_out else None
        dots = torch.empty((T, K), dtype=torch.float32, device=buf.device) if g is not None else None
        rc = _native.cuda().msb_moe_gather_rows(_ptr_array(ptrs), _p(scale), _p(expert), _p(slot), _p(g), _p(out),
                                                _p(dots), T, K, H, self.EL, self.ep, self.me, self.C, _stream())
        _native.check(rc, "moe_gather_rows")
        _count()
        return out, dots


class _DispatchFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, expert, slot, transport):
        ctx.transport = transport
        ctx.save_for_backward(expert, slot)
        return transport.scatter(x.contiguous(), None, expert, slot)

    @staticmethod
    def backward(ctx, dbuf):
        expert, slot = ctx.saved_tensors
        dx, _ = ctx.transport.gather(dbuf.contiguous(), None, expert, slot)
        return dx, None, None, None


class _CombineFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ybuf, weight, expert, slot, transport):
        ctx.transport = transport
        ctx.save_for_backward(ybuf, weight, expert, slot)
        out, _ = transport.gather(ybuf.contiguous(), weight.float().contiguous(), expert, slot)
        return out

    @staticmethod
    def backward(ctx, dout):
        ybuf, weight, expert, slot = ctx.saved_tensors
        dout = dout.contiguous()
        _, dweight = ctx.transport.gather(ybuf.contiguous(), None, expert, slot, g=dout, want_out=False)
        dybuf = ctx.transport.scatter(dout, weight.float().contiguous(), expert, slot)
        return dybuf, dweight.to(weight.dtype), None, None, None


class TopkRouter(Cell):
    """Maps router logits to the dense dispatch / combine tensors of the GShard formulation.

    ``construct(router_logits [..., T, E])`` returns ``(dispatch [..., T, E, C], combine [..., T, E, C], loss)``:
    ``dispatch[t, e, c] = 1`` when token t sits in slot c of expert e, ``combine`` carries the normalised gate there,
    ``loss`` is the load-balance loss (not yet multiplied by ``aux_loss_factor``), averaged over the leading groups.
    Every leading index is one routing group with its own capacity, as in the reference
    (python/mindspore/parallel/_transformer/moe.py:476).  ``MoE`` uses the index form (``route``) directly and never
    builds these tensors."""

    def __init__(self, d_model, moe_config, training=True, parallel_config=None):
        super().__init__()
        self.d_model = d_model
        self.expert_dim = moe_config.expert_num
        self.capacity_factor = moe_config.capacity_factor
        self.num_experts_chosen = moe_config.num_experts_chosen
        self.training = training

    def construct(self, router_logits):
        logits = router_logits.as_subclass(torch.Tensor)
        lead, (T, E) = logits.shape[:-2], logits.shape[-2:]
        k = self.num_experts_chosen
        capacity = calculate_expert_capacity(k, T, self.capacity_factor, E)
        groups = logits.reshape(-1, T, E)
        dispatch, combine, losses = [], [], []
        for g in groups:
            expert, slot, weight, loss = route(g, k, capacity)
            kept = slot >= 0
            flat = (expert.long() * capacity + slot.clamp(min=0).long())          # [T, k] position in E * C
            onehot = torch.nn.functional.one_hot(flat, E * capacity).to(weight.dtype) * kept[..., None]
            dispatch.append(onehot.sum(1).reshape(T, E, capacity))
            combine.append((onehot * weight[..., None]).sum(1).reshape(T, E, capacity))
            losses.append(loss)
        from ..common.tensor import as_tensor
        shape = tuple(lead) + (T, E, capacity)
        return (as_tensor(torch.stack(dispatch).reshape(shape)), as_tensor(torch.stack(combine).reshape(shape)),
                as_tensor(torch.stack(losses).mean()))


class Router(Cell):
    """Router backbone: a bias-free Dense producing one logit per expert (computed in fp32), followed by the
    routing policy (``TopkRouter`` unless ``routing_policy`` is given).  Parity: moe.py:412."""

    def __init__(self, d_model, moe_config, routing_policy=None, training=True, parallel_config=None):
        super().__init__()
        self.d_model, self.expert_dim = d_model, moe_config.expert_num
        self.weight = Parameter(initializer("normal", (self.expert_dim, d_model), torch.float32), name="dense.weight")
        self.router = routing_policy if routing_policy is not None else \
            TopkRouter(d_model, moe_config, training, parallel_config)

    def construct(self, input_tensor):
        x = input_tensor.as_subclass(torch.Tensor).float()
        return self.router(torch.nn.functional.linear(x, self.weight.as_subclass(torch.Tensor).float()))


# ------------------------------------------------------------------------------------------------ GEMMs fused with the exchange
class _FusedExchange:
    """The expert GEMMs as the consumers / producers of the row exchange over symmetric memory.

    * gather form (dispatch -> first GEMM, and the backward of the second): every rank scatters its rows locally
      into an [experts][capacity][H] send buffer in symmetric memory; the owner of expert e multiplies
      ``gather_r(send_r[e]) @ W`` with the AllGather -> MatMul kernel, which pulls rank r's block while it multiplies
      the blocks that have arrived.
    * push form (second GEMM -> combine, and the backward of the first): the MatMul epilogue stores row block r of
      the expert's product straight into slot e of rank r's [experts][capacity][H] receive buffer; after a barrier
      every rank combines its own rows locally.

    Needs capacity % 128 == 0 (a row block is a whole number of GEMM tiles) and bf16."""

    def __init__(self, tr):
        self.tr, self.ctx = tr, tr.symm
        self.E, self.EL, self.C, self.ep, self.me = tr.E, tr.EL, tr.C, tr.ep, tr.me

    def _buf(self, tag, H, device):
        n = self.E * self.C * H
        raw, ptrs = self.ctx.buffer(self.ctx._next("moe_" + tag), n * 2)
        return raw[:n * 2].view(torch.bfloat16), ptrs

    def _local(self, fn_name, *args):
        rc = getattr(_native.cuda(), fn_name)(*args)
        _native.check(rc, fn_name[4:])
        _count()

    def publish(self, src, scale, expert, slot):
        """Local scatter of this rank's rows into a zeroed send buffer; returns the buffer's addresses on every rank
        after the barrier that makes it readable."""
        T, H = src.shape
        buf, ptrs = self._buf("send", H, src.device)
        buf.zero_()
        self._local("msb_moe_scatter_rows", _p(src), _p(scale), _p(expert), _p(slot), _ptr_array([buf.data_ptr()]), T,
                    expert.shape[1], H, self.E, 1, 0, self.C, _stream())
        self.ctx.barrier(1)
        return ptrs

    def gather_gemm(self, ptrs, H, w, b_mn, bias):
        """[EL, ep * C, N] = gathered rows of each local expert times its weight; also returns the gathered rows."""
        from . import fused_comm
        K_ = w.shape[1] if b_mn else w.shape[2]
        N_ = w.shape[2] if b_mn else w.shape[1]
        M_ = self.ep * self.C
        assert K_ == H
        out = torch.empty((self.EL, M_, N_), dtype=torch.bfloat16, device=w.device)
        rows = torch.empty((self.EL, M_, H), dtype=torch.bfloat16, device=w.device)
        for le in range(self.EL):
            off = (self.me * self.EL + le) * self.C * H * 2
            fused_comm.gemm_gather_rows(self.ctx, [p + off for p in ptrs], self.C, w[le], b_mn,
                                        bias[le].reshape(-1) if bias is not None else None, out[le], rows[le])
        return out, rows

    def push_gemm(self, a, w, b_mn, bias, N):
        """Each local expert's product goes to the ranks its rows came from; returns this rank's received
        [E, C, N] rows (a view of the receive buffer: copy what must outlive the next two exchanges)."""
        from . import fused_comm
        buf, ptrs = self._buf("recv", N, a.device)
        for le in range(self.EL):
            fused_comm.gemm_push_rows(self.ctx, a[le], w[le], b_mn, ptrs, self.me * self.EL + le, self.E,
                                      bias[le].reshape(-1) if bias is not None else None)
        self.ctx.barrier(1)
        return buf.view(self.E, self.C, N)

    def combine(self, ybuf, scale, expert, slot, g=None, want_out=True):
        T, K = expert.shape
        H = ybuf.shape[-1]
        out = torch.empty((T, H), dtype=ybuf.dtype, device=ybuf.device) if want_out else None
        dots = torch.empty((T, K), dtype=torch.float32, device=ybuf.device) if g is not None else None
        self._local("msb_moe_gather_rows", _ptr_array([ybuf.data_ptr()]), _p(scale), _p(expert), _p(slot), _p(g),
                    _p(out), _p(dots), T, K, H, self.E, 1, 0, self.C, _stream())
        return out, dots


class _DispatchGemmFn(torch.autograd.Function):
    """h[le] = dispatch(x)[le] @ w1[le] + b1[le]: the row exchange runs inside the GEMM (gather form)."""

    @staticmethod
    def forward(ctx, x, w1, b1, expert, slot, fx):
        x = x.contiguous()
        ptrs = fx.publish(x, None, expert, slot)
        h, rows = fx.gather_gemm(ptrs, x.shape[1], w1, True, b1)
        ctx.fx, ctx.has_bias = fx, b1 is not None
        ctx.save_for_backward(rows, w1, expert, slot)
        return h

    @staticmethod
    def backward(ctx, dh):
        rows, w1, expert, slot = ctx.saved_tensors
        fx = ctx.fx
        dh = dh.contiguous()
        dw1 = fused.matmul(rows, dh, transpose_a=True) if ctx.needs_input_grad[1] else None
        db1 = dh.sum(1, keepdim=True) if ctx.has_bias and ctx.needs_input_grad[2] else None
        dx = None
        if ctx.needs_input_grad[0]:
            recv = fx.push_gemm(dh, w1, False, None, w1.shape[1])          # dh @ w1^T, rows back to their sources
            dx, _ = fx.combine(recv, None, expert, slot)
        return dx, dw1, db1, None, None, None


class _GemmCombineFn(torch.autograd.Function):
    """out = combine(h[le] @ w2[le] + b2[le]): the GEMM's epilogue delivers the rows (push form)."""

    @staticmethod
    def forward(ctx, h, w2, b2, weight, expert, slot, fx):
        h = h.contiguous()
        ctx.weight_dtype = weight.dtype
        weight = weight.float().contiguous()
        ybuf = fx.push_gemm(h, w2, True, b2, w2.shape[2]).clone()
        out, _ = fx.combine(ybuf, weight, expert, slot)
        ctx.fx, ctx.has_bias = fx, b2 is not None
        ctx.save_for_backward(h, w2, ybuf, weight, expert, slot)
        return out

    @staticmethod
    def backward(ctx, dout):
        h, w2, ybuf, weight, expert, slot = ctx.saved_tensors
        fx = ctx.fx
        dout = dout.contiguous()
        _, dweight = fx.combine(ybuf, None, expert, slot, g=dout, want_out=False)
        ptrs = fx.publish(dout, weight, expert, slot)
        dh, dy = fx.gather_gemm(ptrs, dout.shape[1], w2, False, None)      # gather(weight * dout) @ w2^T
        dw2 = fused.matmul(h, dy, transpose_a=True) if ctx.needs_input_grad[1] else None
        db2 = dy.sum(1, keepdim=True) if ctx.has_bias and ctx.needs_input_grad[2] else None
        return dh, dw2, db2, dweight.to(ctx.weight_dtype), None, None, None


# ------------------------------------------------------------------------------------------------ the layer
def _pick_transport(experts, capacity, group, device, fused=True):
    """Kernel transport on CUDA (over symmetric memory when the group has several ranks), torch otherwise."""
    if device.type == "cuda" and _native.cuda() is not None and fused:
        if group is None or group.size == 1:
            return _KernelTransport(experts, capacity)
        from . import fused_comm
        symm = fused_comm.get_context(group)
        if symm is not None:
            return _KernelTransport(experts, capacity, group, symm)
    return _TorchTransport(experts, capacity, group if group is not None and group.size > 1 else None)


class MoE(Cell):
    """Mixture-of-experts feed-forward layer.

    Args follow the reference (``hidden_size, ffn_hidden_size, dropout_rate, hidden_act, param_init_type,
    moe_config, parallel_config``); ``expert_parallel_group`` names the communication group whose ranks share the
    experts (each holds ``expert_num / group size`` of them and routes its own tokens).  ``construct(x)`` takes
    ``[batch, seq, hidden]`` or ``[tokens, hidden]`` and returns ``(output, aux_loss)`` with
    ``aux_loss = aux_loss_factor * load-balance loss``."""

    def __init__(self, hidden_size, ffn_hidden_size, dropout_rate=0.0, hidden_act="gelu",
                 param_init_type=torch.float32, moe_config=default_moe_config, parallel_config=None,
                 expert_parallel_group=None, has_bias=True, fused_transport=True):
        super().__init__()
        from ..communication import management as M
        self.hidden_size, self.ffn_hidden_size = hidden_size, ffn_hidden_size
        self.cfg = moe_config
        self.E, self.k = moe_config.expert_num, moe_config.num_experts_chosen
        self.act = hidden_act
        self.fused_transport = fused_transport
        self.group = M._group(expert_parallel_group) if expert_parallel_group is not None and M.GlobalComm.INITED \
            else None
        ep = self.group.size if self.group is not None else 1
        if self.E % ep:
            raise ValueError("When using MoE, 'expert_num' (%d) must be a multiple of the expert-parallel group "
                             "size (%d)." % (self.E, ep))
        self.ep, self.EL = ep, self.E // ep
        self.ep_rank = self.group.ranks.index(M.get_rank()) if self.group is not None else 0
        up = ffn_hidden_size * (2 if hidden_act == "swiglu" else 1)
        mk = lambda shape, name, init="normal": Parameter(initializer(init, shape, param_init_type), name=name)
        # stored in the model's dtype (one optimizer arena, fp32 master there); the logits are computed in fp32
        self.router_weight = Parameter(initializer("normal", (self.E, hidden_size), param_init_type),
                                       name="router.dense.weight")
        self.w1 = mk((self.EL, hidden_size, up), "ffn.mapping.weight")
        self.w2 = mk((self.EL, ffn_hidden_size, hidden_size), "ffn.projection.weight")
        self.b1 = mk((self.EL, 1, up), "ffn.mapping.bias", "zeros") if has_bias else None
        self.b2 = mk((self.EL, 1, hidden_size), "ffn.projection.bias", "zeros") if has_bias else None
        for p in (self.w1, self.w2, self.b1, self.b2):
            if p is not None:
                p.dp_local = ep > 1            # every rank owns different experts: never all-reduced over the group
                p.expert_shard = (ep, self.ep_rank)
        self.dropout_rate = dropout_rate
        self._transports = {}
        self._exchanges = {}
        # MSB200_MOE_FUSED_GEMM=1 (or setting the attribute): the expert GEMMs run the row exchange themselves
        # (_FusedExchange).  Off by default: with 4 experts per rank on 2 ranks the batched GEMM between the scatter /
        # gather kernels measured 3 % faster than four GEMM launches that each gather or push their own rows.
        self.fused_gemm = os.environ.get("MSB200_MOE_FUSED_GEMM", "0") == "1"

    def _transport(self, capacity, device):
        key = (capacity, device)
        if key not in self._transports:
            self._transports[key] = _pick_transport(self.E, capacity, self.group, device, self.fused_transport)
        return self._transports[key]

    def _activation(self, h):
        if self.act == "swiglu":
            return fused.swiglu(h.reshape(-1, h.shape[-1])).reshape(*h.shape[:-1], h.shape[-1] // 2)
        if self.act == "gelu":
            return torch.nn.functional.gelu(h, approximate="tanh")
        if self.act == "relu":
            return torch.relu(h)
        if self.act in ("silu", "swish"):
            return torch.nn.functional.silu(h)
        raise ValueError("unsupported hidden_act %r" % (self.act,))

    def construct(self, x):
        shape = x.shape
        tokens = x.reshape(-1, shape[-1]).as_subclass(torch.Tensor)
        T = tokens.shape[0]
        logits = torch.nn.functional.linear(tokens.float(), self.router_weight.as_subclass(torch.Tensor).float())
        capacity = calculate_expert_capacity(self.k, T, self.cfg.capacity_factor, self.E)
        plain = lambda p: p.as_subclass(torch.Tensor) if p is not None else None
        w1, w2, b1, b2 = plain(self.w1), plain(self.w2), plain(self.b1), plain(self.b2)
        # expert GEMMs that run the row exchange themselves need whole GEMM tiles per (source rank, expert) block
        fuse_gemm = (self.ep > 1 and tokens.is_cuda and self.fused_transport and self.fused_gemm
                     and all(t is None or t.dtype == torch.bfloat16 for t in (tokens, w1, w2, b1, b2))
                     and all(d % 8 == 0 for d in (shape[-1], w1.shape[-1], w2.shape[-2])))
        if tokens.is_cuda:
            g = 128 if fuse_gemm else 8                # rows per expert stay a multiple of the GEMM granule
            capacity = (capacity + g - 1) // g * g
        expert, slot, weight, aux = route(logits, self.k, capacity)
        tr = self._transport(capacity, tokens.device)
        fuse_gemm = fuse_gemm and isinstance(tr, _KernelTransport) and tr.symm is not None
        if fuse_gemm:
            fx = self._exchanges.get(id(tr))
            if fx is None:
                fx = self._exchanges[id(tr)] = _FusedExchange(tr)
            h = _DispatchGemmFn.apply(tokens, w1, b1, expert, slot, fx)        # [EL, ep * C, up]
        else:
            buf = _DispatchFn.apply(tokens, expert, slot, tr)                 # [EL, ep, C, H]
            h = buf.reshape(self.EL, self.ep * capacity, shape[-1])
            h = fused.matmul(h, w1)
            if b1 is not None:
                h = h + b1
        h = self._activation(h)
        if self.dropout_rate > 0 and self.training:
            h = torch.nn.functional.dropout(h, self.dropout_rate)
        if fuse_gemm:
            out = _GemmCombineFn.apply(h, w2, b2, weight, expert, slot, fx)
        else:
            y = fused.matmul(h, w2)
            if b2 is not None:
                y = y + b2
            y = y.reshape(self.EL, self.ep, capacity, shape[-1])
            out = _CombineFn.apply(y, weight, expert, slot, tr)
        from ..common.tensor import as_tensor
        return as_tensor(out.reshape(shape)), as_tensor(aux * self.cfg.aux_loss_factor)


def moe_reference_forward(x, router_weight, w1, w2, b1, b2, k, capacity_factor, act="gelu"):
    """Dense GShard formulation on one device with all experts (one-hot dispatch and combine tensors, as the
    reference builds them): the oracle for tests."""
    T, H = x.shape
    E = router_weight.shape[0]
    capacity = calculate_expert_capacity(k, T, capacity_factor, E)
    logits = x.float() @ router_weight.float().t()
    expert, slot, weight, aux = router_reference(logits, k, capacity)
    combine = x.new_zeros((T, E, capacity), dtype=torch.float32)
    for j in range(k):
        keep = slot[:, j] >= 0
        ti = torch.nonzero(keep)[:, 0]
        combine[ti, expert[ti, j].long(), slot[ti, j].long()] = weight[ti, j]
    dispatch = (combine != 0).float()
    xin = torch.einsum("tec,th->ech", dispatch, x.float())
    h = torch.einsum("ech,ehf->ecf", xin, w1.float())
    if b1 is not None:
        h = h + b1.float()
    if act == "swiglu":
        f = h.shape[-1] // 2
        h = torch.nn.functional.silu(h[..., :f]) * h[..., f:]
    else:
        h = torch.nn.functional.gelu(h, approximate="tanh")
    y = torch.einsum("ecf,efh->ech", h, w2.float())
    if b2 is not None:
        y = y + b2.float()
    return torch.einsum("tec,ech->th", combine, y), aux
