"""Fused compute + collective operations over NVLink symmetric memory.

One ``SymmContext`` per communication group owns buffers that every rank of the group can address directly
(allocated with ``torch.distributed._symmetric_memory``, which exchanges the CUDA VMM handles once), the flag
pads of the stream-ordered group barrier, and the epoch counters.  The data movement itself is done by this
repository's own kernels:

* ``matmul_reduce_scatter``  - row-parallel Dense: the tcgen05 GEMM epilogue stores every output tile directly
  into the staging buffer of the rank that owns those token rows (peer stores over NVLink while later tiles are
  still being multiplied); after one barrier each rank sums its ``mp`` slots.  Backward = ``allgather_matmul``.
* ``allgather_matmul``       - column-parallel Dense: inside the GEMM kernel a copy warp per CTA pulls the peers'
  token shards with bulk copies into the local gathered operand, chunk by chunk, while the MMA pipeline already
  consumes the chunks that have arrived (own shard first).  Backward = ``matmul_reduce_scatter``.
* ``all_reduce_``            - two-shot all-reduce of a gradient bucket with the mean / unscale factor folded in.
* ``reduce_scatter_adamw``   - parallel-optimizer step: gradient ReduceScatter + unscale + AdamW on the owned
  slice + AllGather of the updated bf16 weights, one kernel per bucket.

Every fused op keeps its un-fused NCCL form (``parallel.tp``, ``communication.comm_func``) as the selectable
baseline: ``set_context(fused_comm=False)`` or the environment variable ``MSB200_FUSED_COMM=0`` turns the fused
path off.  Buffers are double-buffered per tag so that one barrier per operation is enough (see ``_next``).
"""
from __future__ import annotations

import ctypes
import os

import torch

from .. import _native, context
from ..communication import management as M
from ..ops import kernels as K
from ..ops.kernels import _count, _p, _stream
from ..utils.log import logger

_P, _I, _L, _F = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float
_U64P = ctypes.POINTER(ctypes.c_ulonglong)
_native.register_cuda_signature("msb_symm_barrier", _I, [_U64P, _I, _I, _I, _I, _P])
_native.register_cuda_signature("msb_allreduce_symm", _I, [_U64P, _I, _I, _L, _F, _P, _P])
_native.register_cuda_signature("msb_reduce_slots", _I, [_P, _P, _I, _L, _P])
_native.register_cuda_signature("msb_reduce_scatter_adamw", _I, [_U64P, _U64P, _P, _P, _P, _I, _I, _L, _P, _P, _P])
_native.register_cuda_signature("msb_gemm_rs", _I, [_P, _P, _U64P, _I, _I, _I, _I, _L, _L, _I, _I, _I, _P])
_native.register_cuda_signature("msb_gemm_push_rows", _I, [_P, _P, _P, _U64P, _I, _I, _I, _I, _L, _L, _I, _I, _I, _I, _I, _P])
_native.register_cuda_signature("msb_gemm_ag", _I, [_U64P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _L, _L, _I, _I, _I, _I, _P])

_contexts = {}
_disabled = set()
# AllGather -> MatMul: 1 = the copy engines pull the peers' shards (SMs only multiply), 0 = a copy warp per CTA does
# AllGather -> MatMul: who moves the peer shards.  1 = the copy engines (peer copies on two side streams, one flag per
# chunk), 0 = the GEMM kernel's own copy warp.  Measured per op (utils/kernel_bench.py fused_comm): the copy engines
# win at 2 and 4 ranks (186 vs 196 us at 2 ranks for the QKV projection), the copy warp at 8 ranks, where seven small
# peer copies per call cost more in launch and event traffic than they save (118 vs 135 us).  "auto" follows that.
_AG_DMA_ENV = os.environ.get("MSB200_AG_DMA", "auto")
_AG_DMA = None if _AG_DMA_ENV == "auto" else int(_AG_DMA_ENV != "0")


def _ptr_array(ptrs):
    arr = (ctypes.c_ulonglong * 8)()
    for i, p in enumerate(ptrs):
        arr[i] = int(p)
    return arr


class SymmContext:
    CHANNELS = 4

    def __init__(self, group):
        import torch.distributed._symmetric_memory as symm_mem
        self.symm_mem = symm_mem
        self.group = group
        self.world = group.size
        self.rank = M.get_rank(group.name)
        self.pg = group.pg
        self.group_name = self.pg.group_name
        if hasattr(symm_mem, "enable_symm_mem_for_group"):
            try:
                symm_mem.enable_symm_mem_for_group(self.group_name)
            except Exception:  # noqa: BLE001  (already enabled / not needed in this torch version)
                pass
        self.buffers = {}
        self.counters = {}
        pads, self.pad_ptrs = self._alloc_raw(self.CHANNELS * (self.world + 1) * 4)
        pads.zero_()
        torch.cuda.synchronize()
        torch.distributed.barrier(group=self.pg)
        self.pads = pads

    def _alloc_raw(self, nbytes):
        nbytes = (nbytes + 255) // 256 * 256
        dev = torch.device("cuda", torch.cuda.current_device())
        try:
            t = self.symm_mem.empty(nbytes, dtype=torch.uint8, device=dev)
        except RuntimeError:
            # symmetric memory comes straight from the driver: blocks cached by the tensor allocator but not in use
            # (initialisation temporaries) are invisible to it - release them and try once more
            torch.cuda.empty_cache()
            t = self.symm_mem.empty(nbytes, dtype=torch.uint8, device=dev)
        hdl = self.symm_mem.rendezvous(t, group=self.group_name)
        ptrs = [int(p) for p in hdl.buffer_ptrs]
        return t, ptrs

    def buffer(self, tag, nbytes):
        """Symmetric buffer for ``tag`` with at least ``nbytes`` (collective on first use / growth)."""
        ent = self.buffers.get(tag)
        if ent is None or ent[0].numel() < nbytes:
            size = max(nbytes, 1 << 20)
            if ent is not None:
                size = max(size, 2 * ent[0].numel())
            ent = self._alloc_raw(size)
            self.buffers[tag] = ent
        return ent

    def _next(self, tag):
        """Alternates between two buffers of a tag: the buffer written by operation k is free again at operation
        k+2, because every rank passes the barrier of operation k+1 only after finishing operation k."""
        c = self.counters.get(tag, 0)
        self.counters[tag] = c + 1
        return "%s#%d" % (tag, c & 1)

    def barrier(self, channel=0):
        """Stream-ordered group barrier; its epoch counter lives on the device, so it replays inside CUDA graphs."""
        rc = _native.cuda().msb_symm_barrier(_ptr_array(self.pad_ptrs), self.rank, self.world, channel,
                                             self.CHANNELS, _stream())
        _native.check(rc, "symm_barrier")
        _count()


def _enabled():
    if os.environ.get("MSB200_FUSED_COMM", "1") == "0":
        return False
    return bool(context.get_context("fused_comm"))


def get_context(group):
    """Returns the group's SymmContext, creating it on first use (a collective call), or None if unavailable."""
    if group.name in _contexts:
        return _contexts[group.name]
    if group.name in _disabled:
        return None
    ok = (_enabled() and group.pg is not None and not M.is_simulation() and torch.cuda.is_available()
          and M.GlobalComm.BACKEND == "nccl" and 2 <= group.size <= 8)
    ctx = None
    if ok:
        try:
            ctx = SymmContext(group)
        except Exception as e:  # noqa: BLE001
            logger.warning("symmetric memory is not available for group %s (%s): using NCCL collectives",
                           group.name, e)
            ctx = None
        # all ranks must agree, otherwise some would wait in barriers the others never join
        flag = torch.tensor([1 if ctx is not None else 0], device="cuda")
        torch.distributed.all_reduce(flag, op=torch.distributed.ReduceOp.MIN, group=group.pg)
        if int(flag) == 0:
            ctx = None
    if ctx is None:
        _disabled.add(group.name)
    else:
        _contexts[group.name] = ctx
    return ctx


def available(group):
    return get_context(group) is not None


# --------------------------------------------------------------------------------------------- all-reduce
def all_reduce_(tensor, group, scale=1.0, nonfinite=None):
    """In-place sum (x scale) of an fp32 CUDA tensor over the group."""
    ctx = get_context(group)
    assert tensor.dtype == torch.float32 and tensor.is_contiguous()
    n = tensor.numel()
    buf, ptrs = ctx.buffer(ctx._next("allreduce"), n * 4)
    view = buf[:n * 4].view(torch.float32)
    view.copy_(tensor.reshape(-1))
    ctx.barrier(0)
    rc = _native.cuda().msb_allreduce_symm(_ptr_array(ptrs), ctx.rank, ctx.world, n, float(scale), _p(nonfinite),
                                           _stream())
    _native.check(rc, "allreduce_symm")
    _count()
    ctx.barrier(0)
    tensor.reshape(-1).copy_(view)
    return tensor


def all_reduce_symm_(ctx, ptrs, offset, n, scale=1.0, nonfinite=None):
    """In-place sum (x scale) of elements [offset, offset + n) of an fp32 buffer that already lives in symmetric
    memory (``ptrs`` = its address on every rank): no staging copies.  Rank r sums slice r of the range over peer
    loads and stores the result into every rank's buffer; the barriers on both sides order it against the producers
    of the range and against whoever reads it next."""
    assert (offset * 4) % 16 == 0
    ctx.barrier(0)
    rc = _native.cuda().msb_allreduce_symm(_ptr_array([p + offset * 4 for p in ptrs]), ctx.rank, ctx.world, n,
                                           float(scale), _p(nonfinite), _stream())
    _native.check(rc, "allreduce_symm")
    _count()
    ctx.barrier(0)


# --------------------------------------------------------------------------------------------- GEMM + collectives
def _gemm_rs(ctx, a, b, b_mn):
    """partial = a @ op(b) reduced over the group and scattered by token rows -> [M/world, N]."""
    M_, K_ = a.shape
    N_ = b.shape[1] if b_mn else b.shape[0]
    rows = M_ // ctx.world
    stage, ptrs = ctx.buffer(ctx._next("rs_stage"), ctx.world * rows * N_ * 2)
    rc = _native.cuda().msb_gemm_rs(_p(a), _p(b), _ptr_array(ptrs), M_, N_, K_, int(b_mn), a.stride(0), b.stride(0),
                                    ctx.world, ctx.rank, 0, _stream())
    _native.check(rc, "gemm_rs")
    _count()
    ctx.barrier(1)
    out = torch.empty((rows, N_), dtype=torch.bfloat16, device=a.device)
    rc = _native.cuda().msb_reduce_slots(_p(stage), _p(out), ctx.world, rows * N_, _stream())
    _native.check(rc, "reduce_slots")
    _count()
    return out


def _gemm_ag(ctx, a_shard, b, b_mn, bias=None):
    """c = gather(a_shard) @ op(b) -> ([M, N], gathered a [M, K])."""
    rows, K_ = a_shard.shape
    M_ = rows * ctx.world
    N_ = b.shape[1] if b_mn else b.shape[0]
    src, ptrs = ctx.buffer(ctx._next("ag_src"), rows * K_ * 2)
    src[:rows * K_ * 2].view(torch.bfloat16).view(rows, K_).copy_(a_shard)
    ctx.barrier(2)
    gathered = torch.empty((M_, K_), dtype=torch.bfloat16, device=a_shard.device)
    flags = torch.empty(ctx.world, dtype=torch.int32, device=a_shard.device)
    c = torch.empty((M_, N_), dtype=torch.bfloat16, device=a_shard.device)
    rc = _native.cuda().msb_gemm_ag(_ptr_array(ptrs), _p(gathered), _p(flags), _p(b), _p(c), _p(bias), M_, N_, K_,
                                    int(b_mn), b.stride(0), N_, ctx.world, ctx.rank, 0,
                                    int(ctx.world <= 4) if _AG_DMA is None else _AG_DMA, _stream())
    _native.check(rc, "gemm_ag")
    _count()
    return c, gathered


def gemm_gather_rows(ctx, src_ptrs, rows, b, b_mn, bias=None, out=None, gathered=None):
    """c = gather(chunks) @ op(b) (+ bias) -> ([world * rows, N], the gathered operand [world * rows, K]) where chunk c
    is ``rows`` x K bf16 at ``src_ptrs[c]`` in rank c's symmetric memory (already published: the caller has passed a
    barrier after writing it).  Tiles of chunks that have arrived are multiplied while the others are in flight.
    ``out`` / ``gathered``: contiguous bf16 destinations of those shapes (allocated here if None)."""
    K_ = b.shape[0] if b_mn else b.shape[1]
    N_ = b.shape[1] if b_mn else b.shape[0]
    M_ = rows * ctx.world
    if gathered is None:
        gathered = torch.empty((M_, K_), dtype=torch.bfloat16, device=b.device)
    if out is None:
        out = torch.empty((M_, N_), dtype=torch.bfloat16, device=b.device)
    assert out.is_contiguous() and gathered.is_contiguous() and out.shape == (M_, N_) and gathered.shape == (M_, K_)
    flags = torch.empty(ctx.world, dtype=torch.int32, device=b.device)
    rc = _native.cuda().msb_gemm_ag(_ptr_array(src_ptrs), _p(gathered), _p(flags), _p(b), _p(out), _p(bias), M_, N_,
                                    K_, int(b_mn), b.stride(0), N_, ctx.world, ctx.rank, 0,
                                    int(ctx.world <= 4) if _AG_DMA is None else _AG_DMA, _stream())
    _native.check(rc, "gemm_ag")
    _count()
    return out, gathered


def gemm_push_rows(ctx, a, b, b_mn, dst_ptrs, slot, slots, bias=None):
    """Rows [o * M / world, (o + 1) * M / world) of  a @ op(b) (+ bias)  are stored from the GEMM's epilogue into
    slot ``slot`` of rank o's buffer ``dst_ptrs[o]`` (bf16 [slots][M / world][N]); the product is never written
    locally.  The receivers read their slots after the next group barrier."""
    M_, K_ = a.shape
    N_ = b.shape[1] if b_mn else b.shape[0]
    rc = _native.cuda().msb_gemm_push_rows(_p(a), _p(b), _p(bias), _ptr_array(dst_ptrs), M_, N_, K_, int(b_mn),
                                           a.stride(0), b.stride(0), ctx.world, ctx.rank, slot, slots, 0, _stream())
    _native.check(rc, "gemm_push_rows")
    _count()


def _optim():
    from ..nn import optim
    return optim


def _shapes_ok(rows_total, world, *dims):
    return rows_total % world == 0 and (rows_total // world) % 128 == 0 and all(d % 8 == 0 for d in dims)


class _MatmulReduceScatter(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, gname):
        sc = get_context(M._group(gname))
        x = x.contiguous()
        ctx.save_for_backward(x, w)
        ctx.gname, ctx.w_ref = gname, w
        return _gemm_rs(sc, x, w, False)

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        sc = get_context(M._group(ctx.gname))
        dx, dy_full = _gemm_ag(sc, dy.contiguous(), w, True)        # dx[T, K/mp] = gather(dy) @ w
        mg = getattr(ctx.w_ref, "main_grad", None)
        if mg is not None:
            K.linear_wgrad(dy_full, x, out=mg, accumulate=True)
            dw = None
            _optim().notify_grad_written(ctx.w_ref)
        else:
            dw = K.linear_wgrad(dy_full, x, out_dtype=torch.bfloat16)
        return dx, dw, None


class _AllgatherMatmul(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x_shard, w, bias, gname):
        sc = get_context(M._group(gname))
        y, gathered = _gemm_ag(sc, x_shard.contiguous(), w, False, bias)
        ctx.save_for_backward(gathered, w)
        ctx.gname, ctx.w_ref, ctx.has_bias = gname, w, bias is not None
        return y

    @staticmethod
    def backward(ctx, dy):
        gathered, w = ctx.saved_tensors
        sc = get_context(M._group(ctx.gname))
        dy = dy.contiguous()
        dx_shard = _gemm_rs(sc, dy, w, True)                         # reduce_scatter(dy @ w)
        mg = getattr(ctx.w_ref, "main_grad", None)
        if mg is not None:
            K.linear_wgrad(dy, gathered, out=mg, accumulate=True)
            dw = None
            _optim().notify_grad_written(ctx.w_ref)
        else:
            dw = K.linear_wgrad(dy, gathered, out_dtype=torch.bfloat16)
        db = dy.float().sum(0).to(dy.dtype) if ctx.has_bias else None
        return dx_shard, dw, db, None


def matmul_reduce_scatter(x, w_shard, tp):
    """x [T, K/mp] @ w_shard[N, K/mp]^T, summed over the group, token rows scattered -> [T/mp, N]."""
    if x.dtype != torch.bfloat16 or not _shapes_ok(x.shape[0], tp.size, x.shape[1], w_shard.shape[0]):
        from . import tp as _tp
        from ..ops import fused
        return _tp.scatter_tokens_reduce(fused.linear(x, w_shard), tp)
    _optim().note_grad_producer(w_shard)
    return _MatmulReduceScatter.apply(x, w_shard, tp.name)


def allgather_matmul(x_shard, w_shard, tp, bias=None):
    """gather(x_shard [T/mp, K]) @ w_shard[N/mp, K]^T -> [T, N/mp]."""
    if x_shard.dtype != torch.bfloat16 or x_shard.shape[0] % 128 or x_shard.shape[1] % 8 or w_shard.shape[0] % 8:
        from . import tp as _tp
        from ..ops import fused
        return fused.linear(_tp.gather_tokens(x_shard, tp), w_shard, bias)
    _optim().note_grad_producer(w_shard)
    return _AllgatherMatmul.apply(x_shard, w_shard, bias, tp.name)


# --------------------------------------------------------------------------------------------- ZeRO-style AdamW
def reduce_scatter_adamw(ctx, grad_ptrs, weight_ptrs, master, m, v, per, hyper, skip=None):
    rc = _native.cuda().msb_reduce_scatter_adamw(_ptr_array(grad_ptrs), _ptr_array(weight_ptrs), _p(master), _p(m),
                                                 _p(v), ctx.rank, ctx.world, per, _p(hyper), _p(skip), _stream())
    _native.check(rc, "reduce_scatter_adamw")
    _count()


def step_fence():
    """One group barrier at the start of a micro-step for every active symmetric-memory context.  It separates the
    last fused operation of the previous micro-step from the first of this one, so the two-buffer rotation stays
    valid across CUDA-graph replays (where the rotation restarts at buffer 0)."""
    for ctx in _contexts.values():
        ctx.barrier(3)
