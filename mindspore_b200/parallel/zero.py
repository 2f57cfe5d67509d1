"""Data parallelism on the flat parameter arena, with optional optimizer-state sharding (the reference's
``enable_parallel_optimizer``: ZeRO-1/2-like "opt shard").

Without sharding every rank all-reduces the fp32 gradient arena over the data-parallel group and runs the full
update.  With sharding the arena is cut into ``dp`` equal slices; rank r keeps fp32 master weights and Adam moments
for slice r only, and one step is

1. gradient ReduceScatter fused with the 1/dp scale - rank r sums slice r over the peers' gradient arenas with
   peer loads (``msb_reduce_scatter_symm``; NCCL ``reduce_scatter_tensor`` without symmetric memory),
2. squared-norm / overflow pass over the owned slice + one tiny all-reduce, clip factor decided on the device,
3. AdamW on the owned slice fused with the parameter AllGather - the new bf16 weights are stored straight into
   every peer's weight arena (``msb_adamw_allgather``; NCCL ``all_gather_into_tensor`` otherwise).

In the reference the same step is ncclReduceScatter -> Cast -> Mul -> AdamWeightDecay per parameter -> ncclAllGather
(ccsrc/frontend/parallel/parameter_manager.cc + optimizer/opt_param_mgr.cc:95-131 for the slicing rule,
python/mindspore/nn/optim/optimizer.py:_use_parallel_optimizer)."""
from __future__ import annotations

import ctypes
import os

import torch
import torch.distributed as dist

from .. import _native
from ..communication import comm_func as CF
from ..communication import management as M
from ..ops import kernels as K
from ..ops.kernels import _count, _p, _stream

_P, _I, _L, _F = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float
_U64P = ctypes.POINTER(ctypes.c_ulonglong)
_native.register_cuda_signature("msb_reduce_scatter_symm", _I, [_U64P, _I, _I, _L, _L, _F, _P])
_native.register_cuda_signature("msb_adamw_allgather", _I, [_P, _P, _P, _P, _U64P, _I, _L, _L, _P, _P, _P])

_SLICE_ALIGN = 128
_last_overlapped = 0                   # buckets launched from inside backward so far (for tests / logs)
_BUCKET_ELEMS = 64 * 1024 * 1024      # 256 MB of fp32 gradients per all-reduce bucket
_OVERLAP_BUCKET_ELEMS = 4 * 1024 * 1024   # 16 MB buckets when the all-reduce overlaps backward (MSB200_DP_OVERLAP=0 turns it off)


def _ptr_array(ptrs):
    arr = (ctypes.c_ulonglong * 8)()
    for i, p in enumerate(ptrs):
        arr[i] = int(p)
    return arr


class DataParallelArena:
    def __init__(self, opt, group_name, mean=True, shard=False, fused=True):
        self.opt, self.arena = opt, opt.arena
        self.group = M._group(group_name)
        self.world = self.group.size
        self.rank = self.group.ranks.index(M.get_rank())
        self.mean, self.shard = mean, bool(shard) and self.world > 1
        self.overlap = os.environ.get("MSB200_DP_OVERLAP", "1") != "0"
        arena = self.arena
        self.local_only = [(arena.offsets[i], arena.offsets[i] + p.numel()) for i, p in enumerate(arena.params)
                           if getattr(p, "dp_local", False)]
        self.symm = None
        self._symm_grads = None
        if not self.shard:
            if fused and self.world > 1 and arena.grads.is_cuda and os.environ.get("MSB200_SYMM_GRADS", "1") != "0":
                from . import fused_comm
                if fused_comm.available(self.group):
                    # the gradient arena itself lives in symmetric memory: bucket all-reduces run in place on it
                    # (peer loads / peer stores) instead of through a staging buffer
                    ctx = fused_comm.get_context(self.group)
                    graw, ptrs = ctx._alloc_raw(arena.grads.numel() * 4)
                    grads = graw[:arena.grads.numel() * 4].view(torch.float32)
                    grads.copy_(arena.grads)
                    arena.rebind(arena.weights, grads)
                    self._symm_grads = (ctx, ptrs, graw)
                    torch.cuda.synchronize()
                    dist.barrier(group=self.group.pg)
            return
        if self.local_only:
            raise ValueError("optimizer-state sharding over the data-parallel group cannot hold parameters that "
                             "differ per rank (expert-parallel experts); exclude them or turn sharding off")
        per = (arena.total + self.world - 1) // self.world
        self.per = (per + _SLICE_ALIGN - 1) // _SLICE_ALIGN * _SLICE_ALIGN
        self.padded = self.per * self.world
        self.lo, self.hi = self.rank * self.per, (self.rank + 1) * self.per
        dev, wdt = arena.weights.device, arena.weights.dtype
        if fused and dev.type == "cuda" and wdt == torch.bfloat16:
            from . import fused_comm
            self.symm = fused_comm.get_context(self.group)
        if self.symm is not None:
            graw, self.grad_ptrs = self.symm._alloc_raw(self.padded * 4)
            wraw, self.weight_ptrs = self.symm._alloc_raw(self.padded * 2)
            grads = graw[:self.padded * 4].view(torch.float32)
            weights = wraw[:self.padded * 2].view(torch.bfloat16)
            self._keep = (graw, wraw)
        else:
            grads = torch.zeros(self.padded, dtype=torch.float32, device=dev)
            weights = torch.zeros(self.padded, dtype=wdt, device=dev)
        grads.zero_()
        weights.zero_()
        weights[:arena.total].copy_(arena.weights)
        master_full = arena.master if arena.master is not None else arena.weights
        self.master = torch.zeros(self.per, dtype=torch.float32, device=dev)
        n_own = max(0, min(self.hi, arena.total) - self.lo)
        if n_own:
            self.master[:n_own].copy_(master_full[self.lo:self.lo + n_own])
        self.m = torch.zeros(self.per, dtype=torch.float32, device=dev)
        self.v = torch.zeros(self.per, dtype=torch.float32, device=dev)
        arena.rebind(weights, grads)
        arena.master = None                      # the full fp32 copy and full moments are not kept
        opt._m = opt._v = None
        if self.symm is not None:
            torch.cuda.synchronize()
            dist.barrier(group=self.group.pg)

    def state_buffers(self):
        """The sharded moments (this rank's slice), in the order of ``Optimizer._arena_state_names``."""
        return (self.m, self.v)

    # ------------------------------------------------------------------ overlap with backward
    def _bucket_ranges(self):
        if getattr(self, "_reduce_ranges", None) is None:
            arena = self.arena
            ranges, pos = [], 0
            for s, e in sorted(self.local_only):
                if s > pos:
                    ranges.append((pos, s))
                pos = max(pos, (e + _SLICE_ALIGN - 1) // _SLICE_ALIGN * _SLICE_ALIGN)
            if pos < arena.total:
                ranges.append((pos, arena.total))
            step = self._overlap_bucket_elems() if self._overlap_eligible() else _BUCKET_ELEMS
            self._reduce_ranges = [(lo, min(lo + step, hi)) for s, hi in ranges for lo in range(s, hi, step)]
        return self._reduce_ranges

    @staticmethod
    def _overlap_bucket_elems():
        """fp32 gradient elements per overlapped all-reduce bucket: the ``comm_fusion`` all-reduce size threshold of
        the auto-parallel context when one is configured (``{"allreduce": {"mode": "size", "config": MB}}``), else
        16 MB."""
        from .comm_fusion import _policy
        from .. import context
        cf = context.get_auto_parallel_context("comm_fusion") or {}
        if "allreduce" in cf:
            mode, cfg = _policy("allreduce")
            if mode == "size" and cfg:
                return max(_SLICE_ALIGN, int(float(cfg) * 1024 * 1024 / 4) // _SLICE_ALIGN * _SLICE_ALIGN)
        return _OVERLAP_BUCKET_ELEMS

    def _overlap_eligible(self):
        """Overlap runs the gradient all-reduce on a side stream.  It is limited to pure data parallelism: with a
        model-parallel or expert-parallel group the backward pass issues its own collectives over the same symmetric
        buffers and barrier flags, and two streams must not interleave on those."""
        return (self.overlap and self.world > 1 and not self.shard and not self.local_only
                and getattr(self.opt, "_mp_group", None) is None)

    def begin_step(self):
        """Arms the overlap for one backward pass: every bucket whose parameters have all reported their gradient
        (``nn.optim.notify_grad_written``, or a ``.grad`` that autograd accumulated) is all-reduced at once on a side
        stream while backward goes on; ``allreduce`` afterwards only handles what is left and joins the stream.  Use
        it only when the step runs a single backward (no micro-batch accumulation)."""
        if not self._overlap_eligible():
            return False
        from ..nn import optim as _optim
        arena = self.arena
        ranges = self._bucket_ranges()
        if getattr(self, "_bucket_of", None) is None:
            self._bucket_of, self._bucket_size = {}, [0] * len(ranges)
            starts = [lo for lo, _ in ranges]
            import bisect
            for i, p in enumerate(arena.params):
                off = arena.offsets[i]
                b = bisect.bisect_right(starts, off) - 1
                if b < 0 or off >= ranges[b][1] or getattr(p, "dp_local", False):
                    continue
                last = bisect.bisect_right(starts, off + p.numel() - 1) - 1
                members = range(b, last + 1)               # a parameter that straddles buckets counts in each
                self._bucket_of[id(p)] = list(members)
                for m in members:
                    self._bucket_size[m] += 1

                def fold(param):
                    g = param.grad
                    if g is not None and self._armed:
                        param.main_grad.add_(g.to(param.main_grad.dtype))
                        param.grad = None
                        self._on_grad(param)
                if p.requires_grad and hasattr(p, "register_post_accumulate_grad_hook"):
                    p.register_post_accumulate_grad_hook(fold)
            _optim._grad_listeners.append(self._on_grad)
            if arena.grads.is_cuda:
                self._comm_stream = torch.cuda.Stream()
        for p in arena.params:
            p._grad_writers = 0                # producers register again in this step's forward
        self._pending = list(self._bucket_size)
        self._seen = set()
        self._done = [False] * len(ranges)
        self._armed = True
        return True

    def _on_grad(self, param):
        if not getattr(self, "_armed", False):
            return
        key = id(param)
        if key in self._seen or key not in self._bucket_of:
            return
        self._seen.add(key)
        for b in self._bucket_of[key]:
            self._pending[b] -= 1
            if self._pending[b] == 0 and not self._done[b]:
                self._launch(b)

    def _launch(self, b):
        lo, hi = self._reduce_ranges[b]
        scale = 1.0 / self.world if self.mean else 1.0
        stream = getattr(self, "_comm_stream", None)
        if stream is None:
            self._reduce_segment(lo, hi, scale)
        else:
            stream.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(stream):
                self._reduce_segment(lo, hi, scale)
        self._done[b] = True
        self.overlapped_buckets = getattr(self, "overlapped_buckets", 0) + 1
        global _last_overlapped
        _last_overlapped = self.overlapped_buckets

    def _reduce_segment(self, lo, hi, scale):
        from . import symm
        seg = self.arena.grads[lo:hi]
        if self._symm_grads is not None:
            from . import fused_comm
            ctx, ptrs, _ = self._symm_grads
            fused_comm.all_reduce_symm_(ctx, ptrs, lo, hi - lo, scale)
        elif symm.fused_available(self.group):
            symm.all_reduce_(seg, self.group, scale)
        else:
            CF._all_reduce_(seg, "sum", self.group)
            if scale != 1.0:
                seg.mul_(scale)

    # ------------------------------------------------------------------ plain data parallel
    def allreduce(self):
        """All-reduce (mean) of the gradient arena in buckets (``_BUCKET_ELEMS`` fp32 elements each, so the
        symmetric staging buffer stays small), leaving per-rank parameters (expert shards) un-reduced: those are
        only scaled."""
        if self.world == 1:
            return
        arena, scale = self.arena, (1.0 / self.world if self.mean else 1.0)
        armed = getattr(self, "_armed", False)
        self._armed = False
        for b, (lo, hi) in enumerate(self._bucket_ranges()):
            if armed and self._done[b]:
                continue                                   # already reduced on the side stream during backward
            self._reduce_segment(lo, hi, scale)
        if armed and getattr(self, "_comm_stream", None) is not None:
            torch.cuda.current_stream().wait_stream(self._comm_stream)
        if scale != 1.0:
            for s, e in self.local_only:
                arena.grads[s:e].mul_(scale)

    # ------------------------------------------------------------------ sharded step
    def _ranges_in_slice(self, ranges):
        """Intersects [(start, end, tag)] arena ranges with the owned slice; yields (offset in slice, length, tag)."""
        for s, e, tag in ranges:
            lo, hi = max(s, self.lo), min(e, self.hi)
            if lo < hi:
                yield lo - self.lo, hi - lo, tag

    def sharded_step(self, inv_loss_scale=1.0, check_finite=False, advance=True):
        opt, arena = self.opt, self.arena
        scale = 1.0 / self.world if self.mean else 1.0
        own = arena.grads[self.lo:self.hi]
        if self.symm is not None:
            self.symm.barrier(0)                                   # every rank's gradients are complete
            rc = _native.cuda().msb_reduce_scatter_symm(_ptr_array(self.grad_ptrs), self.rank, self.world, self.lo,
                                                        self.per, scale, _stream())
            _native.check(rc, "reduce_scatter_symm")
            _count()
        else:
            out = torch.empty_like(own)
            dist.reduce_scatter_tensor(out, arena.grads, group=self.group.pg)
            own.copy_(out * scale if scale != 1.0 else out)
        # global gradient norm / overflow flag from the owned slice
        skip = None
        if opt.max_grad_norm > 0 or check_finite or inv_loss_scale != 1.0:
            opt._sumsq.zero_()
            opt._nonfinite.zero_()
            mp_group = getattr(opt, "_mp_group", None)
            if mp_group is None:
                K.sumsq_finite(own, opt._sumsq, opt._nonfinite)
            else:
                opt._ensure_mp_runs()
                opt._sumsq_sh.zero_()
                runs = [(s, e, sh) for (s, e), sh in opt._norm_runs]
                for off, n, sharded in self._ranges_in_slice(runs):
                    K.sumsq_finite(own[off:off + n], opt._sumsq_sh if sharded else opt._sumsq, opt._nonfinite)
                CF._all_reduce_(opt._sumsq_sh, "sum", self.group)
                CF._all_reduce_(opt._sumsq_sh, "sum", M._group(mp_group))
                CF._all_reduce_(opt._nonfinite, "max", M._group(mp_group))
            CF._all_reduce_(opt._sumsq, "sum", self.group)
            CF._all_reduce_(opt._nonfinite, "max", self.group)
            if mp_group is not None:
                opt._sumsq.add_(opt._sumsq_sh)
            K.finalize_grad_scale(opt._sumsq, opt._nonfinite, inv_loss_scale, opt.max_grad_norm, opt._gscale,
                                  opt._skip, opt._gnorm)
            skip = opt._skip if check_finite else None
        t = opt._step() + 1
        lr = opt._lr_value(opt.learning_rate, opt._step())
        bc1 = 1 - opt.beta1 ** t if opt.bias_correction else 1.0
        bc2 = 1 - opt.beta2 ** t if opt.bias_correction else 1.0
        groups = []
        for gi, (first, last, wd) in enumerate(opt._arena_groups):
            s, e = arena.segment(first, last)
            groups.append((s, e, gi))
        wds = {gi: wd for gi, (_f, _l, wd) in enumerate(opt._arena_groups)}
        lp_slice = None
        if self.symm is None:
            lp_slice = arena.weights[self.lo:self.hi]
        for off, n, gi in self._ranges_in_slice(groups):
            h = opt._hyper[gi]
            from ..nn.optim import _fill_hyper
            _fill_hyper(h, 0, [lr, opt.beta1, opt.beta2, opt.eps, wds[gi], bc1, bc2])
            h[7:8].copy_(opt._gscale)
            if self.symm is not None:
                rc = _native.cuda().msb_adamw_allgather(_p(self.master[off:]), _p(self.m[off:]), _p(self.v[off:]),
                                                        _p(own[off:]), _ptr_array(self.weight_ptrs), self.world,
                                                        self.lo + off, n, _p(h), _p(skip), _stream())
                _native.check(rc, "adamw_allgather")
                _count()
            else:
                K.adamw_step(self.master[off:off + n], self.m[off:off + n], self.v[off:off + n], own[off:off + n],
                             lp_slice[off:off + n], h, skip)
        if self.symm is not None:
            self.symm.barrier(0)                                   # every peer's stores into this arena landed
        else:
            gathered = torch.empty_like(arena.weights)
            dist.all_gather_into_tensor(gathered, lp_slice.contiguous(), group=self.group.pg)
            arena.weights.copy_(gathered)
        if advance:
            opt._advance()
        return True
