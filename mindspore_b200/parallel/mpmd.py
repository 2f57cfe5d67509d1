"""MPMD execution by placement labels: ``cell.place(role, rank_id)`` pins a sub-cell to one process; ``run_placed``
runs a forward pass in which every labelled cell executes only on its process and tensors that cross from one
process to another are sent point to point.

    net.encoder.place("MS_WORKER", 0)
    net.decoder.place("MS_WORKER", 1)
    out = run_placed(net, x)            # every rank calls it with the same inputs; `out` is returned on all ranks

How it works: while the network's ``construct`` runs on every rank, a call of a labelled cell is intercepted.  On the
owning rank the cell runs (after receiving those inputs that were produced elsewhere); on the other ranks it returns
a placeholder that remembers the producer.  A rank that holds a real tensor produced by one of its own cells sends
it when a cell owned by someone else consumes it.  Unlabelled code runs everywhere, on placeholders where its inputs
are remote (a placeholder absorbs any tensor operation).  The result is broadcast from its producer.

The reference splits the compiled graph by the same labels and inserts ``RpcSend`` / ``RpcRecv`` kernels with a
route table resolved through the scheduler (frontend/parallel/graph_util/graph_splitter.cc, runtime/graph_scheduler/
rpc_node_scheduler.cc, ``Cell.place`` nn/cell.py:2406); tensors travel over its TCP RPC.  Here they travel over the
process group (NCCL p2p on GPUs, gloo on CPU).  Forward only: training across placement boundaries uses pipeline
parallelism (``parallel.pipeline``), which also schedules micro-batches."""
from __future__ import annotations

import torch
import torch.distributed as dist

from ..common.tensor import Tensor
from ..communication import management as M
from ..nn.cell import Cell

_DTYPES = [torch.float32, torch.float16, torch.bfloat16, torch.float64, torch.int64, torch.int32, torch.int16,
           torch.int8, torch.uint8, torch.bool]


class Remote(torch.Tensor):
    """Placeholder for a tensor that lives on rank ``producer``; tensor operations on it give another placeholder."""

    @staticmethod
    def make(producer, tag):
        t = torch.Tensor._make_subclass(Remote, torch.empty(0))
        t.producer, t.tag = producer, tag
        return t

    @classmethod
    def __torch_function__(cls, func, types, args=(), kwargs=None):
        if getattr(func, "__name__", "") == "__get__":
            with torch._C.DisableTorchFunctionSubclass():
                return func(*args, **(kwargs or {}))
        src = next((a for a in _flatten(args) if isinstance(a, Remote)), None)
        return Remote.make(src.producer if src is not None else -1, src.tag if src is not None else -1)

    def __repr__(self):
        return "Remote(rank=%s)" % getattr(self, "producer", "?")


class Local(Tensor):
    """A tensor that only this rank holds: the output of a cell placed here, or anything computed from one (tensor
    operations keep the subclass).  The other ranks see a ``Remote`` in its place."""


def _mark_local(x):
    if isinstance(x, torch.Tensor) and not isinstance(x, Remote):
        return x.as_subclass(Local)
    if isinstance(x, tuple):
        return tuple(_mark_local(y) for y in x)
    if isinstance(x, list):
        return [_mark_local(y) for y in x]
    if isinstance(x, dict):
        return {k: _mark_local(v) for k, v in x.items()}
    return x


def _flatten(x):
    if isinstance(x, (list, tuple)):
        for y in x:
            yield from _flatten(y)
    elif isinstance(x, dict):
        for y in x.values():
            yield from _flatten(y)
    else:
        yield x


def _send(t, dst):
    t = t.detach().contiguous()
    meta = torch.zeros(10, dtype=torch.int64)
    meta[0], meta[1] = _DTYPES.index(t.dtype), t.dim()
    meta[2:2 + t.dim()] = torch.tensor(list(t.shape), dtype=torch.int64)
    dev = t.device if dist.get_backend() == "nccl" else torch.device("cpu")
    dist.send(meta.to(dev), dst)
    dist.send(t.to(dev), dst)


def _recv(src, device):
    dev = device if dist.get_backend() == "nccl" else torch.device("cpu")
    meta = torch.zeros(10, dtype=torch.int64, device=dev)
    dist.recv(meta, src)
    m = meta.tolist()
    t = torch.empty(tuple(m[2:2 + m[1]]), dtype=_DTYPES[m[0]], device=dev)
    dist.recv(t, src)
    return t.to(device)


class PlacedRuntime:
    def __init__(self, net, role="MS_WORKER"):
        self.net, self.role = net, role
        self.rank = M.get_rank() if M.GlobalComm.INITED else 0
        self.world = M.get_group_size() if M.GlobalComm.INITED else 1
        self.placed = [(n, c) for n, c in net.cells_and_names() if getattr(c, "_placement", None) is not None]
        for name, c in self.placed:
            r = c._placement[1]
            if not 0 <= r < self.world:
                raise ValueError("cell %s is placed on rank %d, but the job has %d ranks" % (name, r, self.world))
        self._tag = 0
        self.device = next((p.device for p in net.get_parameters()), torch.device("cpu"))

    def _hook(self, cell, inputs, kwargs):
        placement = getattr(cell, "_placement", None)
        if placement is None or self._inside:
            return cell._call_impl(inputs, kwargs)
        owner = placement[1]
        flat = [a for a in _flatten((inputs, kwargs)) if isinstance(a, torch.Tensor)]
        if owner == self.rank:
            received = {}
            for a in flat:
                if isinstance(a, Remote) and id(a) not in received:
                    if a.producer in (self.rank, -1):
                        raise RuntimeError("cell needs a value that no other rank can supply (producer %s)" % a.producer)
                    received[id(a)] = _recv(a.producer, self.device)

            def real(x):
                if isinstance(x, Remote):
                    return received[id(x)]
                if isinstance(x, tuple):
                    return tuple(real(y) for y in x)
                if isinstance(x, list):
                    return [real(y) for y in x]
                if isinstance(x, dict):
                    return {k: real(v) for k, v in x.items()}
                return x
            self._inside = True
            try:
                out = cell._call_impl(real(inputs), real(kwargs))
            finally:
                self._inside = False
            n_out = sum(1 for t in _flatten(out) if isinstance(t, torch.Tensor))
            self._tag += max(n_out, getattr(cell, "_placed_outputs", 1))
            return _mark_local(out)
        # not the owner: ship what this rank produced and the owner needs, then stand in with a placeholder
        sent = set()
        for a in flat:
            if isinstance(a, Local) and id(a) not in sent:
                _send(a, owner)
                sent.add(id(a))
            elif isinstance(a, Remote) and a.producer not in (owner, -1) and a.producer == self.rank:
                raise RuntimeError("placeholder for a value of this rank: the value lost its Local mark on the way "
                                   "(a layer between placed cells rebuilt the tensor)")
        n_out = getattr(cell, "_placed_outputs", 1)
        outs = []
        for _ in range(n_out):
            self._tag += 1
            outs.append(Remote.make(owner, self._tag))
        return outs[0] if n_out == 1 else tuple(outs)

    def run(self, *inputs, broadcast_output=True):
        self._tag, self._inside = 0, False
        prev = Cell._stage_hook
        saved = []
        for _, c in self.placed:                         # the interception point of Cell.__call__ keys on this attribute
            saved.append(c._pipeline_stage)
            c._pipeline_stage = c._placement[1]
        Cell._stage_hook = self._hook
        try:
            with torch.no_grad():
                out = self.net(*inputs)
        finally:
            Cell._stage_hook = prev
            for (_, c), s in zip(self.placed, saved):
                c._pipeline_stage = s
        if not broadcast_output or self.world == 1:
            return out

        # which rank holds which result leaf for real?  the lowest holder sends to every rank that lacks it
        leaves = [t for t in _flatten(out) if isinstance(t, torch.Tensor)]
        mine = [-1 if not isinstance(t, Remote) else int(t.producer) for t in leaves]
        table = [None] * self.world
        dist.all_gather_object(table, mine)
        got = {}
        for i, t in enumerate(leaves):
            holders = [r for r in range(self.world) if table[r][i] == -1]
            if not holders:
                raise RuntimeError("result %d of the placed network is held by no rank" % i)
            sender = holders[0]
            for r in range(self.world):
                if table[r][i] == -1:
                    continue
                if self.rank == sender:
                    _send(t, r)
                elif self.rank == r:
                    got[i] = _recv(sender, self.device)
        it = iter(range(len(leaves)))

        def rebuild(x):
            if isinstance(x, torch.Tensor):
                i = next(it)
                return got.get(i, x)
            if isinstance(x, (tuple, list)):
                return type(x)(rebuild(y) for y in x)
            if isinstance(x, dict):
                return {k: rebuild(v) for k, v in x.items()}
            return x
        return rebuild(out)


def run_placed(net, *inputs, broadcast_output=True):
    rt = getattr(net, "_placed_runtime", None)
    if rt is None:
        rt = PlacedRuntime(net)
        object.__setattr__(net, "_placed_runtime", rt)
    return rt.run(*inputs, broadcast_output=broadcast_output)
