"""Pipeline-parallel runtime: stage-local execution of a network whose cells carry ``pipeline_stage`` tags.

The reference splits the traced graph by stage colour and inserts Send/Receive nodes at stage borders
(ccsrc/frontend/parallel/pipeline_transformer/pipeline_split.cc:210-306, pipeline_transformer.cc; scheduling in
pipeline_scheduler.cc: GPipe, 1F1B, interleaved 1F1B).  Here the split happens while the network runs: every rank
executes ``construct`` of the whole network, and a hook on tagged cells decides per cell

* stage of the cell < stage of this rank : the cell is skipped and yields a placeholder that absorbs every
  operation applied to it (a cell that returns a tuple declares its length as ``cell.pipeline_outputs``);
* same stage                             : placeholders among its inputs are replaced by tensors received from the
  previous stage (first own cell only), then the cell runs;
* later stage                            : the activations this cell would consume are sent to the next stage and
  this rank's part of the forward pass ends.

Backward is the mirror image on the autograd graph of the stage: gradients for the sent activations arrive from
the next stage, ``torch.autograd.backward`` runs the stage, and gradients of the received activations go to the
previous stage.  The order of forward and backward micro-batches comes from the native scheduler
(``planner.pipeline_schedule``).  Activations travel with NCCL point-to-point calls on two communicators, one per
direction, so a send towards the next stage never queues behind a send towards the previous one.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from .. import context
from . import planner

_DTYPES = [torch.float32, torch.float16, torch.bfloat16, torch.float64, torch.int32, torch.int64, torch.int8,
           torch.uint8, torch.bool, torch.int16]
_META_LEN = 192
_MAX_DIMS = 8


class _StageDone(Exception):
    """Unwinds ``construct`` once this stage has handed its activations to the next one."""


class Skipped(torch.Tensor):
    """Stands for a value computed on an earlier stage.  Any torch function applied to it yields another one."""

    @staticmethod
    def make():
        return torch.Tensor._make_subclass(Skipped, torch.empty(0))

    @classmethod
    def __torch_function__(cls, func, types, args=(), kwargs=None):
        if getattr(func, "__name__", "") == "__get__":
            with torch._C.DisableTorchFunctionSubclass():
                return func(*args, **(kwargs or {}))
        return Skipped.make()

    def __repr__(self):
        return "Skipped()"


def _is_skipped(x):
    return isinstance(x, Skipped)


_groups = {}


def _direction_groups():
    """Two world-wide process groups used only for point-to-point traffic (forward / backward direction)."""
    if "fwd" not in _groups:
        _groups["fwd"] = dist.new_group()
        _groups["bwd"] = dist.new_group()
    return _groups["fwd"], _groups["bwd"]


def _comm_device(like=None):
    if dist.get_backend() == "nccl":
        return torch.device("cuda", torch.cuda.current_device())
    return torch.device("cpu")


def _encode_meta(tensors):
    """dtype, requires_grad, shape and - for a tensor that carries a parallel layout - device matrix, tensor map and
    full shape of every tensor of a hand-over, as one int64 vector.  The layout travels with the activation because
    the receiving stage continues the sharded computation where the sender stopped."""
    from . import spmd
    meta = torch.zeros(_META_LEN, dtype=torch.int64)
    meta[0] = len(tensors)
    pos = 1
    for t in tensors:
        lay = spmd.get_layout(t)
        flat_map = lay is not None and not any(isinstance(m, tuple) for m in lay.tensor_map)
        need = 4 + t.dim() + ((1 + len(lay.device_matrix) + 2 * t.dim()) if flat_map else 0)
        if t.dim() > _MAX_DIMS or pos + need > _META_LEN:
            raise ValueError("pipeline border: too many / too high-rank tensors for one hand-over")
        meta[pos] = _DTYPES.index(t.dtype)
        meta[pos + 1] = int(t.requires_grad)
        meta[pos + 2] = t.dim()
        for k, d in enumerate(t.shape):
            meta[pos + 3 + k] = d
        pos += 3 + t.dim()
        meta[pos] = len(lay.device_matrix) if flat_map else -1
        pos += 1
        if flat_map:
            for v in list(lay.device_matrix) + list(lay.tensor_map) + list(lay.shape):
                meta[pos] = v
                pos += 1
    return meta


def _decode_meta(meta):
    """-> [(dtype, requires_grad, shape, layout or None)]"""
    from .layout import TensorLayout
    meta = meta.tolist()
    out, pos = [], 1
    for _ in range(meta[0]):
        nd = meta[pos + 2]
        dtype, rg, shape = _DTYPES[meta[pos]], bool(meta[pos + 1]), tuple(meta[pos + 3:pos + 3 + nd])
        pos += 3 + nd
        ndm = meta[pos]
        pos += 1
        lay = None
        if ndm >= 0:
            dm = meta[pos:pos + ndm]
            tmap = meta[pos + ndm:pos + ndm + nd]
            full = meta[pos + ndm + nd:pos + ndm + 2 * nd]
            pos += ndm + 2 * nd
            lay = TensorLayout(dm, tmap, full)
        out.append((dtype, rg, shape, lay))
    return out


class PipelineRuntime:
    """Runs one ``PipelineCell`` on the stage this rank belongs to."""

    def __init__(self, cell):
        self.cell = cell
        self.stages = context.get_auto_parallel_context("pipeline_stages")
        self.world = context.get_auto_parallel_context("device_num")
        self.rank = context.get_auto_parallel_context("global_rank")
        if self.world % self.stages != 0:
            raise ValueError("device_num %d is not divisible by pipeline_stages %d" % (self.world, self.stages))
        self.per_stage = self.world // self.stages
        self.stage = self.rank // self.per_stage
        self.micro = cell.micro_size
        self.scheduler = context.get_auto_parallel_context("pipeline_config").get("pipeline_scheduler", "1f1b") \
            if isinstance(context.get_auto_parallel_context("pipeline_config"), dict) else "1f1b"
        if self.scheduler not in ("1f1b", "gpipe"):
            self.scheduler = "1f1b"
        self._meta_cache = {}
        self._pending = []
        self._depth = 0
        self._rec = None
        self._train = True

    # ------------------------------------------------------------------ point to point
    @property
    def _next(self):
        return self.rank + self.per_stage

    @property
    def _prev(self):
        return self.rank - self.per_stage

    def _send(self, tensors, dst, group, key):
        dev = _comm_device()
        if key not in self._meta_cache:
            meta = _encode_meta(tensors).to(dev)
            self._pending.append((dist.isend(meta, dst, group=group), meta))
            self._meta_cache[key] = True
        for t in tensors:
            buf = t.detach().contiguous()
            if buf.device != dev:
                buf = buf.to(dev)
            self._pending.append((dist.isend(buf, dst, group=group), buf))

    def _recv(self, src, group, key, like_device):
        dev = _comm_device()
        if key not in self._meta_cache:
            meta = torch.zeros(_META_LEN, dtype=torch.int64, device=dev)
            dist.recv(meta, src, group=group)
            self._meta_cache[key] = _decode_meta(meta.cpu())
        out = []
        from . import spmd
        for dtype, needs_grad, shape, lay in self._meta_cache[key]:
            buf = torch.empty(shape, dtype=dtype, device=dev)
            dist.recv(buf, src, group=group)
            if buf.device != like_device:
                buf = buf.to(like_device)
            out.append((buf, needs_grad, lay))
        return out

    def _drain(self):
        for work, _keep in self._pending:
            work.wait()
        self._pending = []

    # ------------------------------------------------------------------ stage hook
    def _hook(self, cell, inputs, kwargs):
        if self._depth > 0:
            return cell._call_impl(inputs, kwargs)
        t, s = cell._pipeline_stage, self.stage
        if t < s:
            # a cell of an earlier stage: placeholders stand for its results (``pipeline_outputs`` on the cell says
            # how many when it returns a tuple that the caller unpacks)
            n = int(getattr(cell, "pipeline_outputs", 1) or 1)
            return Skipped.make() if n == 1 else tuple(Skipped.make() for _ in range(n))
        fwd, _ = _direction_groups()
        if t == s:
            n_skipped = sum(1 for a in inputs if _is_skipped(a))
            if n_skipped:
                if self._rec["x_in"]:
                    raise RuntimeError("cell %s of stage %d consumes a value of an earlier stage after the stage has "
                                       "started; only the first cell of a stage may do so" % (cell.cls_name, s))
                got = self._recv(self._prev, fwd, "fwd_in", self._device)
                if len(got) != n_skipped:
                    raise RuntimeError("stage %d expects %d activations from stage %d but %d were sent"
                                       % (s, n_skipped, s - 1, len(got)))
                it = iter(got)
                new_inputs = []
                for a in inputs:
                    if _is_skipped(a):
                        buf, needs_grad, lay = next(it)
                        from ..common.tensor import as_tensor
                        from . import spmd
                        buf = as_tensor(buf)
                        if lay is not None:
                            spmd.set_layout(buf, lay)
                        if self._train and needs_grad and buf.is_floating_point():
                            buf.requires_grad_(True)
                        self._rec["x_in"].append(buf)
                        new_inputs.append(buf)
                    else:
                        new_inputs.append(a)
                inputs = tuple(new_inputs)
            self._depth += 1
            try:
                out = cell._call_impl(inputs, kwargs)
            finally:
                self._depth -= 1
            for o in (out if isinstance(out, (tuple, list)) else (out,)):
                if isinstance(o, torch.Tensor):
                    o._ms_stage_out = s
            return out
        if t != s + 1:
            raise RuntimeError("stage %d hands over to stage %d: stages must be consecutive" % (s, t))
        send = []
        for a in inputs:
            if _is_skipped(a):
                raise RuntimeError("a value of a stage before %d is consumed by stage %d: pass it through stage %d"
                                   % (s, t, s))
            if isinstance(a, torch.Tensor) and (a.requires_grad or getattr(a, "_ms_stage_out", None) is not None):
                send.append(a)
        self._send(send, self._next, fwd, "fwd_out")
        self._rec["y_out"] = send
        raise _StageDone()

    # ------------------------------------------------------------------ one micro-batch
    def _forward(self, i, inputs):
        from ..nn.cell import Cell
        micro_inputs = self.cell.micro_inputs(i, *inputs)
        self._device = next((t.device for t in micro_inputs if isinstance(t, torch.Tensor)), torch.device("cpu"))
        rec = {"x_in": [], "y_out": [], "loss": None}
        self._rec = rec
        prev_hook = Cell._stage_hook
        Cell._stage_hook = self._hook
        try:
            with torch.set_grad_enabled(self._train):
                out = self.cell.network(*micro_inputs)
            if self.stage != self.stages - 1:
                raise RuntimeError("stage %d reached the end of the network without handing over to stage %d; tag "
                                   "the remaining cells with pipeline_stage" % (self.stage, self.stage + 1))
            rec["loss"] = out
        except _StageDone:
            pass
        finally:
            Cell._stage_hook = prev_hook
            self._rec = None
        return rec

    def _backward(self, rec, scale):
        _, bwd = _direction_groups()
        if self.stage == self.stages - 1:
            loss = rec["loss"]
            (loss * scale if scale != 1.0 else loss).backward()
        else:
            outs = [y for y in rec["y_out"] if y.requires_grad]
            grads = []
            dev = _comm_device()
            for y in outs:
                g = torch.empty(y.shape, dtype=y.dtype, device=dev)
                dist.recv(g, self._next, group=bwd)
                grads.append(g if g.device == y.device else g.to(y.device))
            if outs:
                torch.autograd.backward(outs, grads)
        if self.stage > 0:
            dev = _comm_device()
            for x in rec["x_in"]:
                if x.requires_grad:
                    g = x.grad if x.grad is not None else torch.zeros_like(x)
                    g = g.detach().contiguous()
                    if g.device != dev:
                        g = g.to(dev)
                    self._pending.append((dist.isend(g, self._prev, group=bwd), g))
        rec["x_in"], rec["y_out"] = [], []

    # ------------------------------------------------------------------ whole step
    def run(self, inputs, scale=1.0, train=True):
        """Forward (+ backward when ``train``) of all micro-batches in schedule order.  Returns the mean loss on
        the last stage and zero elsewhere."""
        self._train = train
        steps = planner.pipeline_schedule(self.stages, self.stage, self.micro, 1, self.scheduler)
        live, losses = {}, []
        for kind, mb, _chunk in steps:
            if kind == planner.FORWARD:
                rec = self._forward(mb, inputs)
                if rec["loss"] is not None:
                    losses.append(rec["loss"].detach())
                if train:
                    live[mb] = rec
            elif train:
                self._backward(live.pop(mb), scale)
        self._drain()
        if losses:
            return torch.stack([l.float() for l in losses]).mean()
        dev = next((t.device for t in inputs if isinstance(t, torch.Tensor)), torch.device("cpu"))
        return torch.zeros((), device=dev)


def runtime_for(cell):
    rt = getattr(cell, "_pipeline_runtime", None)
    if rt is None:
        rt = PipelineRuntime(cell)
        object.__setattr__(cell, "_pipeline_runtime", rt)
    return rt


def run_pipeline_forward(cell, inputs):
    """Forward-only pass through the pipeline (evaluation / prediction)."""
    return runtime_for(cell).run(inputs, train=False)


def run_pipeline_step(cell, inputs, scale):
    """Forward and backward of every micro-batch; gradients accumulate in the parameters of this stage."""
    return runtime_for(cell).run(inputs, scale=scale, train=True)
