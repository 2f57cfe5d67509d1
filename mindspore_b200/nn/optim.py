"""Optimizers.

Two execution forms share one class hierarchy:

* the reference's per-parameter form - ``optimizer(grads)`` walks (param, grad, state) triples; state
  tensors are Parameters (``moments.*``, ``moment1.*``, ``moment2.*``, ``global_step``), so they are saved
  in checkpoints exactly like the reference's;
* the arena form (``use_arena=True``, default for CUDA bf16 models) - parameters, fp32 masters, moments and
  fp32 gradient accumulators live in flat buffers and one sm_100a kernel per weight-decay group updates
  everything, reading loss-scale / clip factors and the overflow flag from device memory.

Parity: mindspore/python/mindspore/nn/optim/optimizer.py:72-843 (group params, dynamic LR, weight decay,
loss_scale, grad centralization), momentum.py:50, sgd.py, adam.py:471 (Adam), :866 (AdamWeightDecay),
lamb.py, rmsprop.py, adagrad.py, ada_grad, adadelta.py, adamax.py, asgd.py, ftrl.py, lars.py, rprop.py,
proximal_ada_grad.py, adafactor.py.
"""
from __future__ import annotations

import math

import torch

from ..common import dtype as mstype
from ..common.initializer import initializer
from ..common.parameter import Parameter, ParameterTuple
from ..common.tensor import Tensor
from ..ops import kernels as K
from ..ops.primitive import _wrap_out
from .cell import Cell
from .lr_schedule import LearningRateSchedule

_ALIGN = 128  # arena slots are multiples of 128 elements (256 B in bf16, 512 B in fp32)


def _clone_state(params, prefix, init="zeros", dtype=None):
    out = []
    for p in params:
        t = torch.zeros_like(p.detach().as_subclass(torch.Tensor), dtype=dtype or
                             (torch.float32 if p.dtype in (torch.bfloat16, torch.float16) else p.dtype))
        s = Parameter(t, name=prefix + "." + p.name, requires_grad=False, device=p.device)
        s.param_layout = p.param_layout
        s.cloned_from = p
        out.append(s)
    return ParameterTuple(out)


_grad_listeners = []


def note_grad_producer(param):
    """Called in forward (with gradients enabled) by every op whose backward will accumulate into
    ``param.main_grad``.  A parameter used several times in one step (tied embedding / LM head, shared layers) has
    several producers; its gradient is complete only after the last of them has written."""
    param = getattr(param, "_param_ref", param)     # the graph executor hands operators a fresh alias of the parameter
    if getattr(param, "main_grad", None) is not None and torch.is_grad_enabled():
        param._grad_writers = getattr(param, "_grad_writers", 0) + 1


def notify_grad_written(param):
    """Called by backward kernels right after they have accumulated ``param``'s gradient into its arena slice
    (``main_grad``).  Listeners are told once the last registered producer of this step has written; they use it to
    start the gradient collective of a bucket as soon as the bucket is complete."""
    param = getattr(param, "_param_ref", param)
    n = getattr(param, "_grad_writers", 0)
    if n > 1:
        param._grad_writers = n - 1
        return
    param._grad_writers = 0
    for fn in _grad_listeners:
        fn(param)


class ParamArena:
    """Flat storage for a list of same-dtype parameters: low-precision weights, fp32 master copy and fp32
    gradient accumulator, each one contiguous buffer; every parameter becomes a view of the weight buffer and
    gets ``main_grad`` (a view of the gradient buffer) that the wgrad kernels accumulate into."""

    def __init__(self, params, need_master=True):
        assert params, "empty arena"
        dev, dt = params[0].device, params[0].dtype
        for p in params:
            if p.device != dev or p.dtype != dt:
                raise ValueError("arena parameters must share device and dtype")
        self.params = list(params)
        self.offsets = []
        off = 0
        for p in params:
            self.offsets.append(off)
            off += (p.numel() + _ALIGN - 1) // _ALIGN * _ALIGN
        self.total = off
        self.weights = torch.zeros(off, dtype=dt, device=dev)
        self.grads = torch.zeros(off, dtype=torch.float32, device=dev)
        self.master = None
        for p, o in zip(params, self.offsets):
            n = p.numel()
            view = self.weights[o:o + n].view(p.shape)
            view.copy_(p.detach().as_subclass(torch.Tensor))
            p.data = view
            p.main_grad = self.grads[o:o + n].view(p.shape)
            p.arena = self
            p.arena_offset = o
        if need_master and dt != torch.float32:
            self.master = self.weights.float()
        elif dt == torch.float32:
            self.master = self.weights

    def zero_grad(self):
        self.grads.zero_()

    def rebind(self, weights, grads):
        """Moves the arena into other buffers (at least ``total`` elements; e.g. symmetric memory): parameters and
        their ``main_grad`` become views of the new buffers.  ``weights`` must already hold the values."""
        self.weights, self.grads = weights, grads
        for p, o in zip(self.params, self.offsets):
            n = p.numel()
            p.data = weights[o:o + n].view(p.shape)
            p.main_grad = grads[o:o + n].view(p.shape)

    def segment(self, first, last):
        """[start, end) element range covering params[first:last]."""
        start = self.offsets[first]
        end = self.offsets[last] if last < len(self.params) else self.total
        return start, end


class Optimizer(Cell):
    def __init__(self, learning_rate, parameters, weight_decay=0.0, loss_scale=1.0):
        super().__init__(auto_prefix=False)
        parameters = list(parameters) if not isinstance(parameters, (list, tuple)) else list(parameters)
        if not parameters:
            raise ValueError("For 'Optimizer', the argument parameters must not be empty.")
        if isinstance(loss_scale, int):
            loss_scale = float(loss_scale)
        if not isinstance(loss_scale, float) or loss_scale <= 0:
            raise ValueError("For 'Optimizer', 'loss_scale' must be a positive float, got %r" % (loss_scale,))
        self.loss_scale = loss_scale
        self.reciprocal_scale = 1.0 / loss_scale
        self.is_group = isinstance(parameters[0], dict)
        self.is_group_lr = False
        self.is_group_params_ordered = False
        self.group_lr, self.group_weight_decay, self.group_grad_centralization = [], [], []
        if self.is_group:
            flat = []
            ordered = None
            default_lr = learning_rate
            for g in parameters:
                if "order_params" in g:
                    ordered = list(g["order_params"])
                    self.is_group_params_ordered = True
                    continue
                if "params" not in g:
                    raise ValueError("group param dict needs the key 'params'")
                for k in g:
                    if k not in ("params", "lr", "weight_decay", "grad_centralization", "order_params"):
                        raise KeyError("group param key %r is not supported" % k)
                for p in g["params"]:
                    flat.append(p)
                    self.group_lr.append(g.get("lr", default_lr))
                    self.group_weight_decay.append(g.get("weight_decay", weight_decay))
                    self.group_grad_centralization.append(g.get("grad_centralization", False))
                if "lr" in g:
                    self.is_group_lr = True
            if ordered is not None:
                idx = {id(p): i for i, p in enumerate(flat)}
                order = [idx[id(p)] for p in ordered]
                flat = [flat[i] for i in order]
                self.group_lr = [self.group_lr[i] for i in order]
                self.group_weight_decay = [self.group_weight_decay[i] for i in order]
                self.group_grad_centralization = [self.group_grad_centralization[i] for i in order]
            parameters = flat
        else:
            self.group_weight_decay = [weight_decay] * len(parameters)
            self.group_lr = [learning_rate] * len(parameters)
            self.group_grad_centralization = [False] * len(parameters)
        for p in parameters:
            if not isinstance(p, Parameter):
                raise TypeError("For 'Optimizer', all elements of 'parameters' must be Parameter, got %s" % type(p))
        if isinstance(weight_decay, (int, float)) and weight_decay < 0:
            raise ValueError("For 'Optimizer', 'weight_decay' must be >= 0")
        self._parameters = ParameterTuple(parameters)
        self.parameters = self._parameters
        self.weight_decay = weight_decay
        self.exec_weight_decay = any((not isinstance(w, (int, float))) or w > 0 for w in self.group_weight_decay)
        self.learning_rate = learning_rate
        self.dynamic_lr = isinstance(learning_rate, (LearningRateSchedule, list, tuple)) or (
            isinstance(learning_rate, torch.Tensor) and learning_rate.dim() == 1)
        self.global_step = Parameter(torch.zeros(1, dtype=torch.int32), name="global_step", requires_grad=False)
        self._step_host = 0
        self.use_arena = False
        self.arena = None

    # ------------------------------------------------------------------ lr / decay helpers
    def _step(self):
        """The step the update is computed for.  Eagerly a host int.  While a graph is being traced it is the
        ``global_step`` tensor, so that the learning-rate schedule and Adam's bias correction are computed by graph
        nodes at every replay instead of being frozen at their trace-time value."""
        from ..graph import tracer
        if tracer.is_tracing():
            return self.global_step.reshape(()).to(torch.float32)
        return self._step_host

    def _lr_value(self, spec, step):
        if isinstance(step, torch.Tensor):
            if isinstance(spec, LearningRateSchedule):
                return spec(step).to(torch.float32)
            if isinstance(spec, (list, tuple)) or (isinstance(spec, torch.Tensor) and spec.dim() == 1):
                table = torch.as_tensor(spec, dtype=torch.float32, device=step.device)
                return table[step.long().clamp(max=table.numel() - 1)]
            if isinstance(spec, torch.Tensor):
                return float(spec)
            return float(spec)
        if isinstance(spec, LearningRateSchedule):
            v = spec(torch.tensor(step))
            return float(v)
        if isinstance(spec, torch.Tensor):
            if spec.dim() == 0:
                return float(spec)
            return float(spec[min(step, spec.numel() - 1)])
        if isinstance(spec, (list, tuple)):
            return float(spec[min(step, len(spec) - 1)])
        if isinstance(spec, (int, float)):
            if spec < 0:
                raise ValueError("For 'Optimizer', 'learning_rate' must be >= 0")
            return float(spec)
        raise TypeError("learning_rate must be float, Tensor, Iterable or LearningRateSchedule, got %s" % type(spec))

    def get_lr_parameter(self, param):
        """The learning rate (current value) that applies to ``param`` (or to each of a list of parameters)."""
        def one(p):
            if not self.is_group_lr:
                return self.get_lr()
            for i, q in enumerate(self._parameters):
                if q is p or q.name == getattr(p, "name", None):
                    return self.get_lr()[i]
            raise ValueError("The parameter %s is not in the optimizer" % getattr(p, "name", p))
        if isinstance(param, (list, tuple)):
            return [one(p) for p in param]
        return one(param)

    @property
    def target(self):
        """Where the update runs: 'GPU' for CUDA parameters, else 'CPU'."""
        ps = self._parameters
        return self.__dict__.get("_target") or ("GPU" if ps and ps[0].is_cuda else "CPU")

    @target.setter
    def target(self, value):
        if value not in ("CPU", "GPU", "Ascend"):
            raise ValueError("The value must be 'CPU', 'Ascend' or 'GPU', but got value %r" % (value,))
        object.__setattr__(self, "_target", value)

    def get_lr(self):
        step = self._step_host
        if self.is_group_lr:
            return tuple(_wrap_out(torch.tensor(self._lr_value(s, step))) for s in self.group_lr)
        return _wrap_out(torch.tensor(self._lr_value(self.learning_rate, step)))

    def _lrs(self):
        step = self._step()
        if self.is_group_lr:
            return [self._lr_value(s, step) for s in self.group_lr]
        v = self._lr_value(self.learning_rate, step)
        return [v] * len(self._parameters)

    def _wd(self, i):
        w = self.group_weight_decay[i]
        if isinstance(w, (int, float)):
            return float(w)
        if isinstance(w, Cell):
            return float(w(torch.tensor(self._step_host)))
        return float(w)

    def get_weight_decay(self):
        return tuple(self._wd(i) for i in range(len(self._parameters))) if self.is_group else self._wd(0)

    def decay_weight(self, gradients):
        if not self.exec_weight_decay:
            return gradients
        out = []
        for i, (p, g) in enumerate(zip(self._parameters, gradients)):
            wd = self._wd(i)
            out.append(g + wd * p.detach().to(g.dtype) if wd > 0 and self._decay_flag(p) else g)
        return tuple(out)

    @staticmethod
    def _decay_flag(p):
        return True

    def scale_grad(self, gradients):
        if self.reciprocal_scale == 1.0:
            return gradients
        return tuple(g * self.reciprocal_scale for g in gradients)

    def gradients_centralization(self, gradients):
        out = []
        for flag, g in zip(self.group_grad_centralization, gradients):
            if flag and g.dim() > 1:
                g = g - g.mean(tuple(range(1, g.dim())), keepdim=True)
            out.append(g)
        return tuple(out)

    def flatten_gradients(self, gradients):
        return gradients

    def _advance(self):
        self._step_host += 1
        with torch.no_grad():
            torch.Tensor.add_(self.global_step, 1)

    def broadcast_params(self, optim_result):
        return optim_result

    def predicated(self, gradients, skip):
        """The update, applied unless the 0-d bool tensor ``skip`` is set - without reading ``skip`` on the host,
        so the whole step stays one graph (and one CUDA graph).  Every tensor the update writes (parameters, the
        optimizer's states and its step counter) is put back where ``skip`` holds.  Arena optimizers do the same
        inside their kernels (``fused_step(check_finite=True)``)."""
        if self.use_arena:
            raise RuntimeError("arena optimizers skip an update inside their kernels: use fused_step(check_finite=True)")
        touched, seen = [], set()
        for p in list(self._parameters) + list(self.get_parameters()):
            if id(p) not in seen:
                seen.add(id(p))
                touched.append(p)
        old = [p.detach().as_subclass(torch.Tensor).clone() for p in touched]
        out = self(gradients)
        keep = skip.reshape(()).to(torch.bool)
        with torch.no_grad():
            for p, o in zip(touched, old):
                cur = p.detach().as_subclass(torch.Tensor)      # in-place on the detached alias replays in any grad mode
                cur.copy_(torch.where(keep, o, cur))
        return out

    @property
    def unique(self):
        return True

    def _prep(self, gradients):
        gradients = self.flatten_gradients(gradients)
        gradients = self.decay_weight(gradients)
        gradients = self.gradients_centralization(gradients)
        return self.scale_grad(gradients)

    def construct(self, gradients):
        raise NotImplementedError

    # ------------------------------------------------------------------ arena form
    def _enable_arena(self, decay_fn=None):
        """Packs parameters into flat buffers, decayed parameters first."""
        params = list(self._parameters)
        wds = [self._wd(i) if (decay_fn is None or decay_fn(p)) else 0.0 for i, p in enumerate(params)]
        order = sorted(range(len(params)), key=lambda i: (wds[i] == 0.0, i))
        self._arena_order = order
        ordered = [params[i] for i in order]
        self.arena = ParamArena(ordered)
        import weakref
        self.arena.owner = weakref.ref(self)
        # contiguous runs of equal weight decay -> one kernel launch each
        self._arena_groups = []
        start = 0
        for j in range(1, len(order) + 1):
            if j == len(order) or wds[order[j]] != wds[order[start]]:
                self._arena_groups.append((start, j, wds[order[start]]))
                start = j
        self.use_arena = True
        dev = self.arena.weights.device
        self._hyper = [torch.zeros(8, dtype=torch.float32, device=dev) for _ in self._arena_groups]
        self._sumsq = torch.zeros(1, dtype=torch.float32, device=dev)
        self._nonfinite = torch.zeros(1, dtype=torch.int32, device=dev)
        self._skip = torch.zeros(1, dtype=torch.int32, device=dev)
        self._gscale = torch.ones(1, dtype=torch.float32, device=dev)
        self._gnorm = torch.zeros(1, dtype=torch.float32, device=dev)
        return self.arena

    def zero_grad(self):
        if self.arena is not None:
            self.arena.zero_grad()

    # ------------------------------------------------------------------ arena state <-> checkpoints
    def _state_views(self, buf, prefix):
        """Per-parameter Parameters ``<prefix>.<name>`` that alias slices of the flat state buffer ``buf``: they are
        saved and loaded like the reference's cloned optimizer states (``adam_m.*``, ``adam_v.*``, ``moments.*``;
        nn/optim/adam.py:866, momentum.py:50) while the fused kernels keep working on the flat buffer."""
        out = []
        for prm, off in zip(self.arena.params, self.arena.offsets):
            s = Parameter(torch.empty(0, dtype=buf.dtype), name=prefix + "." + prm.name, requires_grad=False,
                          device=buf.device)
            s.data = buf[off:off + prm.numel()].view(prm.shape)
            s.param_layout = prm.param_layout
            s.cloned_from = prm
            out.append(s)
        return ParameterTuple(out)

    def _flat_state(self, buf, name):
        s = Parameter(torch.empty(0, dtype=buf.dtype), name=name, requires_grad=False, device=buf.device)
        s.data = buf
        return ParameterTuple([s])

    def _expose_arena_state(self):
        """(Re)builds the checkpoint view of the arena state.  Full arena: per-parameter views of the moments and of
        the fp32 master copy.  Sharded over a data-parallel group: this rank's slice of master / moments as three
        flat tensors (``*.opt_shard``), saved per rank like the reference's sliced optimizer states."""
        arena = self.arena
        if arena is None:
            return
        dp = getattr(self, "_dp", None)
        names = self._arena_state_names()
        if dp is not None and dp.shard:
            for (attr, prefix), buf in zip(names, dp.state_buffers()):
                setattr(self, attr, self._flat_state(buf, prefix + ".opt_shard"))
            self.fp32_master = self._flat_state(dp.master, "fp32_master.opt_shard")
            return
        for (attr, prefix), buf in zip(names, self._arena_state_buffers()):
            setattr(self, attr, self._state_views(buf, prefix))
        if arena.master is not None and arena.master is not arena.weights:
            self.fp32_master = self._state_views(arena.master, "fp32_master")

    def _arena_state_names(self):
        return ()

    def _arena_state_buffers(self):
        return ()

    def sync_step_from_checkpoint(self):
        """After ``global_step`` was loaded from a checkpoint: the host-side step (learning-rate schedule, bias
        correction) follows it."""
        self._step_host = int(self.global_step.detach().reshape(-1)[0])

    def write_master(self, param, value):
        """Copies ``value`` (what was just written into ``param``) into the fp32 master copy of ``param`` (full
        arena, or the owned part of a sharded one), so that the next update does not bring the old weights back from
        the master."""
        arena = self.arena
        if arena is None or getattr(param, "arena", None) is not arena:
            return
        new = value.detach().as_subclass(torch.Tensor).to(param.device)
        o, n = param.arena_offset, param.numel()
        flat = new.reshape(-1).float()
        dp = getattr(self, "_dp", None)
        if dp is not None and dp.shard:
            lo, hi = max(o, dp.lo), min(o + n, dp.hi)
            if lo < hi:
                dp.master[lo - dp.lo:hi - dp.lo].copy_(flat[lo - o:hi - o])
        elif arena.master is not None and arena.master is not arena.weights:
            arena.master[o:o + n].copy_(flat)

    # ------------------------------------------------------------------ model-parallel awareness (arena form)
    def set_model_parallel_group(self, group_name):
        """Tells the optimizer that parameters flagged ``tp_sharded`` hold different shards on every rank of
        ``group_name`` while the others are replicated there.  The global gradient norm then sums the sharded
        part across the group, and gradients of parameters flagged ``tp_grad_reduce`` (replicated parameters fed
        by token-sharded activations) are all-reduced before the update - over their ``mirror_group`` when the
        parallel dispatcher recorded one, else over ``group_name``.  The flags are read at the first step, so
        they may be set by the first forward pass."""
        assert self.arena is not None, "set_model_parallel_group needs the arena form"
        self._mp_group = group_name
        self._mp_runs_ready = False
        self._sumsq_sh = torch.zeros_like(self._sumsq)

    def set_pipeline_parallel_group(self, group_name):
        """Ranks of ``group_name`` hold the same parameter slices but train different pipeline stages: a parameter
        has a non-zero gradient on its own stage only, so the squared gradient norm (and the overflow flag) is
        summed over the group to give every stage the global norm."""
        self._pp_group = group_name

    def _ensure_mp_runs(self):
        if getattr(self, "_mp_runs_ready", True):
            return
        arena = self.arena

        def runs(key):
            out, start, cur = [], 0, None
            for i, p in enumerate(arena.params):
                f = key(p)
                if cur is None:
                    cur, start = f, i
                elif f != cur:
                    out.append((arena.segment(start, i), cur))
                    cur, start = f, i
            out.append((arena.segment(start, len(arena.params)), cur))
            return out
        self._norm_runs = runs(lambda p: bool(getattr(p, "tp_sharded", False)))
        self._reduce_runs = [(seg, g) for seg, g in runs(
            lambda p: (getattr(p, "mirror_group", None) or self._mp_group)
            if getattr(p, "tp_grad_reduce", False) else None) if g is not None]
        self._mp_runs_ready = True

    def set_data_parallel_group(self, group_name, mean=True, shard=False, fused=True):
        """Gradients of the arena are averaged over ``group_name`` before the update.  With ``shard`` the fp32
        master weights and the moments are split over the group (parallel optimizer): every rank updates one slice
        and the new weights are gathered back (``parallel.zero``)."""
        assert self.arena is not None, "set_data_parallel_group needs the arena form"
        from ..parallel.zero import DataParallelArena
        self._dp = DataParallelArena(self, group_name, mean, shard, fused)
        self._expose_arena_state()

    def sync_data_parallel_grads(self):
        dp = getattr(self, "_dp", None)
        if dp is not None and not dp.shard:
            dp.allreduce()

    def sync_model_parallel_grads(self):
        group = getattr(self, "_mp_group", None)
        if group is None:
            return
        from ..communication import comm_func as CF
        from ..communication import management as M
        self._ensure_mp_runs()
        for (s, e), gname in self._reduce_runs:
            CF._all_reduce_(self.arena.grads[s:e], "sum", M._group(gname))

    def _accumulate_sumsq(self):
        arena = self.arena
        self._sumsq.zero_()
        self._nonfinite.zero_()
        group = getattr(self, "_mp_group", None)
        dp = getattr(self, "_dp", None)
        if group is None and dp is not None and dp.local_only and not dp.shard:
            # parameters that differ per data-parallel rank (expert shards): their squared norms add up over the
            # group, the replicated rest counts once - every rank ends with the same global norm
            from ..communication import comm_func as CF
            part = torch.zeros_like(self._sumsq)
            pos = 0
            for s, e in sorted(dp.local_only):
                if s > pos:
                    K.sumsq_finite(arena.grads[pos:s], self._sumsq, self._nonfinite)
                K.sumsq_finite(arena.grads[s:e], part, self._nonfinite)
                pos = e
            if pos < arena.total:
                K.sumsq_finite(arena.grads[pos:arena.total], self._sumsq, self._nonfinite)
            CF._all_reduce_(part, "sum", dp.group)
            CF._all_reduce_(self._nonfinite, "max", dp.group)
            self._sumsq.add_(part)
            return
        if group is None:
            K.sumsq_finite(arena.grads, self._sumsq, self._nonfinite)
            return
        from ..communication import comm_func as CF
        from ..communication import management as M
        self._ensure_mp_runs()
        self._sumsq_sh.zero_()
        for (s, e), sharded in self._norm_runs:
            K.sumsq_finite(arena.grads[s:e], self._sumsq_sh if sharded else self._sumsq, self._nonfinite)
        g = M._group(group)
        CF._all_reduce_(self._sumsq_sh, "sum", g)
        CF._all_reduce_(self._nonfinite, "max", g)
        self._sumsq.add_(self._sumsq_sh)
        pp = getattr(self, "_pp_group", None)
        if pp is not None:
            CF._all_reduce_(self._sumsq, "sum", M._group(pp))
            CF._all_reduce_(self._nonfinite, "max", M._group(pp))


def _to_plain(t):
    return t.detach().as_subclass(torch.Tensor) if isinstance(t, torch.Tensor) else t


def _fill_hyper(h, start, values):
    """Writes scalars (host numbers, or 0-d tensors when the step is traced) into the device hyper-parameter
    vector: one host-to-device copy when all are numbers."""
    if not any(isinstance(v, torch.Tensor) for v in values):
        h[start:start + len(values)] = torch.tensor(values, dtype=torch.float32)
        return
    for i, v in enumerate(values):
        if isinstance(v, torch.Tensor):
            h[start + i:start + i + 1].copy_(v.reshape(1).to(h.dtype))
        else:
            h[start + i] = float(v)


class Momentum(Optimizer):
    def __init__(self, params, learning_rate, momentum, weight_decay=0.0, loss_scale=1.0, use_nesterov=False,
                 use_arena=None, decay_filter=None):
        super().__init__(learning_rate, params, weight_decay, loss_scale)
        if isinstance(momentum, float) and momentum < 0.0:
            raise ValueError("For 'Momentum', the argument 'momentum' must be at least 0.0, but got %s" % momentum)
        self.momentum = float(momentum)
        self.use_nesterov = use_nesterov
        p0 = self._parameters[0]
        same = all(p.device == p0.device and p.dtype == p0.dtype for p in self._parameters)
        if use_arena is None:
            use_arena = same and p0.is_cuda and p0.dtype == torch.bfloat16
        if use_arena:
            # flat form: bf16 weights, fp32 master + accumulator, one kernel per weight-decay group
            arena = self._enable_arena(decay_filter or (lambda p: p.dim() > 1))
            self._accum = torch.zeros(arena.total, dtype=torch.float32, device=arena.weights.device)
            self._expose_arena_state()
        else:
            self.moments = _clone_state(self._parameters, "moments")

    def _arena_state_names(self):
        return (("moments", "moments"),)

    def _arena_state_buffers(self):
        return (self._accum,)

    def fused_step(self, inv_loss_scale=1.0, check_finite=False, advance=True):
        arena = self.arena
        lr = self._lr_value(self.learning_rate, self._step())
        skip = None
        if check_finite or inv_loss_scale != 1.0:
            self._accumulate_sumsq()
            K.finalize_grad_scale(self._sumsq, self._nonfinite, inv_loss_scale, 0.0, self._gscale, self._skip,
                                  self._gnorm)
            skip = self._skip if check_finite else None
        for gi, (first, last, wd) in enumerate(self._arena_groups):
            s, e = arena.segment(first, last)
            h = self._hyper[gi]
            _fill_hyper(h, 0, [lr, self.momentum, wd])
            h[3:4].copy_(self._gscale)
            h[4] = 1.0 if self.use_nesterov else 0.0
            lp = arena.weights[s:e] if arena.master is not arena.weights else None
            K.momentum_step(arena.master[s:e], self._accum[s:e], arena.grads[s:e], lp, h, skip)
        if advance:
            self._advance()
        return True

    def construct(self, gradients=None):
        if self.use_arena:
            return self.fused_step()
        gradients = self._prep(gradients)
        lrs = self._lrs()
        with torch.no_grad():
            for p, g, m, lr in zip(self._parameters, gradients, self.moments, lrs):
                pt, mt, gt = _to_plain(p), _to_plain(m), _to_plain(g).to(m.dtype)
                mt.mul_(self.momentum).add_(gt)
                upd = gt + mt * self.momentum if self.use_nesterov else mt
                if pt.dtype != mt.dtype:
                    pt.copy_((pt.to(mt.dtype) - lr * upd).to(pt.dtype))
                else:
                    pt.sub_(upd * lr)
        self._advance()
        return True


class SGD(Optimizer):
    def __init__(self, params, learning_rate=0.1, momentum=0.0, dampening=0.0, weight_decay=0.0, nesterov=False,
                 loss_scale=1.0):
        super().__init__(learning_rate, params, weight_decay, loss_scale)
        if nesterov and (momentum <= 0 or dampening != 0):
            raise ValueError("For 'SGD', if 'nesterov' is true, 'momentum' must be > 0.0 and 'dampening' must be 0.0")
        self.momentum, self.dampening, self.nesterov = float(momentum), float(dampening), nesterov
        self.accum = _clone_state(self._parameters, "accum")
        self._first = True

    def construct(self, gradients):
        gradients = self._prep(gradients)
        lrs = self._lrs()
        with torch.no_grad():
            for p, g, a, lr in zip(self._parameters, gradients, self.accum, lrs):
                pt, at, gt = _to_plain(p), _to_plain(a), _to_plain(g).to(a.dtype)
                if self.momentum != 0:
                    step = self._step()
                    if isinstance(step, torch.Tensor):
                        # traced: "first step" is decided by the step counter at every replay
                        at.copy_(torch.where(step == 0, gt, at * self.momentum + gt * (1 - self.dampening)))
                    elif self._first:
                        at.copy_(gt)
                    else:
                        at.mul_(self.momentum).add_(gt, alpha=1 - self.dampening)
                    gt = gt + self.momentum * at if self.nesterov else at
                pt.sub_((lr * gt).to(pt.dtype))
        self._first = False
        self._advance()
        return True


class Adam(Optimizer):
    def __init__(self, params, learning_rate=1e-3, beta1=0.9, beta2=0.999, eps=1e-8, use_locking=False,
                 use_nesterov=False, weight_decay=0.0, loss_scale=1.0, use_amsgrad=False, **kwargs):
        super().__init__(learning_rate, params, weight_decay, loss_scale)
        if not 0 < beta1 < 1 or not 0 < beta2 < 1:
            raise ValueError("For 'Adam', beta1 and beta2 must be in (0, 1)")
        if eps <= 0:
            raise ValueError("For 'Adam', eps must be positive")
        self.beta1, self.beta2, self.eps, self.use_nesterov, self.use_amsgrad = beta1, beta2, eps, use_nesterov, use_amsgrad
        self.moment1 = _clone_state(self._parameters, "moment1")
        self.moment2 = _clone_state(self._parameters, "moment2")
        self.vhat = _clone_state(self._parameters, "vhat") if use_amsgrad else None

    def construct(self, gradients):
        gradients = self._prep(gradients)
        lrs = self._lrs()
        t = self._step() + 1
        bc1, bc2 = 1 - self.beta1 ** t, 1 - self.beta2 ** t
        with torch.no_grad():
            for i, (p, g, m, v, lr) in enumerate(zip(self._parameters, gradients, self.moment1, self.moment2, lrs)):
                pt, mt, vt, gt = _to_plain(p), _to_plain(m), _to_plain(v), _to_plain(g).to(m.dtype)
                mt.mul_(self.beta1).add_(gt, alpha=1 - self.beta1)
                vt.mul_(self.beta2).addcmul_(gt, gt, value=1 - self.beta2)
                vv = vt
                if self.use_amsgrad:
                    vh = _to_plain(self.vhat[i])
                    torch.maximum(vh, vt, out=vh)
                    vv = vh
                lr_t = lr * bc2 ** 0.5 / bc1
                num = (self.beta1 * mt + (1 - self.beta1) * gt) if self.use_nesterov else mt
                upd = lr_t * num / (vv.sqrt() + self.eps)
                pt.copy_((pt.to(upd.dtype) - upd).to(pt.dtype))
        self._advance()
        return True


class AdamWeightDecay(Optimizer):
    """AdamW without bias correction in the per-parameter form (reference adam.py:866 semantics); the arena
    form applies bias correction (``bias_correction=True``), the usual choice for LLM pre-training."""

    def __init__(self, params, learning_rate=1e-3, beta1=0.9, beta2=0.999, eps=1e-6, weight_decay=0.0,
                 use_arena=None, bias_correction=None, max_grad_norm=0.0, decay_filter=None):
        super().__init__(learning_rate, params, weight_decay, 1.0)
        if not 0 < beta1 < 1 or not 0 < beta2 < 1:
            raise ValueError("For 'AdamWeightDecay', beta1 and beta2 must be in (0, 1)")
        if eps <= 0:
            raise ValueError("For 'AdamWeightDecay', eps must be positive")
        self.beta1, self.beta2, self.eps = beta1, beta2, eps
        self.max_grad_norm = max_grad_norm
        p0 = self._parameters[0]
        same = all(p.device == p0.device and p.dtype == p0.dtype for p in self._parameters)
        if use_arena is None:
            use_arena = same and p0.is_cuda and p0.dtype == torch.bfloat16
        self.bias_correction = bool(use_arena) if bias_correction is None else bias_correction
        self.decay_filter = decay_filter or (lambda p: p.dim() > 1)
        if use_arena:
            arena = self._enable_arena(self.decay_filter)
            self._m = torch.zeros(arena.total, dtype=torch.float32, device=arena.weights.device)
            self._v = torch.zeros(arena.total, dtype=torch.float32, device=arena.weights.device)
            self._expose_arena_state()
        else:
            self.moment1 = _clone_state(self._parameters, "adam_m")
            self.moment2 = _clone_state(self._parameters, "adam_v")

    def _decay_flag(self, p):
        return self.decay_filter(p)

    def _arena_state_names(self):
        return (("moment1", "adam_m"), ("moment2", "adam_v"))

    def _arena_state_buffers(self):
        return (self._m, self._v)

    def decay_weight(self, gradients):
        return gradients  # decoupled decay is applied in the update itself

    def construct(self, gradients=None):
        if self.use_arena:
            return self.fused_step()
        gradients = self._prep(gradients)
        lrs = self._lrs()
        t = self._step() + 1
        bc1 = 1 - self.beta1 ** t if self.bias_correction else 1.0
        bc2 = 1 - self.beta2 ** t if self.bias_correction else 1.0
        with torch.no_grad():
            for i, (p, g, m, v, lr) in enumerate(zip(self._parameters, gradients, self.moment1, self.moment2, lrs)):
                pt, mt, vt, gt = _to_plain(p), _to_plain(m), _to_plain(v), _to_plain(g).to(m.dtype)
                mt.mul_(self.beta1).add_(gt, alpha=1 - self.beta1)
                vt.mul_(self.beta2).addcmul_(gt, gt, value=1 - self.beta2)
                wd = self._wd(i) if self.decay_filter(p) else 0.0
                upd = (mt / bc1) / ((vt / bc2).sqrt() + self.eps) + wd * pt.to(mt.dtype)
                pt.copy_((pt.to(mt.dtype) - lr * upd).to(pt.dtype))
        self._advance()
        return True

    def fused_step(self, inv_loss_scale=1.0, check_finite=False, advance=True):
        """One kernel per decay group over the flat arena; clip and overflow-skip decided on the device.  With
        ``advance=False`` the caller advances the step counter itself (after it has read the skip flag)."""
        dp = getattr(self, "_dp", None)
        if dp is not None and dp.shard:
            return dp.sharded_step(inv_loss_scale, check_finite, advance)
        arena = self.arena
        t = self._step() + 1
        lr = self._lr_value(self.learning_rate, self._step())
        bc1 = 1 - self.beta1 ** t if self.bias_correction else 1.0
        bc2 = 1 - self.beta2 ** t if self.bias_correction else 1.0
        skip = None
        if self.max_grad_norm > 0 or check_finite or inv_loss_scale != 1.0:
            self._accumulate_sumsq()
            K.finalize_grad_scale(self._sumsq, self._nonfinite, inv_loss_scale, self.max_grad_norm, self._gscale,
                                  self._skip, self._gnorm)
            skip = self._skip if check_finite else None
        for gi, (first, last, wd) in enumerate(self._arena_groups):
            s, e = arena.segment(first, last)
            h = self._hyper[gi]
            _fill_hyper(h, 0, [lr, self.beta1, self.beta2, self.eps, wd, bc1, bc2])
            h[7:8].copy_(self._gscale)
            lp = arena.weights[s:e] if arena.master is not arena.weights else None
            K.adamw_step(arena.master[s:e], self._m[s:e], self._v[s:e], arena.grads[s:e], lp, h, skip)
        if advance:
            self._advance()
        return True


AdamW = AdamWeightDecay


class Lamb(Optimizer):
    def __init__(self, params, learning_rate, beta1=0.9, beta2=0.999, eps=1e-6, weight_decay=0.0):
        super().__init__(learning_rate, params, weight_decay, 1.0)
        self.beta1, self.beta2, self.eps = beta1, beta2, eps
        self.moment1 = _clone_state(self._parameters, "lamb_m")
        self.moment2 = _clone_state(self._parameters, "lamb_v")

    def decay_weight(self, gradients):
        return gradients

    def construct(self, gradients):
        gradients = self._prep(gradients)
        lrs = self._lrs()
        t = self._step() + 1
        with torch.no_grad():
            for i, (p, g, m, v, lr) in enumerate(zip(self._parameters, gradients, self.moment1, self.moment2, lrs)):
                pt, mt, vt, gt = _to_plain(p), _to_plain(m), _to_plain(v), _to_plain(g).to(m.dtype)
                mt.mul_(self.beta1).add_(gt, alpha=1 - self.beta1)
                vt.mul_(self.beta2).addcmul_(gt, gt, value=1 - self.beta2)
                mh, vh = mt / (1 - self.beta1 ** t), vt / (1 - self.beta2 ** t)
                upd = mh / (vh.sqrt() + self.eps) + self._wd(i) * pt.to(mt.dtype)
                wn, un = pt.float().norm(), upd.norm()
                trust = torch.where((wn > 0) & (un > 0), wn / un, torch.ones_like(wn))
                pt.copy_((pt.to(mt.dtype) - lr * trust * upd).to(pt.dtype))
        self._advance()
        return True


class RMSProp(Optimizer):
    def __init__(self, params, learning_rate=0.1, decay=0.9, momentum=0.0, epsilon=1e-10, use_locking=False,
                 centered=False, loss_scale=1.0, weight_decay=0.0):
        super().__init__(learning_rate, params, weight_decay, loss_scale)
        self.decay, self.momentum, self.epsilon, self.centered = decay, momentum, epsilon, centered
        self.ms = _clone_state(self._parameters, "mean_square")
        self.mom = _clone_state(self._parameters, "moment")
        self.mg = _clone_state(self._parameters, "mean_grad") if centered else None

    def construct(self, gradients):
        gradients = self._prep(gradients)
        lrs = self._lrs()
        with torch.no_grad():
            for i, (p, g, s, mo, lr) in enumerate(zip(self._parameters, gradients, self.ms, self.mom, lrs)):
                pt, st, mt, gt = _to_plain(p), _to_plain(s), _to_plain(mo), _to_plain(g).to(s.dtype)
                st.mul_(self.decay).addcmul_(gt, gt, value=1 - self.decay)
                denom = st
                if self.centered:
                    mg = _to_plain(self.mg[i])
                    mg.mul_(self.decay).add_(gt, alpha=1 - self.decay)
                    denom = st - mg * mg
                mt.mul_(self.momentum).add_(lr * gt / (denom + self.epsilon).sqrt())
                pt.sub_(mt.to(pt.dtype))
        self._advance()
        return True


class Adagrad(Optimizer):
    def __init__(self, params, accum=0.1, learning_rate=0.001, update_slots=True, loss_scale=1.0, weight_decay=0.0):
        super().__init__(learning_rate, params, weight_decay, loss_scale)
        self.accum = _clone_state(self._parameters, "accum")
        with torch.no_grad():
            for a in self.accum:
                _to_plain(a).fill_(accum)

    def construct(self, gradients):
        gradients = self._prep(gradients)
        with torch.no_grad():
            for p, g, a, lr in zip(self._parameters, gradients, self.accum, self._lrs()):
                pt, at, gt = _to_plain(p), _to_plain(a), _to_plain(g).to(a.dtype)
                at.addcmul_(gt, gt)
                pt.sub_((lr * gt / at.sqrt()).to(pt.dtype))
        self._advance()
        return True


class Adadelta(Optimizer):
    def __init__(self, params, learning_rate=1.0, rho=0.9, epsilon=1e-6, loss_scale=1.0, weight_decay=0.0):
        super().__init__(learning_rate, params, weight_decay, loss_scale)
        self.rho, self.epsilon = rho, epsilon
        self.accum = _clone_state(self._parameters, "accum")
        self.accum_update = _clone_state(self._parameters, "accum_update")

    def construct(self, gradients):
        gradients = self._prep(gradients)
        with torch.no_grad():
            for p, g, a, au, lr in zip(self._parameters, gradients, self.accum, self.accum_update, self._lrs()):
                pt, at, ut, gt = _to_plain(p), _to_plain(a), _to_plain(au), _to_plain(g).to(a.dtype)
                at.mul_(self.rho).addcmul_(gt, gt, value=1 - self.rho)
                upd = (ut + self.epsilon).sqrt() / (at + self.epsilon).sqrt() * gt
                ut.mul_(self.rho).addcmul_(upd, upd, value=1 - self.rho)
                pt.sub_((lr * upd).to(pt.dtype))
        self._advance()
        return True


class AdaMax(Optimizer):
    def __init__(self, params, learning_rate=0.001, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.0,
                 loss_scale=1.0):
        super().__init__(learning_rate, params, weight_decay, loss_scale)
        self.beta1, self.beta2, self.eps = beta1, beta2, eps
        self.moment1 = _clone_state(self._parameters, "moment1")
        self.moment2 = _clone_state(self._parameters, "moment2")

    def construct(self, gradients):
        gradients = self._prep(gradients)
        t = self._step() + 1
        with torch.no_grad():
            for p, g, m, v, lr in zip(self._parameters, gradients, self.moment1, self.moment2, self._lrs()):
                pt, mt, vt, gt = _to_plain(p), _to_plain(m), _to_plain(v), _to_plain(g).to(m.dtype)
                mt.mul_(self.beta1).add_(gt, alpha=1 - self.beta1)
                torch.maximum(vt * self.beta2, gt.abs(), out=vt)
                pt.sub_((lr / (1 - self.beta1 ** t) * mt / (vt + self.eps)).to(pt.dtype))
        self._advance()
        return True


class ASGD(Optimizer):
    def __init__(self, params, learning_rate=0.1, lambd=1e-4, alpha=0.75, t0=1e6, weight_decay=0.0):
        super().__init__(learning_rate, params, weight_decay, 1.0)
        self.lambd, self.alpha, self.t0 = lambd, alpha, t0
        self.ax = _clone_state(self._parameters, "ax")
        self.eta, self.mu = None, 1.0

    def construct(self, gradients):
        gradients = self._prep(gradients)
        step = self._step() + 1
        with torch.no_grad():
            for p, g, ax, lr in zip(self._parameters, gradients, self.ax, self._lrs()):
                eta = lr / ((1 + self.lambd * lr * step) ** self.alpha)
                pt, at, gt = _to_plain(p), _to_plain(ax), _to_plain(g).to(ax.dtype)
                pt.mul_(1 - self.lambd * eta).sub_((eta * gt).to(pt.dtype))
                mu = 1 / max(1, step - self.t0)
                at.add_((pt.to(at.dtype) - at) * mu)
        self._advance()
        return True


class Rprop(Optimizer):
    def __init__(self, params, learning_rate=0.1, etas=(0.5, 1.2), step_sizes=(1e-6, 50.0), weight_decay=0.0):
        super().__init__(learning_rate, params, weight_decay, 1.0)
        self.etaminus, self.etaplus = etas
        self.smin, self.smax = step_sizes
        self.prev = _clone_state(self._parameters, "prev")
        self.step_size = _clone_state(self._parameters, "step_size")
        with torch.no_grad():
            for s, lr in zip(self.step_size, self._lrs()):
                _to_plain(s).fill_(lr)

    def construct(self, gradients):
        gradients = self._prep(gradients)
        with torch.no_grad():
            for p, g, pr, ss in zip(self._parameters, gradients, self.prev, self.step_size):
                pt, prt, st, gt = _to_plain(p), _to_plain(pr), _to_plain(ss), _to_plain(g).to(pr.dtype).clone()
                sign = (gt * prt).sign()
                factor = torch.where(sign > 0, self.etaplus, torch.where(sign < 0, self.etaminus, 1.0))
                st.mul_(factor).clamp_(self.smin, self.smax)
                gt[sign < 0] = 0
                pt.sub_((gt.sign() * st).to(pt.dtype))
                prt.copy_(gt)
        self._advance()
        return True


class FTRL(Optimizer):
    def __init__(self, params, initial_accum=0.1, learning_rate=0.001, lr_power=-0.5, l1=0.0, l2=0.0,
                 use_locking=False, loss_scale=1.0, weight_decay=0.0):
        super().__init__(learning_rate, params, weight_decay, loss_scale)
        self.lr_power, self.l1, self.l2 = lr_power, l1, l2
        self.accum = _clone_state(self._parameters, "accum")
        self.linear = _clone_state(self._parameters, "linear")
        with torch.no_grad():
            for a in self.accum:
                _to_plain(a).fill_(initial_accum)

    def construct(self, gradients):
        gradients = self._prep(gradients)
        with torch.no_grad():
            for p, g, a, l, lr in zip(self._parameters, gradients, self.accum, self.linear, self._lrs()):
                pt, at, lt, gt = _to_plain(p), _to_plain(a), _to_plain(l), _to_plain(g).to(a.dtype)
                new_a = at + gt * gt
                sigma = (new_a.pow(-self.lr_power) - at.pow(-self.lr_power)) / lr
                lt.add_(gt - sigma * pt.to(at.dtype))
                quad = new_a.pow(-self.lr_power) / lr + 2 * self.l2
                pt.copy_(torch.where(lt.abs() > self.l1, (lt.sign() * self.l1 - lt) / quad,
                                     torch.zeros_like(lt)).to(pt.dtype))
                at.copy_(new_a)
        self._advance()
        return True


class ProximalAdagrad(Optimizer):
    def __init__(self, params, accum=0.1, learning_rate=0.001, l1=0.0, l2=0.0, use_locking=False, loss_scale=1.0,
                 weight_decay=0.0):
        super().__init__(learning_rate, params, weight_decay, loss_scale)
        self.l1, self.l2 = l1, l2
        self.accum = _clone_state(self._parameters, "accum")
        with torch.no_grad():
            for a in self.accum:
                _to_plain(a).fill_(accum)

    def construct(self, gradients):
        gradients = self._prep(gradients)
        with torch.no_grad():
            for p, g, a, lr in zip(self._parameters, gradients, self.accum, self._lrs()):
                pt, at, gt = _to_plain(p), _to_plain(a), _to_plain(g).to(a.dtype)
                at.addcmul_(gt, gt)
                eta = lr / at.sqrt()
                prox = pt.to(at.dtype) - eta * gt
                new = prox.sign() * torch.clamp(prox.abs() - eta * self.l1, min=0) / (1 + eta * self.l2)
                pt.copy_(new.to(pt.dtype))
        self._advance()
        return True


class LARS(Optimizer):
    """Layer-wise adaptive rate scaling wrapped around another optimizer (nn/optim/lars.py)."""

    def __init__(self, optimizer, epsilon=1e-5, coefficient=0.001, use_clip=False, lars_filter=lambda x: "LayerNorm"
                 not in x.name):
        super().__init__(optimizer.learning_rate, list(optimizer._parameters), 0.0, 1.0)
        self.opt, self.epsilon, self.coefficient, self.lars_filter = optimizer, epsilon, coefficient, lars_filter

    def construct(self, gradients):
        out = []
        for i, (p, g) in enumerate(zip(self._parameters, gradients)):
            if self.lars_filter(p):
                wn, gn = _to_plain(p).float().norm(), _to_plain(g).float().norm()
                wd = self.opt._wd(i)
                trust = torch.where((wn > 0) & (gn > 0), self.coefficient * wn / (gn + wd * wn + self.epsilon),
                                    torch.ones_like(wn))
                g = (g + wd * p.detach().to(g.dtype)) * trust.to(g.dtype)
            out.append(g)
        return self.opt(tuple(out))


class AdaFactor(Optimizer):
    def __init__(self, params, learning_rate=None, eps=(1e-30, 1e-3), clip_threshold=1.0, decay_rate=0.8, beta1=0.9,
                 weight_decay=0.0, scale_lr=True, scale_parameter=True, relative_step=True, warmup_init=False,
                 compression=False, loss_scale=1.0):
        super().__init__(learning_rate if learning_rate is not None else 1e-3, params, weight_decay, loss_scale)
        self._torch_opt = None
        self._kw = dict(lr=learning_rate, eps2=eps, clip=clip_threshold, decay=decay_rate, beta1=beta1)
        self.exp_avg_sq_row = _clone_state([p for p in self._parameters if p.dim() >= 2], "exp_avg_sq_row")
        self.exp_avg_sq = _clone_state(self._parameters, "exp_avg_sq")

    def construct(self, gradients):
        gradients = self._prep(gradients)
        t = self._step() + 1
        rho = 1 - t ** (-self._kw["decay"])
        e1, e2 = self._kw["eps2"]
        with torch.no_grad():
            for p, g, v, lr in zip(self._parameters, gradients, self.exp_avg_sq, self._lrs()):
                pt, vt, gt = _to_plain(p), _to_plain(v), _to_plain(g).float()
                vt.mul_(rho).add_((gt * gt + e1) * (1 - rho))
                upd = gt / vt.sqrt()
                upd = upd / max(1.0, float((upd.pow(2).mean().sqrt()) / self._kw["clip"]))
                scale = max(e2, float(pt.float().pow(2).mean().sqrt()))
                pt.sub_((lr * scale * upd).to(pt.dtype))
        self._advance()
        return True


from .optim_ext import *  # noqa: E402,F401,F403
