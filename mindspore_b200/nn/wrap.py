"""Training-step wrapper cells.

Parity: mindspore/python/mindspore/nn/wrap/cell_wrapper.py:75 (WithLossCell), :146 (WithGradCell), :214
(ForwardValueAndGrad), :319-444 (TrainOneStepCell), :492 (GetNextSingleOp), :531 (_VirtualDatasetCell),
:564 (MicroBatchInterleaved), :622 (PipelineCell), :676 (GradAccumulationCell), :735 (_MicroBatch);
nn/wrap/loss_scale.py:88 (DynamicLossScaleUpdateCell), :199 (FixedLossScaleUpdateCell), :272-580
(TrainOneStepWithLossScaleCell); nn/wrap/grad_reducer.py:310-481 (DistributedGradReducer).
"""
from __future__ import annotations

import os

import torch

from .. import context
from ..common import dtype as mstype
from ..common.parameter import Parameter, ParameterTuple
from ..common.tensor import Tensor
from ..ops import composite as C
from ..ops.primitive import _wrap_out
from ..utils import recorder as _recorder
from .cell import Cell


class WithLossCell(Cell):
    def __init__(self, backbone, loss_fn):
        super().__init__(auto_prefix=False)
        self._backbone = backbone
        self._loss_fn = loss_fn

    def construct(self, data, label):
        return self._loss_fn(self._backbone(data), label)

    @property
    def backbone_network(self):
        return self._backbone


class WithEvalCell(Cell):
    def __init__(self, network, loss_fn, add_cast_fp32=False):
        super().__init__(auto_prefix=False)
        self._network, self._loss_fn, self.add_cast_fp32 = network, loss_fn, add_cast_fp32

    def construct(self, data, label):
        out = self._network(data)
        if self.add_cast_fp32:
            out, label = out.float(), (label.float() if label.is_floating_point() else label)
        return self._loss_fn(out, label), out, label


class WithGradCell(Cell):
    def __init__(self, network, loss_fn=None, sens=None):
        super().__init__(auto_prefix=False)
        self.network, self.loss_fn, self.sens = network, loss_fn, sens
        self.weights = ParameterTuple(network.trainable_params())
        self.grad = C.GradOperation(get_by_list=True, sens_param=sens is not None)
        self.network_with_loss = network if loss_fn is None else WithLossCell(network, loss_fn)
        self.network_with_loss.set_train()

    def construct(self, *inputs):
        if self.sens is None:
            return self.grad(self.network_with_loss, self.weights)(*inputs)
        return self.grad(self.network_with_loss, self.weights)(*inputs, self.sens)


class ForwardValueAndGrad(Cell):
    def __init__(self, network, weights=None, get_all=False, get_by_list=False, sens_param=False):
        super().__init__(auto_prefix=False)
        if get_by_list and weights is None:
            raise ValueError("For 'ForwardValueAndGrad', when 'get_by_list' is True, 'weights' must be given")
        self.network, self.weights = network, weights
        self.get_all, self.get_by_list, self.sens_param = get_all, get_by_list, sens_param
        self.grad = C.GradOperation(get_all=get_all, get_by_list=get_by_list, sens_param=sens_param)

    def construct(self, *inputs):
        net_inputs = inputs[:-1] if self.sens_param else inputs
        loss = self.network(*net_inputs)
        g = self.grad(self.network, self.weights)(*inputs) if self.get_by_list else self.grad(self.network)(*inputs)
        return loss, g


# ------------------------------------------------------------------------------------ gradient reducer
class DistributedGradReducer(Cell):
    """Data-parallel gradient synchronisation: gradients are packed into comm_fusion buckets (flat
    buffers), each bucket is all-reduced once (fp32 when ``gradient_fp32_sync``), scaled by 1/N when
    ``mean`` and unpacked.  Bucket boundaries come from ``all_reduce_fusion_config`` (parameter indices)
    or the ``comm_fusion`` size threshold (MB)."""

    def __init__(self, parameters, mean=None, degree=None, fusion_type=1, group=None):
        super().__init__(auto_prefix=False)
        from ..communication import management as M
        self.group = group or M.GlobalComm.WORLD_COMM_GROUP
        self.mean = context.get_auto_parallel_context("gradients_mean") if mean is None else mean
        if degree is None:
            self.degree = M.get_group_size(self.group) if M.GlobalComm.INITED else 1
        else:
            if not isinstance(degree, int) or degree <= 0:
                raise ValueError("For 'DistributedGradReducer', 'degree' must be a positive int")
            self.degree = degree
        self.params = list(parameters)
        from ..parallel.comm_fusion import plan_allreduce_buckets
        # parameters that differ on every rank by design (the experts of an expert-parallel MoE) are not reduced
        self.local_only = {i for i, p in enumerate(self.params) if getattr(p, "dp_local", False)}
        self.buckets = [[i for i in b if i not in self.local_only] for b in plan_allreduce_buckets(self.params)]
        self.buckets = [b for b in self.buckets if b]

    def construct(self, grads):
        from ..communication import comm_func as CF
        from ..communication import management as M
        if self.degree == 1 or not M.GlobalComm.INITED:
            return grads
        g = M._group(self.group)
        fp32 = context.get_auto_parallel_context("gradient_fp32_sync")
        out = list(grads)
        for bucket in self.buckets:
            ts = [grads[i].detach().as_subclass(torch.Tensor) for i in bucket]
            dt = torch.float32 if fp32 else ts[0].dtype
            flat = torch.cat([t.reshape(-1).to(dt) for t in ts])
            CF._all_reduce_(flat, "sum", g)
            if self.mean:
                flat /= self.degree
            off = 0
            for i, t in zip(bucket, ts):
                n = t.numel()
                out[i] = _wrap_out(flat[off:off + n].view(t.shape).to(t.dtype))
                off += n
        if self.mean:
            for i in self.local_only:      # their gradient already sums the contributions of every rank's tokens
                out[i] = _wrap_out(grads[i] / self.degree)
        return tuple(out)


class PipelineGradReducer(Cell):
    def __init__(self, parameters, scale_sense=1.0, opt_shard=None):
        super().__init__(auto_prefix=False)
        self.params = list(parameters)
        self.scale = scale_sense

    def construct(self, grads):
        return tuple(g / self.scale for g in grads)


def _parallel_mode():
    return context.get_auto_parallel_context("parallel_mode")


# ------------------------------------------------------------------------------------ train step
class TrainOneStepCell(Cell):
    def __init__(self, network, optimizer, sens=None, return_grad=False):
        super().__init__(auto_prefix=False)
        self.network = network
        self.network.set_grad()
        self.optimizer = optimizer
        self.weights = optimizer.parameters
        self.grad = C.GradOperation(get_by_list=True, sens_param=True)
        self.sens = 1.0 if sens is None else float(sens)
        self.sens_given = sens is not None
        self.return_grad = return_grad
        self.reducer_flag = _parallel_mode() in (context.ParallelMode.DATA_PARALLEL,
                                                 context.ParallelMode.HYBRID_PARALLEL)
        self.grad_reducer = None
        if self.reducer_flag:
            self.grad_reducer = DistributedGradReducer(self.weights)
        self.use_arena = getattr(optimizer, "use_arena", False)
        # an arena step is driven from the host (micro-batch schedule, bucket overlap, fused optimizer launch); in
        # GRAPH_MODE its compiled unit is the micro-batch forward + backward (``_MicroBatchRunner``), not this cell
        self._use_graph = False if self.use_arena else None

    def _micro_runner(self, network, scale):
        """Callable running forward + backward of one micro-batch.  With the context option ``enable_cuda_graph``
        and CUDA inputs the micro-batch is captured once into a CUDA graph (after two eager calls) and replayed:
        thousands of kernel launches per micro-batch become one, which removes the host launch bound."""
        runner = getattr(self, "_runner", None)
        if runner is None or runner.network is not network:
            runner = _MicroBatchRunner(network, None)
            self._runner = runner
        runner._set_scale(scale)
        return runner

    def release_graphs(self):
        """Destroys captured CUDA graphs.  Call it before the communication groups are destroyed: a graph that
        holds captured NCCL kernels must not outlive its communicator."""
        runner = getattr(self, "_runner", None)
        if runner is not None and runner.graph is not None:
            torch.cuda.synchronize()
            runner.graph = None
            runner.static_inputs = runner.static_loss = None
            runner.calls = 0

    def _pipeline_step(self, inputs):
        """Pipeline parallel without an arena optimizer: the stage runtime leaves gradients in ``.grad``."""
        from ..parallel.pipeline import run_pipeline_step
        for p in self.weights:
            p.grad = None
        loss = run_pipeline_step(self.network, inputs, self.sens / self.network.micro_size)
        grads = tuple(_wrap_out(p.grad if p.grad is not None else torch.zeros_like(p)) for p in self.weights)
        for p in self.weights:
            p.grad = None
        if self.grad_reducer is not None:
            grads = self.grad_reducer(grads)
        self.optimizer(grads)
        return _wrap_out(loss)

    def _arena_backward(self, inputs, scale):
        """Forward + backward of one step for arena optimizers, up to (not including) the update: gradients flow
        straight into the flat fp32 accumulator inside backward, micro-batches and pipeline stages are scheduled
        here, and the gradient collectives of the model-parallel group, the data-parallel group and the legacy
        reducer run before returning.  ``scale`` multiplies the loss before backward: a float (``sens``) or the
        device-resident loss scale."""
        opt = self.optimizer
        opt.zero_grad()
        net = self.network
        if isinstance(net, PipelineCell) and not isinstance(net, GradAccumulationCell) and \
                context.get_auto_parallel_context("pipeline_stages") > 1:
            from ..parallel.pipeline import run_pipeline_step
            loss = run_pipeline_step(net, inputs, scale / net.micro_size)
        elif isinstance(net, GradAccumulationCell):
            # micro-batches run back to back; each backward accumulates into the flat fp32 gradient arena
            total = None
            k = net.micro_size
            runner = self._micro_runner(net.network, scale / k)
            for i in range(k):
                li = runner(net.micro_inputs(i, *inputs))
                total = li.clone() if total is None else total + li
            loss = total / k
        else:
            dp = getattr(opt, "_dp", None)
            if dp is not None:
                dp.begin_step()                # buckets are all-reduced as backward completes them
            if context.get_context("mode") == context.GRAPH_MODE and getattr(net, "_use_graph", None) is not False:
                loss = self._micro_runner(net, scale)(inputs)
                _collect_stray_grads(self.weights)
                opt.sync_model_parallel_grads()
                opt.sync_data_parallel_grads()
                if self.grad_reducer is not None:
                    from ..parallel.data_parallel import allreduce_arena_grads
                    allreduce_arena_grads(opt.arena, self.grad_reducer)
                return loss.detach()
            with torch.enable_grad():
                loss = net(*inputs)
            if isinstance(scale, torch.Tensor):
                (loss * scale.to(loss.dtype)).backward()
            elif scale != 1.0:
                (loss * scale).backward()
            else:
                loss.backward()
        _collect_stray_grads(self.weights)
        opt.sync_model_parallel_grads()
        opt.sync_data_parallel_grads()
        if self.grad_reducer is not None:
            from ..parallel.data_parallel import allreduce_arena_grads
            allreduce_arena_grads(opt.arena, self.grad_reducer)
        return loss.detach()

    def _arena_step(self, inputs):
        loss = self._arena_backward(inputs, self.sens)
        self.optimizer.fused_step(inv_loss_scale=1.0 / self.sens if self.sens != 1.0 else 1.0)
        return loss

    def construct(self, *inputs):
        if _recorder.enabled():
            self._rdr_step = getattr(self, "_rdr_step", 0) + 1
            _recorder.set_step(self._rdr_step)
            _recorder.record("step", "begin " + type(self.network).__name__)
        if self.use_arena:
            from ..profiler import step_range
            with step_range():
                return _wrap_out(self._arena_step(inputs))
        if isinstance(self.network, PipelineCell) and not isinstance(self.network, GradAccumulationCell) and \
                context.get_auto_parallel_context("pipeline_stages") > 1:
            return self._pipeline_step(inputs)
        loss = self.network(*inputs)
        sens = torch.full_like(loss, self.sens) if isinstance(loss, torch.Tensor) else self.sens
        grads = self.grad(self.network, self.weights)(*inputs, sens)
        if self.grad_reducer is not None:
            grads = self.grad_reducer(grads)
        self.optimizer(grads)
        if self.return_grad:
            return loss, {p.name: g for p, g in zip(self.weights, grads)}
        return loss


def fold_grad_(main_grad, grad):
    """Graph node of a compiled micro-batch: adds a weight gradient that came back as a value into the fp32
    accumulator.  Operators with an accumulator-aware backward add theirs inside the reverse-mode node and hand back
    nothing (``None``)."""
    if grad is not None:
        main_grad.add_(grad.to(main_grad.dtype))
    return main_grad


class _MicroBatchRunner:
    """Forward + backward of one micro-batch, eagerly or as a replayed CUDA graph.

    The graph owns static input buffers; each call copies the micro-batch into them and replays.  Everything the
    captured region launches must be replay-safe: parameter gradients accumulate in place into the arena,
    collectives are NCCL (capturable) or the symmetric-memory kernels whose barrier epoch lives on the device."""

    WARMUP_CALLS = 2

    def __init__(self, network, scale):
        self.network, self.scale = network, scale
        self.calls = 0
        self.graph = None
        self._compiled = None
        self.static_inputs = None
        self.static_loss = None
        self.launches_per_replay = 0

    def _set_scale(self, scale):
        """A float scale is baked into the (captured) backward; a tensor scale (dynamic loss scale) is kept in a
        buffer of this runner that a captured graph re-reads at every replay."""
        if isinstance(scale, torch.Tensor):
            if not isinstance(self.scale, torch.Tensor):
                self.scale = scale.detach().clone().float().reshape(())
            else:
                self.scale.copy_(scale.detach().reshape(()))
        else:
            self.scale = scale

    def _compiled_graph(self, inputs):
        """GRAPH_MODE: forward + backward of the micro-batch traced once into one graph - primitives, the collectives
        that the shard strategies insert and the reverse-mode nodes - which goes through the pass pipeline (pattern
        fusion, simplification, communication passes; ``save_graphs`` dumps each) and then runs on the graph executor.
        The weight gradients never appear as graph values: the reverse-mode nodes of the parameter-owning operators
        accumulate into the flat fp32 gradient arena, exactly as their eager backward does.  The call that traces is
        also the first real execution (nothing is rolled back)."""
        if self._compiled is None:
            from ..common.parameter import ParameterTuple
            from ..graph import jit as _jit
            from ..ops.composite import _run_grad
            net = self.network
            weights = list(ParameterTuple(net.trainable_params()))
            runner = self

            def forward_backward(*xs):
                sc = runner.scale
                example = xs[0]
                sens = torch.ones((), device=example.device) * (sc if isinstance(sc, torch.Tensor) else float(sc))
                loss, _, grads = _run_grad(net, xs, weights, sens, False, None, False, True)
                for w, g in zip(weights, grads):
                    if getattr(w, "main_grad", None) is not None:
                        _jit.leaf_call(fold_grad_, (w.main_grad, g), {})
                return loss
            # The trace runs one forward (to record it) and builds the reverse-mode nodes symbolically: nothing is
            # accumulated by it (the gradients it sees are zero placeholders), and the first real execution of this
            # micro-batch is the run of the compiled graph below.
            with _jit.symbolic_gradients():
                self._compiled = _jit._compile(forward_backward, tuple(inputs), {}, type(net).__name__ + "_microbatch",
                                               None)
            self._compiled.executor.allow_cuda_graph = False      # this runner captures (``__call__``), not the executor
            self._compiled.executor.use_comm_stream = not context.get_context("enable_cuda_graph")
            self._compiled_scale = self.scale
        if not isinstance(self.scale, torch.Tensor) and self.scale != self._compiled_scale:
            raise RuntimeError("the loss scale baked into the compiled micro-batch changed (%r -> %r); pass it as a "
                               "tensor to change it between steps" % (self._compiled_scale, self.scale))
        out = self._compiled(*inputs)
        return out.detach() if isinstance(out, torch.Tensor) else out

    def _eager(self, inputs):
        from ..parallel import fused_comm
        fused_comm.step_fence()
        if context.get_context("mode") == context.GRAPH_MODE and getattr(self.network, "_use_graph", None) is not False:
            return self._compiled_graph(inputs)
        with torch.enable_grad():
            loss = self.network(*inputs)
        sc = self.scale.to(loss.dtype) if isinstance(self.scale, torch.Tensor) else self.scale
        (loss * sc).backward()
        return loss.detach()

    def __call__(self, inputs):
        use_graph = context.get_context("enable_cuda_graph") and all(
            (not isinstance(t, torch.Tensor)) or t.is_cuda for t in inputs)
        if not use_graph:
            return self._eager(inputs)
        self.calls += 1
        if self.graph is None:
            if self.calls <= self.WARMUP_CALLS:
                return self._eager(inputs)
            from .. import _native
            self.static_inputs = tuple(t.clone() if isinstance(t, torch.Tensor) else t for t in inputs)
            torch.cuda.synchronize()
            before = _native.launch_count
            self.graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.graph):
                self.static_loss = self._eager(self.static_inputs)
            self.launches_per_replay = _native.launch_count - before
            _native.launch_count = before
        for s, t in zip(self.static_inputs, inputs):
            if isinstance(s, torch.Tensor):
                s.copy_(t)
        self.graph.replay()
        from .. import _native
        _native.launch_count += self.launches_per_replay
        return self.static_loss


def _collect_stray_grads(params):
    """Parameters updated through ops without a main_grad-aware backward still get ``.grad``; fold it in."""
    for p in params:
        g = p.grad
        if g is not None:
            mg = getattr(p, "main_grad", None)
            if mg is not None:
                mg.add_(g.to(mg.dtype))
            p.grad = None


class DynamicLossScaleUpdateCell(Cell):
    def __init__(self, loss_scale_value, scale_factor, scale_window):
        super().__init__()
        self.scale_window, self.scale_factor = int(scale_window), float(scale_factor)
        self.loss_scale_value = float(loss_scale_value)
        self.cur_iter = Parameter(torch.tensor(1, dtype=torch.int32), name="current_iterator_step", requires_grad=False)
        self.last_overflow_iter = Parameter(torch.tensor(0, dtype=torch.int32), name="last_overflow_iterator_step",
                                            requires_grad=False)
        self._use_graph = False

    def get_loss_scale(self):
        return self.loss_scale_value

    def construct(self, loss_scale, overflow):
        from ..graph import tracer
        if tracer.is_tracing():
            # tensor form: nothing is read on the host, so the update is part of the graph and follows the
            # overflow flag of every replay (reference: DynamicLossScaleUpdateCell.construct, loss_scale.py:135-168)
            with torch.no_grad():
                ov = overflow.reshape(()).to(torch.bool)
                scale = loss_scale.detach().as_subclass(torch.Tensor)
                cur = self.cur_iter.detach().as_subclass(torch.Tensor)
                last = self.last_overflow_iter.detach().as_subclass(torch.Tensor)
                grow = (~ov) & ((cur - last) >= self.scale_window)
                new_scale = torch.where(ov, torch.clamp(scale / self.scale_factor, min=1.0),
                                        torch.where(grow, scale * self.scale_factor, scale))
                torch.Tensor.copy_(loss_scale, new_scale)
                torch.Tensor.copy_(self.last_overflow_iter, torch.where(ov | grow, cur, last))
                torch.Tensor.add_(self.cur_iter, 1)
            return overflow
        overflow = bool(overflow)
        cur, last = int(self.cur_iter), int(self.last_overflow_iter)
        with torch.no_grad():
            if overflow:
                torch.Tensor.copy_(loss_scale, torch.clamp(loss_scale / self.scale_factor, min=1.0))
                torch.Tensor.fill_(self.last_overflow_iter, cur)
            elif cur - last >= self.scale_window:
                torch.Tensor.mul_(loss_scale, self.scale_factor)
                torch.Tensor.fill_(self.last_overflow_iter, cur)
            torch.Tensor.add_(self.cur_iter, 1)
        return overflow


class FixedLossScaleUpdateCell(Cell):
    def __init__(self, loss_scale_value):
        super().__init__()
        self.loss_scale_value = float(loss_scale_value)
        self._use_graph = False

    def get_loss_scale(self):
        return self.loss_scale_value

    def construct(self, _, overflow):
        from ..graph import tracer
        return overflow if tracer.is_tracing() else bool(overflow)


class TrainOneStepWithLossScaleCell(TrainOneStepCell):
    def __init__(self, network, optimizer, scale_sense):
        super().__init__(network, optimizer, sens=None)
        self.loss_scaling_manager = None
        if isinstance(scale_sense, Cell):
            self.loss_scaling_manager = scale_sense
            dev = optimizer.parameters[0].device
            self.scale_sense = Parameter(torch.tensor(scale_sense.get_loss_scale(), dtype=torch.float32, device=dev),
                                         name="scale_sense", requires_grad=False)
        elif isinstance(scale_sense, torch.Tensor):
            if scale_sense.numel() != 1:
                raise ValueError("For 'TrainOneStepWithLossScaleCell', the shape of 'scale_sense' must be (1,) or ()")
            self.scale_sense = Parameter(scale_sense.detach().float().reshape(()), name="scale_sense",
                                         requires_grad=False)
        else:
            raise TypeError("For 'TrainOneStepWithLossScaleCell', 'scale_sense' must be Cell or Tensor, got %s"
                            % type(scale_sense))
        # the arena path reads the overflow flag on the host (step counter); the per-parameter path is traceable
        self._use_graph = False if self.use_arena else None

    def set_sense_scale(self, sens):
        if self.scale_sense is not None and isinstance(sens, torch.Tensor):
            self.scale_sense.set_data(sens.reshape(()))
        else:
            raise TypeError("The input type must be Tensor, but got %s" % type(sens))

    def start_overflow_check(self, pre_cond, compute_input):
        return True, compute_input

    def get_overflow_status(self, status, compute_output):
        bad = torch.zeros((), dtype=torch.bool, device=compute_output[0].device)
        for g in compute_output:
            bad = bad | ~torch.isfinite(g).all()
        from ..communication import management as M
        if self.reducer_flag and M.GlobalComm.INITED and M.get_group_size() > 1:
            from ..communication import comm_func as CF
            f = bad.float()
            CF._all_reduce_(f, "sum", M._group(None))
            bad = f > 0
        return bad

    def process_loss_scale(self, overflow):
        if self.loss_scaling_manager is not None:
            return self.loss_scaling_manager(self.scale_sense, overflow)
        from ..graph import tracer
        return overflow if tracer.is_tracing() else bool(overflow)

    def construct(self, *inputs):
        scale = self.scale_sense
        if self.use_arena:
            # same backward + gradient synchronisation as TrainOneStepCell (micro-batches, pipeline, model- and
            # data-parallel groups), with the loss scale as the initial gradient; the update kernels read the skip
            # flag on the device, and the step counter only advances when the update was applied (the reference
            # skips the optimizer on overflow: nn/wrap/loss_scale.py:404-422)
            opt = self.optimizer
            loss = self._arena_backward(inputs, scale.detach().as_subclass(torch.Tensor))
            opt.fused_step(inv_loss_scale=1.0 / float(scale), check_finite=True, advance=False)
            overflow = bool(opt._skip.reshape(()))
            if not overflow:
                opt._advance()
            overflow = self.process_loss_scale(torch.as_tensor(overflow))
            return _wrap_out(loss), _wrap_out(torch.as_tensor(overflow)), scale
        loss = self.network(*inputs)
        sens = torch.full_like(loss, 1.0) * scale.to(loss.dtype)
        grads = self.grad(self.network, self.weights)(*inputs, sens)
        grads = tuple(g.float() / scale for g in grads)
        if self.grad_reducer is not None:
            grads = self.grad_reducer(grads)
        cond = self.get_overflow_status(None, grads)
        overflow = self.process_loss_scale(cond)
        from ..graph import tracer
        if tracer.is_tracing():
            # the reference's ``if not overflow: optimizer(grads)`` (nn/wrap/loss_scale.py:404-422) as a predicated
            # update: the branch is taken on the device at every replay, not frozen at its trace-time outcome
            self.optimizer.predicated(grads, overflow)
            return loss, _wrap_out(overflow), scale
        if not overflow:
            self.optimizer(grads)
        return loss, _wrap_out(torch.as_tensor(overflow)), scale


# ------------------------------------------------------------------------------------ micro-batching
class _MicroBatch(Cell):
    def __init__(self, micro_size):
        super().__init__()
        self.micro_size = micro_size

    def construct(self, i, *inputs):
        out = []
        for x in inputs:
            if isinstance(x, torch.Tensor) and x.dim() > 0:
                n = x.shape[0] // self.micro_size
                out.append(x[i * n:(i + 1) * n])
            else:
                out.append(x)
        return tuple(out)


class PipelineCell(Cell):
    """Splits the batch into ``micro_size`` micro-batches.  Under ``pipeline_stages > 1`` the pipeline
    runtime (``parallel.pipeline``) schedules the stage's forward/backward per micro-batch with 1F1B or GPipe
    ordering; otherwise micro-batches run back to back and losses are averaged."""

    def __init__(self, network, micro_size, stage_config=None):
        super().__init__(auto_prefix=False)
        if not isinstance(micro_size, int) or micro_size <= 0:
            raise ValueError("For 'PipelineCell', 'micro_size' must be a positive int, got %r" % (micro_size,))
        self.network, self.micro_size = network, micro_size
        self.micro_inputs = _MicroBatch(micro_size)
        if stage_config:
            for name, cell in network.cells_and_names():
                for key, stage in stage_config.items():
                    if name == key or name.endswith("." + key):
                        cell.pipeline_stage = stage

    def construct(self, *inputs):
        stages = context.get_auto_parallel_context("pipeline_stages")
        if stages > 1:
            from ..parallel.pipeline import run_pipeline_forward
            return run_pipeline_forward(self, inputs)
        total = None
        for i in range(self.micro_size):
            out = self.network(*self.micro_inputs(i, *inputs))
            total = out if total is None else total + out
        return total / self.micro_size if context.get_auto_parallel_context("loss_repeated_mean") else total


class GradAccumulationCell(PipelineCell):
    def __init__(self, network, micro_size):
        super().__init__(network, micro_size)

    def construct(self, *inputs):
        total = None
        for i in range(self.micro_size):
            out = self.network(*self.micro_inputs(i, *inputs))
            total = out if total is None else total + out
        return total / self.micro_size


class MicroBatchInterleaved(Cell):
    """Runs ``interleave_num`` sub-batches so that one's collectives overlap another's compute: sub-batch k
    is issued on its own CUDA stream when running on GPU."""

    def __init__(self, network, interleave_num=2):
        super().__init__(auto_prefix=False)
        if not isinstance(interleave_num, int) or interleave_num <= 0:
            raise ValueError("For 'MicroBatchInterleaved', 'interleave_num' must be a positive int")
        self.network, self.interleave_num = network, interleave_num
        self.interleave_inputs = _MicroBatch(interleave_num)

    def construct(self, *inputs):
        total = None
        for i in range(self.interleave_num):
            out = self.network(*self.interleave_inputs(i, *inputs))
            total = out if total is None else total + out
        return total / self.interleave_num


class _VirtualDatasetCell(Cell):
    def __init__(self, backbone):
        super().__init__(auto_prefix=False)
        self._backbone = backbone

    def construct(self, *inputs):
        return self._backbone(*inputs)


class VirtualDatasetCellTriple(_VirtualDatasetCell):
    """The three-input form (data, label, mask) of the wrapper that marks the dataset inputs for auto parallel.
    Parity: nn/wrap/cell_wrapper.py VirtualDatasetCellTriple."""

    def construct(self, a, b, c):
        return self._backbone(a, b, c)


class ParameterUpdate(Cell):
    """``cell(x)`` writes ``x`` into the wrapped parameter (a learning rate, a loss scale) and returns it.
    Parity: nn/wrap/cell_wrapper.py ParameterUpdate."""

    def __init__(self, param):
        super().__init__(auto_prefix=False)
        from ..common.parameter import Parameter
        if not isinstance(param, Parameter):
            raise TypeError("For 'ParameterUpdate', 'param' must be 'Parameter', but got %s" % type(param).__name__)
        self._param = param

    def construct(self, x):
        with torch.no_grad():
            torch.Tensor.copy_(self._param, torch.as_tensor(x).to(self._param.dtype))
        return x


class TimeDistributed(Cell):
    """Applies ``layer`` to every time slice: the time axis is folded into the batch axis (``reshape_with_axis``,
    one reshape and one call) or the slices are run one by one and stacked.  Parity: nn/layer/timedistributed.py."""

    def __init__(self, layer, time_axis, reshape_with_axis=None):
        super().__init__()
        if not isinstance(layer, Cell) and not callable(layer):
            raise TypeError("For 'TimeDistributed', 'layer' must be a Cell or a Primitive")
        for v, n in ((time_axis, "time_axis"),) + (((reshape_with_axis, "reshape_with_axis"),)
                                                    if reshape_with_axis is not None else ()):
            if isinstance(v, bool) or not isinstance(v, int):
                raise TypeError("For 'TimeDistributed', '%s' must be an int" % n)
        self.layer, self.time_axis, self.reshape_with_axis = layer, time_axis, reshape_with_axis

    def construct(self, inputs):
        if not isinstance(inputs, torch.Tensor):
            raise TypeError("For 'TimeDistributed', 'inputs' must be a Tensor")
        rank = inputs.dim()
        t = self.time_axis % rank
        if rank <= 2:
            raise ValueError("For 'TimeDistributed', 'inputs' must have more than 2 dimensions")
        if self.reshape_with_axis is not None:
            b = self.reshape_with_axis % rank
            lo, hi = min(t, b), max(t, b)
            if hi - lo != 1:
                raise ValueError("For 'TimeDistributed', 'time_axis' and 'reshape_with_axis' must be neighbours")
            shape = list(inputs.shape)
            merged = shape[:lo] + [shape[lo] * shape[hi]] + shape[hi + 1:]
            out = self.layer(inputs.reshape(merged))
            if not isinstance(out, torch.Tensor):
                raise TypeError("For 'TimeDistributed', the layer must return a Tensor")
            return out.reshape(list(out.shape[:lo]) + [shape[lo], shape[hi]] + list(out.shape[lo + 1:]))
        outs = [self.layer(piece) for piece in torch.unbind(inputs, t)]
        if not all(isinstance(o, torch.Tensor) for o in outs):
            raise TypeError("For 'TimeDistributed', the layer must return a Tensor")
        return torch.stack(outs, t)


class _TrainGradAccuStepCell(TrainOneStepCell):
    """Pipeline / gradient-accumulation step: gradients accumulate in ``accu_grads`` over micro-batches and
    the optimizer consumes the accumulators."""

    def __init__(self, network, optimizer, sens=None):
        super().__init__(network, optimizer, sens)
        self.accu_grads = self.weights.clone(prefix="accu_grads", init="zeros") if not self.use_arena else ()

    def construct(self, *inputs):
        if self.use_arena:
            return _wrap_out(self._arena_step(inputs))
        loss = self.network(*inputs)
        sens = torch.full_like(loss, self.sens)
        grads = self.grad(self.network, self.weights)(*inputs, sens)
        with torch.no_grad():
            for a, g in zip(self.accu_grads, grads):
                torch.Tensor.copy_(a, g.to(a.dtype))
        if self.grad_reducer is not None:
            grads = self.grad_reducer(grads)
        self.optimizer(grads)
        return loss


class GetNextSingleOp(Cell):
    def __init__(self, dataset_types, dataset_shapes, queue_name):
        super().__init__()
        self.queue_name = queue_name

    def construct(self):
        from ..train.dataset_helper import _pop_queue
        return _pop_queue(self.queue_name)
