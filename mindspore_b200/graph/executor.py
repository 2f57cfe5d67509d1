"""Graph executor: replays a FuncGraph node list on the current CUDA stream (or CPU).

Forward nodes that the autodiff pass marked ``requires_vjp`` run with detached inputs under ``enable_grad``
and keep (inputs, output) for their ``vjp`` node.  Values are freed after their last use.  With the context
option ``enable_cuda_graph`` and CUDA inputs, the second run is captured into a ``torch.cuda.CUDAGraph`` and
later runs replay it with inputs copied into the captured buffers - one launch per step instead of one per
node, which is what replaces the reference's per-kernel actor dispatch
(runtime/graph_scheduler/graph_scheduler.cc:781, actor/kernel_actor.cc:323).
"""
import operator

import torch
import torch.fx as fx

from .. import context
from ..common.tensor import Tensor
from . import autodiff


def _wrap(o):
    if isinstance(o, torch.Tensor):
        return o if isinstance(o, Tensor) else o.as_subclass(Tensor)
    if isinstance(o, tuple):
        return tuple(_wrap(x) for x in o)
    if isinstance(o, list):
        return [_wrap(x) for x in o]
    return o


class GraphExecutor:
    def __init__(self, fg):
        self.fg = fg
        self.nodes = list(fg.graph.nodes)
        self.last_use = {}
        for i, n in enumerate(self.nodes):
            for a in n.all_input_nodes:
                self.last_use[a] = i
        self.vjp_needed = {n.args[0] for n in self.nodes if n.op == "call_function" and n.target is autodiff.vjp}
        self.memory_plan = self._plan_memory()
        self._comm_stream = None
        self._cuda_graph = None
        self.allow_cuda_graph = True      # a caller that captures the run itself (the micro-batch runner) clears it
        self.use_comm_stream = True       # ... and this: inside its capture every node runs on the capturing stream
        self._static_inputs = None
        self._static_outputs = None
        self._runs = 0

    def _plan_memory(self):
        """Static memory plan of the graph's intermediate values (the reference's SOMAS role,
        backend/common/somas/somas.cc): every node output with a known shape is a tensor living from its node to its
        last user; the native best-fit planner (``msb_memory_plan``) packs them into one arena.  The plan gives
        the peak activation footprint of a replay before anything runs - ``jit`` reports it with ``save_graphs``
        and warns when it exceeds ``max_device_memory`` - and each node's planned offset (``meta['mem_offset']``).
        Execution itself takes its buffers from the caching allocator, which frees at the same last-use points."""
        sizes, starts, ends, owners = [], [], [], []
        for i, n in enumerate(self.nodes):
            shp, dt = n.meta.get("shape"), n.meta.get("dtype")
            if n.op != "call_function" or shp is None or dt is None:
                continue
            numel = 1
            for d in shp:
                numel *= int(d)
            if numel == 0:
                continue
            nbytes = numel * torch.empty((), dtype=dt).element_size()
            end = self.last_use.get(n, i)
            if n.meta.get("requires_vjp") and n.name in self.vjp_needed:
                # kept for its vjp node: alive until that node has run
                end = max(end, next((j for j, m in enumerate(self.nodes) if m.op == "call_function"
                                     and m.target is autodiff.vjp and m.args[0] == n.name), end))
            sizes.append(nbytes)
            starts.append(i)
            ends.append(max(end, i))
            owners.append(n)
        if not sizes:
            return {"arena_bytes": 0, "sum_bytes": 0, "tensors": 0}
        try:
            from ..parallel import planner
            offsets, total = planner.memory_plan(sizes, starts, ends)
        except Exception:  # noqa: BLE001  (host library unavailable: keep running without a plan)
            return {"arena_bytes": None, "sum_bytes": sum(sizes), "tensors": len(sizes)}
        for n, off in zip(owners, offsets):
            n.meta["mem_offset"] = int(off)
        return {"arena_bytes": int(total), "sum_bytes": int(sum(sizes)), "tensors": len(sizes)}

    def run(self, inputs):
        use_cg = self.allow_cuda_graph and context.get_context("enable_cuda_graph") and inputs and all(
            isinstance(t, torch.Tensor) and t.is_cuda for t in inputs)
        if not use_cg:
            return self._run_nodes(inputs)
        self._runs += 1
        if self._cuda_graph is None:
            if self._runs < 2:
                return self._run_nodes(inputs)
            self._static_inputs = [t.clone() for t in inputs]
            torch.cuda.synchronize()
            self._cuda_graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self._cuda_graph):
                self._static_outputs = self._run_nodes(self._static_inputs)
        for s, t in zip(self._static_inputs, inputs):
            s.copy_(t)
        self._cuda_graph.replay()
        return self._static_outputs

    def _run_nodes(self, inputs):
        env = {}
        saved = {}
        it = iter(inputs)
        result = None
        pending = {}       # node -> event: its value is being produced on the communication stream
        on_cuda = any(isinstance(t, torch.Tensor) and t.is_cuda for t in inputs)
        for i, n in enumerate(self.nodes):
            if pending:
                for a in n.all_input_nodes:
                    ev = pending.pop(a, None)
                    if ev is not None:
                        torch.cuda.current_stream().wait_event(ev)
            if n.op == "placeholder":
                env[n] = next(it)
            elif n.op == "get_attr":
                env[n] = n.meta["param"] if "param" in n.meta else n.meta["const"]
            elif n.op == "call_function":
                if n.target is autodiff.vjp:
                    env[n] = self._run_vjp(n, env, saved)
                else:
                    args = fx.node.map_arg(n.args, lambda a: env[a])
                    kwargs = fx.node.map_arg(n.kwargs, lambda a: env[a])
                    if n.meta.get("requires_vjp") and n.name in self.vjp_needed:
                        env[n] = self._run_recorded(n, args, kwargs, saved)
                    elif on_cuda and n.meta.get("comm_stream") and self.use_comm_stream:
                        # a collective whose result is needed later: issue it on the communication stream, the
                        # nodes up to its first user overlap it (optimize_gradients_allreduce_overlap.cc's role)
                        if self._comm_stream is None:
                            self._comm_stream = torch.cuda.Stream()
                        cur = torch.cuda.current_stream()
                        self._comm_stream.wait_stream(cur)
                        with torch.cuda.stream(self._comm_stream):
                            out = n.target(*args, **kwargs)
                        ev = torch.cuda.Event()
                        ev.record(self._comm_stream)
                        for o in (out if isinstance(out, (tuple, list)) else (out,)):
                            if isinstance(o, torch.Tensor):
                                o.record_stream(cur)
                        pending[n] = ev
                        env[n] = out
                    else:
                        env[n] = n.target(*args, **kwargs)
            elif n.op == "output":
                result = fx.node.map_arg(n.args[0], lambda a: env[a])
            for a in n.all_input_nodes:
                if self.last_use.get(a) == i and a.op != "get_attr":
                    env.pop(a, None)
        for ev in pending.values():                       # results nobody consumed: still join the stream
            torch.cuda.current_stream().wait_event(ev)
        return _wrap(result)

    @staticmethod
    def _run_recorded(n, args, kwargs, saved):
        leaves = []

        def prep(a):
            if isinstance(a, torch.Tensor):
                if a.is_floating_point() or a.is_complex():
                    d = a.detach()
                    if type(a) is not type(d) and getattr(a, "main_grad", None) is not None:
                        # A parameter of an arena optimizer: the operator adds its gradient into ``main_grad`` and
                        # hands back nothing.  It sees a fresh alias, not the parameter object: the parameter's
                        # gradient accumulator node lives on the stream it was first used on, and differentiating
                        # with respect to it inside a stream capture would tie the capture to that stream.
                        d = d.as_subclass(type(a))
                        d.__dict__.update(a.__dict__)        # name, layouts, main_grad, flags of the dispatcher
                        d._param_ref = a
                    d.requires_grad_(True)
                    leaves.append(d)
                    return d
                leaves.append(None)
                return a
            if isinstance(a, tuple):
                return tuple(prep(x) for x in a)
            if isinstance(a, list):
                return [prep(x) for x in a]
            if isinstance(a, dict):
                return {k: prep(v) for k, v in a.items()}
            if isinstance(a, slice):
                return slice(prep(a.start), prep(a.stop), prep(a.step))
            return a

        a2 = prep(args)
        k2 = prep(kwargs)
        with torch.enable_grad():
            out = n.target(*a2, **k2)
        saved[n.name] = (leaves, out)
        return out

    @staticmethod
    def _run_vjp(n, env, saved):
        fwd_name, spec = n.args
        leaves, out = saved.pop(fwd_name)
        spec = fx.node.map_arg(spec, lambda a: env[a])
        if isinstance(spec, dict):
            outs, gouts = [], []
            for idx, gval in spec.items():
                o = out[idx]
                if isinstance(o, torch.Tensor) and o.requires_grad and gval is not None:
                    outs.append(o)
                    gouts.append(gval.to(o.dtype) if gval.dtype != o.dtype else gval)
        else:
            outs, gouts = ([out], [spec.to(out.dtype) if spec.dtype != out.dtype else spec]) if (
                isinstance(out, torch.Tensor) and out.requires_grad and spec is not None) else ([], [])
        targets = [l for l in leaves if l is not None and l.requires_grad]
        grads = iter(torch.autograd.grad(outs, targets, gouts, allow_unused=True) if outs and targets
                     else [None] * len(targets))
        res = []
        for l in leaves:
            res.append(next(grads) if (l is not None and l.requires_grad) else None)
        return tuple(res)
