"""Graph mode: ``@jit`` and GRAPH_MODE cell compilation.

Pipeline (the reference's action list, pipeline/jit/ps/action.cc:1887-2038, re-thought for this runtime):

1. **trace**   - ``construct`` runs once on the example inputs under a ``TorchFunctionMode``; every Primitive /
   fused-op call and every other torch call becomes one node of a ``torch.fx.Graph`` in execution (ANF) order.
   Python control flow is unrolled and shapes are specialised, as graph mode does for constants.
2. **autodiff** - ``GradOperation`` inside the traced function triggers the IR-level reverse-mode transform
   (``graph.autodiff``): one explicit VJP node per forward node plus explicit gradient accumulation nodes, so
   backward collectives are real graph nodes that passes can reorder.
3. **passes**  - dead-code elimination, common-subexpression elimination, then the parallel passes
   (``parallel.step_parallel``) when a parallel mode is set; ``save_graphs`` dumps the IR after each pass.
4. **execute** - ``graph.executor.GraphExecutor`` replays the node list; with ``enable_cuda_graph`` the replay is
   captured once into a CUDA graph.

Parity: mindspore/python/mindspore/common/api.py:798-983 (jit), :516-758 (_MindsporeFunctionExecutor),
:1668-1912 (_CellGraphExecutor); ccsrc/pipeline/jit/ps/pipeline.cc:1213-1299,1618-1723.
"""
from __future__ import annotations

import functools
import os

import torch
import torch.fx as fx
from torch.overrides import TorchFunctionMode

from .. import context
from ..common.parameter import Parameter
from ..common.tensor import Tensor
from ..ops import primitive as _prim_mod
from . import tracer as _trace_state
from .autodiff import build_backward
from .executor import GraphExecutor
from .ir import FuncGraph, dump_graph
from .passes import run_default_passes

_SKIP_FUNCS = set()


def _is_tensor(x):
    return isinstance(x, torch.Tensor)


_SYMBOLIC_GRADS = False


class symbolic_gradients:
    """Within this context a trace builds its reverse-mode nodes without computing concrete gradients: the values
    that ``GradOperation`` hands back during the trace are zero placeholders.  For callers that only want the graph
    and run it afterwards (the arena micro-batch, whose first real execution is the compiled graph itself)."""

    def __enter__(self):
        global _SYMBOLIC_GRADS
        self._old, _SYMBOLIC_GRADS = _SYMBOLIC_GRADS, True

    def __exit__(self, *exc):
        global _SYMBOLIC_GRADS
        _SYMBOLIC_GRADS = self._old


class _Recorder(TorchFunctionMode):
    """Records executed torch-level calls into an fx.Graph while really executing them."""

    def __init__(self, fg, parent=None):
        super().__init__()
        self.fg = fg
        self.parent = parent        # enclosing recorder when this one traces a branch of a Switch
        self.captured = []          # values of the enclosing trace this sub-graph reads: [(tensor, placeholder)]
        self.depth = 0
        self.node_of = {}   # id(tensor) -> fx.Node
        self.alias = {}     # (data_ptr, shape, stride, dtype) -> fx.Node, for untracked aliases (as_subclass ...)
        self.keep = []      # keep recorded tensors alive so ids and data pointers stay unique
        self.symbolic_grads = _SYMBOLIC_GRADS   # trace_grad builds the reverse-mode nodes without running a tape

    @staticmethod
    def _akey(t):
        try:
            ptr = t.data_ptr()
        except RuntimeError:
            return None
        if ptr == 0:
            return None
        return (ptr, tuple(t.shape), tuple(t.stride()), t.dtype)

    # ---- value <-> node mapping
    def bind(self, value, node):
        if _is_tensor(value):
            node.meta.setdefault("shape", tuple(value.shape))
            node.meta.setdefault("dtype", value.dtype)
            self.node_of[id(value)] = node
            k = self._akey(value)
            if k is not None:
                self.alias[k] = node
            self.keep.append(value)
        elif isinstance(value, (tuple, list)):
            for i, v in enumerate(value):
                if _is_tensor(v) or isinstance(v, (tuple, list)):
                    import operator
                    self.bind(v, self.fg.graph.call_function(operator.getitem, (node, i)))

    def arg(self, a):
        if _is_tensor(a):
            n = self.node_of.get(id(a))
            if n is not None:
                return n
            k = self._akey(a)
            if isinstance(a, Parameter):
                n = self.fg.param_node(a)
            elif k is not None and k in self.alias:
                n = self.alias[k]
            elif self.parent is not None and self.parent.knows(a):
                # a value computed by the enclosing trace: it becomes an extra input of this sub-graph
                with self.fg.graph.inserting_before(next(iter(self.fg.graph.nodes), None)):
                    n = self.fg.graph.placeholder("cap%d" % len(self.captured))
                n.meta["example"] = (tuple(a.shape), a.dtype)
                self.captured.append((a, n))
            else:
                n = self.fg.const_node(a)
            n.meta.setdefault("shape", tuple(a.shape))
            n.meta.setdefault("dtype", a.dtype)
            self.node_of[id(a)] = n
            if k is not None and k not in self.alias:
                self.alias[k] = n
            self.keep.append(a)
            return n
        if isinstance(a, tuple):
            return tuple(self.arg(x) for x in a)
        if isinstance(a, list):
            return [self.arg(x) for x in a]
        if isinstance(a, dict):
            return {k: self.arg(v) for k, v in a.items()}
        if isinstance(a, slice):
            return slice(self.arg(a.start), self.arg(a.stop), self.arg(a.step))
        return a

    def _remap(self, replaced):
        """Nodes that a rewrite replaced: tensors recorded against them now belong to the replacement."""
        if not replaced:
            return

        def final(n):
            while n in replaced:
                n = replaced[n]
            return n
        for table in (self.node_of, self.alias):
            for k, n in list(table.items()):
                if n in replaced:
                    table[k] = final(n)

    def knows(self, t):
        if id(t) in self.node_of:
            return True
        k = self._akey(t)
        if k is not None and k in self.alias:
            return True
        return self.parent is not None and self.parent.knows(t)

    def record(self, target, args, kwargs, out):
        node = self.fg.graph.call_function(target, self.arg(tuple(args)), self.arg(dict(kwargs or {})))
        self.bind(out, node)
        return node

    # ---- torch function interception
    def __torch_function__(self, func, types, args=(), kwargs=None):
        kwargs = kwargs or {}
        if self.depth > 0:
            return func(*args, **kwargs)
        self.depth += 1
        try:
            out = func(*args, **kwargs)
        finally:
            self.depth -= 1
        name = getattr(func, "__name__", "")
        if name in ("__get__", "__set__") or not _has_tensor(out):
            return out  # attribute reads (shape, dtype ...) and non-tensor results are trace-time constants
        if not _has_tensor(args) and not _has_tensor(kwargs):
            self.bind(out, self.fg.const_node(out) if _is_tensor(out) else None) if _is_tensor(out) else None
            return out
        self.record(func, args, kwargs, out)
        return out

    def primitive_hook(self, prim, args, kwargs):
        if self.depth > 0:
            return NotImplemented
        self.depth += 1
        try:
            out = _prim_mod._wrap_out(prim._execute(*args, **kwargs))
        finally:
            self.depth -= 1
        if _has_tensor(out) or prim._update_parameter or prim.name in ("Send", "Barrier"):
            node = self.record(prim, args, kwargs, out)
            node.meta["primitive"] = prim.name
            from ..parallel import spmd as _spmd
            if _spmd.last_dispatch is not None:
                # the sharded primitive is one node; the communication its SPMD execution performs rides along
                node.meta.update({k: v for k, v in _spmd.last_dispatch.items() if v})
                _spmd.last_dispatch = None
        return out

    def leaf_call(self, fn, args, kwargs):
        """Used by ops.fused: record a fused kernel wrapper as one node."""
        if self.depth > 0:
            return fn(*args, **kwargs)
        self.depth += 1
        try:
            out = fn(*args, **kwargs)
        finally:
            self.depth -= 1
        self.record(fn, args, kwargs, out)
        return out

    # ---- GradOperation under trace
    def trace_grad(self, fn, inputs, weights, sens, want_inputs, input_positions, has_aux, return_value):
        fg = self.fg
        before = list(fg.graph.nodes)
        anchor = before[-1] if before else None
        out = fn(*inputs)  # forward recorded inline (second copy of the forward; CSE merges it with the first)
        # operator chains that have one fused kernel are rewritten now, before reverse mode is built on them; the
        # pass runs over the whole graph so that an earlier copy of the same forward is fused identically
        from .fusion import fuse_patterns
        self._remap(fuse_patterns(fg))
        nodes = list(fg.graph.nodes)
        if anchor is not None and anchor not in nodes:          # the anchor itself was fused away
            anchor = next((n for n in reversed(before) if n in set(nodes)), None)
        fwd_nodes = nodes[nodes.index(anchor) + 1:] if anchor is not None else nodes
        primary = out[0] if has_aux else out
        out_nodes = [self.node_of[id(o)] for o in _flat_tensors(primary) if id(o) in self.node_of]
        in_targets = [x for i, x in enumerate(inputs) if want_inputs and (input_positions is None or i in input_positions)
                      and _is_tensor(x) and x.is_floating_point()]
        w_targets = list(weights or [])
        target_nodes = [self.arg(t) for t in in_targets + w_targets]
        seeds = None
        if sens is not None:
            seeds = [self.arg(s) if _is_tensor(s) else s for s in (_flat_tensors(sens) or [sens])]
        grad_nodes = build_backward(fg, fwd_nodes, out_nodes, target_nodes, seeds,
                                    none_as_zero=not self.symbolic_grads)
        if self.symbolic_grads:
            # the caller wants the graph only (it runs the compiled graph afterwards for the real values): no second
            # forward and no tape, so tracing a large network holds one forward's activations, not three
            gs = [None] * (len(in_targets) + len(w_targets))
        else:
            # concrete values for the rest of the trace: compute with the tape
            with torch.enable_grad():
                work = [x.detach().requires_grad_(True) if _is_tensor(x) and x.is_floating_point() else x
                        for x in inputs]
                self.depth += 1
                try:
                    o2 = fn(*work)
                    p2 = o2[0] if has_aux else o2
                    outs = [o for o in _flat_tensors(p2) if o.requires_grad]
                    tg = [w for w, x in zip(work, inputs) if any(x is t for t in in_targets)] + w_targets
                    sd = [torch.ones_like(o) for o in outs] if sens is None else \
                        [(s if _is_tensor(s) else torch.full_like(o, float(s))).to(o.dtype).expand_as(o)
                         for s, o in zip(_flat_tensors(sens) or [sens] * len(outs), outs)]
                    gs = torch.autograd.grad(outs, tg, sd, allow_unused=True) if outs and tg else [None] * len(tg)
                finally:
                    self.depth -= 1
        vals = []
        for g, t, n in zip(gs, in_targets + w_targets, grad_nodes):
            in_accumulator = g is None and getattr(t, "main_grad", None) is not None and not self.symbolic_grads
            if in_accumulator or (g is None and self.symbolic_grads):
                # no graph value: the operator's backward added this gradient into the parameter's fp32 accumulator
                # (or no concrete gradients are computed at all in this trace)
                g = torch.zeros((), dtype=t.dtype, device=t.device).expand(t.shape)
            v = (torch.zeros_like(t.detach()) if g is None else g).detach().as_subclass(Tensor)
            if in_accumulator:
                v.in_accumulator = True
            self.node_of[id(v)] = n
            self.keep.append(v)
            vals.append(v)
        ig, wg = tuple(vals[:len(in_targets)]), tuple(vals[len(in_targets):])
        return out, ig, wg


def _has_tensor(x):
    if _is_tensor(x):
        return True
    if isinstance(x, (tuple, list)):
        return any(_has_tensor(v) for v in x)
    if isinstance(x, dict):
        return any(_has_tensor(v) for v in x.values())
    return False


def _flat_tensors(x):
    if _is_tensor(x):
        return [x]
    if isinstance(x, (tuple, list)):
        out = []
        for v in x:
            out += _flat_tensors(v)
        return out
    return []


_warned_branches = set()


class _TraceSession:
    def __init__(self, rec):
        self.rec = rec

    def note_host_branch(self, t):
        """``bool(tensor)`` during a trace: if the tensor was computed by the graph (it is not a constant of the
        trace), the Python branch taken now is frozen into the graph.  Said once per call site."""
        rec = self.rec
        if rec.depth > 0:
            return
        n = rec.node_of.get(id(t))
        if n is None or n.op == "get_attr":
            return
        import traceback
        frame = next((f for f in reversed(traceback.extract_stack(limit=8)[:-2])
                      if "mindspore_b200/common/tensor.py" not in f.filename), None)
        key = (frame.filename, frame.lineno) if frame else None
        if key in _warned_branches:
            return
        _warned_branches.add(key)
        from ..utils.log import logger
        logger.warning("graph mode: a Python branch on a tensor value (%s:%s) is decided at trace time and stays "
                       "fixed in the compiled graph; use ops.cond(pred, true_fn, false_fn, ...) or ops.select to "
                       "keep it data dependent", *(key or ("?", "?")))

    def trace_grad(self, *a, **k):
        return self.rec.trace_grad(*a, **k)


def trace_callable(fn, example_inputs, name="graph"):
    """Runs ``fn`` on the example inputs and returns (FuncGraph, example_outputs)."""
    fg = FuncGraph(name)
    rec = _Recorder(fg)
    placeholders = []
    for i, x in enumerate(example_inputs):
        if _is_tensor(x):
            n = fg.graph.placeholder("arg%d" % i)
            n.meta["example"] = (tuple(x.shape), x.dtype)
            rec.bind(x, n)
            placeholders.append(i)
    fg.input_positions = placeholders
    prev_hook, prev_cur = _prim_mod._trace_hook, _trace_state.current()
    _prim_mod._set_trace_hook(rec.primitive_hook)
    _trace_state._set_current(_TraceSession(rec))
    try:
        with rec:
            out = fn(*example_inputs)
    finally:
        _prim_mod._set_trace_hook(prev_hook)
        _trace_state._set_current(prev_cur)
    fg.set_output(rec.arg(out) if _has_tensor(out) else out, out)
    fg.example_outputs = out
    return fg, out


def trace_branch(fn, operands, outer, name):
    """Traces one branch of a ``cond`` into its own FuncGraph while the enclosing trace is suspended.  Returns
    (graph, example outputs, captured outer tensors).  ``graph.operand_positions`` lists which operands are tensor
    inputs; the captured values follow them in the sub-graph's input order."""
    fg = FuncGraph(name)
    rec = _Recorder(fg, parent=outer)
    positions = []
    for i, x in enumerate(operands):
        if _is_tensor(x):
            n = fg.graph.placeholder("arg%d" % i)
            n.meta["example"] = (tuple(x.shape), x.dtype)
            rec.bind(x, n)
            positions.append(i)
    prev_hook, prev_cur = _prim_mod._trace_hook, _trace_state.current()
    _prim_mod._set_trace_hook(rec.primitive_hook)
    _trace_state._set_current(_TraceSession(rec))
    outer.depth += 1               # the enclosing recorder must not record what the branch executes
    try:
        with rec:
            out = fn(*operands)
    finally:
        outer.depth -= 1
        _prim_mod._set_trace_hook(prev_hook)
        _trace_state._set_current(prev_cur)
    fg.set_output(rec.arg(out) if _has_tensor(out) else out, out)
    fg.example_outputs = out
    # placeholders were created as: operand args (in order), captured ones inserted at the front later; the
    # executor feeds inputs in node order, so move the captured placeholders behind the operand placeholders
    fg.operand_positions = positions
    ordered = [n for n in fg.graph.nodes if n.op == "placeholder" and n.name.startswith("arg")]
    caps = [n for _, n in rec.captured]
    last = ordered[-1] if ordered else None
    for c in caps:
        if last is not None:
            last.append(c)
        last = c
    fg.input_positions = list(range(len(ordered) + len(caps)))
    run_default_passes(fg, name, 0, ".")
    return fg, out, [t for t, _ in rec.captured]


def leaf_call(fn, args, kwargs):
    """Entry point for fused ops: inside a trace the whole call becomes one node."""
    cur = _trace_state.current()
    if cur is None:
        return fn(*args, **kwargs)
    return cur.rec.leaf_call(fn, args, kwargs)


def _signature(inputs, kwargs, training):
    sig = []
    for x in inputs:
        if _is_tensor(x):
            sig.append(("T", tuple(x.shape), x.dtype, x.device.type))
        elif isinstance(x, (int, float, bool, str, type(None))):
            sig.append(("C", x))
        else:
            sig.append(("O", id(x)))
    return (tuple(sig), tuple(sorted(kwargs.items())) if kwargs else (), training,
            context.get_auto_parallel_context("parallel_mode"))


class CompiledGraph:
    def __init__(self, fg, first_outputs):
        self.fg = fg
        self.executor = GraphExecutor(fg)
        self.first_outputs = first_outputs
        self.used_first = False

    def __call__(self, *inputs):
        tensors = [inputs[i] for i in self.fg.input_positions]
        return self.executor.run(tensors)

    def memory_report(self):
        """{'arena_bytes': planned peak of intermediate values, 'sum_bytes': without reuse, 'tensors': count}."""
        return dict(self.executor.memory_plan)


def _search_strategies(fn, inputs, kwargs, name, owner):
    """auto_parallel: one trace on full shapes (parallel mode switched off), then the strategy search writes
    ``in_strategy`` onto the primitives that the real trace will dispatch."""
    from ..context import _AutoParallelContext
    from ..parallel import auto_parallel
    store = _AutoParallelContext()._v
    mode = store["parallel_mode"]
    snapshot = _snapshot_state(owner)
    store["parallel_mode"] = context.ParallelMode.STAND_ALONE
    try:
        fg0, _ = trace_callable(lambda *a: fn(*a, **kwargs), inputs, name + "_shapes")
    finally:
        store["parallel_mode"] = mode
        _restore_state(snapshot)
    devices = store["device_num"] // max(1, store["pipeline_stages"])
    chosen = auto_parallel.search(fg0, devices, store.get("search_mode", "sharding_propagation"))
    if owner is not None:
        object.__setattr__(owner, "_searched_strategies", chosen)
    return chosen


def _compile(fn, inputs, kwargs, name, owner=None):
    if context.get_auto_parallel_context("parallel_mode") == context.ParallelMode.AUTO_PARALLEL:
        _search_strategies(fn, inputs, kwargs, name, owner)
    snapshot = _snapshot_state(owner)
    fg, out = trace_callable(lambda *a: fn(*a, **kwargs), inputs, name)
    _restore_state(snapshot)   # tracing really executed one step; roll parameters / optimizer state back
    level = context.get_context("save_graphs")
    path = context.get_context("save_graphs_path")
    if level:
        dump_graph(fg, os.path.join(path, "%s_00_trace.ir" % name))
    run_default_passes(fg, name, level, path)
    mode = context.get_auto_parallel_context("parallel_mode")
    if mode in (context.ParallelMode.SEMI_AUTO_PARALLEL, context.ParallelMode.AUTO_PARALLEL) and owner is not None:
        from ..parallel.step_parallel import annotate_graph
        annotate_graph(fg, owner)
        if level:
            dump_graph(fg, os.path.join(path, "%s_step_parallel_end.ir" % name))
    if level:
        from .abstract import annotate_graph
        annotate_graph(fg, inputs)
        dump_graph(fg, os.path.join(path, "%s_validate.ir" % name))
    cg = CompiledGraph(fg, out)
    from .flops import note_compiled
    note_compiled("train" if (owner is None or getattr(owner, "training", True)) else "predict", fg)
    plan = cg.executor.memory_plan
    if level:
        with open(os.path.join(path, "%s_memory_plan.txt" % name), "w") as f:
            f.write("intermediate tensors %d\nwithout reuse %d bytes\nplanned arena %s bytes\n"
                    % (plan["tensors"], plan["sum_bytes"], plan["arena_bytes"]))
    limit = context.get_context("max_device_memory")
    if plan.get("arena_bytes") and isinstance(limit, str) and limit.upper().endswith("GB"):
        try:
            cap = float(limit[:-2]) * 2 ** 30
            if plan["arena_bytes"] > cap:
                from ..utils.log import logger
                logger.warning("graph %s: the planned activation arena (%.2f GB) exceeds max_device_memory (%s)",
                               name, plan["arena_bytes"] / 2 ** 30, limit)
        except ValueError:
            pass
    return cg


def _snapshot_state(owner):
    if owner is None or not hasattr(owner, "get_parameters"):
        return None
    snap = []
    seen = set()

    def add(cell):
        for p in cell.get_parameters():
            if id(p) not in seen:
                seen.add(id(p))
                snap.append((p, p.detach().as_subclass(torch.Tensor).clone()))
    add(owner)
    opt = getattr(owner, "optimizer", None)
    host = None
    if opt is not None:
        add(opt)
        host = (opt, opt._step_host)
    return snap, host, torch.get_rng_state()


def _restore_state(snapshot):
    if snapshot is None:
        return
    snap, host, rng = snapshot
    with torch.no_grad():
        for p, v in snap:
            if tuple(p.shape) != tuple(v.shape):
                # the trace sliced this parameter to its shard (first use under a layout): restore the shard
                lay = getattr(p, "param_layout", None)
                if lay is None:
                    continue
                from .. import context as _ctx
                from ..parallel.layout import slice_for_rank
                rank = _ctx.get_auto_parallel_context("global_rank")
                per = max(1, _ctx.get_auto_parallel_context("device_num") //
                          _ctx.get_auto_parallel_context("pipeline_stages"))
                v = slice_for_rank(v, lay, rank % per)
            torch.Tensor.copy_(p, v)
    if host is not None:
        host[0]._step_host = host[1]
    torch.set_rng_state(rng)


def compile_cell(cell, inputs, kwargs):
    key = _signature(inputs, kwargs, cell.training)
    cg = cell._compiled.get(key)
    if cg is None:
        declared = getattr(cell, "_dynamic_inputs", None)
        if declared:
            from .abstract import check_signature
            check_signature(declared, inputs, "set_inputs")
        cg = _compile(cell._run_construct_traced, inputs, kwargs, type(cell).__name__, owner=cell)
        cell._compiled[key] = cg
    return cg


def compile_and_run_cell(cell, inputs, kwargs):
    if not hasattr(cell, "_run_construct_traced"):
        cell._run_construct_traced = lambda *a, **k: cell._run_construct(a, k)
    if getattr(cell, "_use_graph", None) is False:
        return cell._run_construct(inputs, kwargs)
    cg = compile_cell(cell, inputs, kwargs)
    return cg(*inputs)


def trace_cell(cell, inputs):
    from ..nn.cell import Cell
    Cell._graph_depth += 1
    try:
        fg, _ = trace_callable(lambda *a: cell._run_construct(a, {}), inputs, type(cell).__name__)
    finally:
        Cell._graph_depth -= 1
    return fg


def load_graph_text(path):
    with open(path) as f:
        text = f.read()
    fg = FuncGraph(os.path.basename(path))
    fg.text = text
    return fg


def jit(fn=None, mode="PSJit", input_signature=None, hash_args=None, jit_config=None, compile_once=False):
    """Decorator: compile ``fn`` once per input signature and replay the graph on later calls."""
    if mode not in ("PSJit", "PIJit"):
        raise ValueError("For 'jit', 'mode' must be 'PSJit' or 'PIJit', but got %r" % (mode,))

    def deco(f):
        cache = {}

        @functools.wraps(f)
        def wrapper(*args, **kwargs):
            from ..nn.cell import Cell
            if _trace_state.is_tracing() or os.environ.get("MS_JIT") == "0":
                return f(*args, **kwargs)
            if input_signature is not None:
                from .abstract import check_signature
                check_signature(input_signature, args[1:] if args and isinstance(args[0], Cell) else args)
            key = _signature(args, kwargs, None)
            cg = cache.get(key)
            Cell._graph_depth += 1
            try:
                if cg is None:
                    owner = args[0] if args and isinstance(args[0], Cell) else None
                    from .ast_transform import convert_function
                    cg = _compile(convert_function(f), args, kwargs, getattr(f, "__name__", "jit_fn"), owner=owner)
                    cache[key] = cg
                return cg(*args)
            finally:
                Cell._graph_depth -= 1

        def infer_outputs(*abstract_args, **kw):
            """Abstract outputs for abstract / placeholder inputs (the input signature when none are given)."""
            from .abstract import infer
            if not abstract_args and input_signature is not None:
                abstract_args = tuple(input_signature) if isinstance(input_signature, (tuple, list)) else (
                    input_signature,)
            return infer(f, *abstract_args, **kw)

        wrapper.__jit_cache__ = cache
        wrapper.infer = infer_outputs
        return wrapper

    return deco(fn) if fn is not None else deco


ms_function = jit
