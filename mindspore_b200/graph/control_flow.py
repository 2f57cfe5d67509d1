"""Structured control flow for graph mode.

The graph front end executes ``construct`` once and records what ran, so a Python ``if`` on a tensor value is
decided at trace time and frozen into the graph.  ``cond(pred, true_fn, false_fn, *operands)`` is the traceable
form: both branches are traced into sub-graphs (values they take from the enclosing trace are lifted to extra
inputs automatically, parameters are shared), and ONE ``Switch`` node is recorded whose execution reads the
predicate and runs the chosen sub-graph - the role of the reference's Switch / SwitchLayer after the parser has
turned ``if`` statements into sub-graphs (ccsrc/pipeline/jit/ps/parse/parse.cc: ParseIf, core/ops/switch.cc).
Reverse mode works through the node: its vjp is the autograd tape of whichever branch ran.

Eagerly ``cond`` is just the Python conditional.
"""
from __future__ import annotations

import torch

from . import tracer as _trace_state


class Switch:
    """Target of a Switch node: holds the two traced branches."""

    def __init__(self, true_graph, false_graph, n_operands, n_true_caps, n_false_caps):
        from .executor import GraphExecutor
        self.graphs = (true_graph, false_graph)
        self.executors = (GraphExecutor(true_graph), GraphExecutor(false_graph))
        self.n_operands, self.n_true_caps, self.n_false_caps = n_operands, n_true_caps, n_false_caps
        self.__name__ = "Switch"
        self.last_taken = None

    def pure(self):
        from .passes import is_impure
        return not any(is_impure(n) for g in self.graphs for n in g.graph.nodes)

    def _inputs(self, branch, vals):
        ops = list(vals[:self.n_operands])
        t_caps = list(vals[self.n_operands:self.n_operands + self.n_true_caps])
        f_caps = list(vals[self.n_operands + self.n_true_caps:])
        fg = self.graphs[branch]
        caps = t_caps if branch == 0 else f_caps
        operand_inputs = [ops[i] for i in fg.operand_positions]
        return operand_inputs + caps

    def __call__(self, pred, *vals):
        capturing = pred.is_cuda and torch.cuda.is_current_stream_capturing()
        if capturing:
            if not self.pure():
                raise RuntimeError("a Switch whose branches update state can not be captured into a CUDA graph: "
                                   "the predicate would have to be read on the host")
            t = self.executors[0].run(self._inputs(0, vals))
            f = self.executors[1].run(self._inputs(1, vals))
            return _select(pred, t, f)
        taken = 0 if bool(pred) else 1
        self.last_taken = taken
        return self.executors[taken].run(self._inputs(taken, vals))


def _select(pred, t, f):
    if isinstance(t, torch.Tensor):
        return torch.where(pred, t, f)
    if isinstance(t, (tuple, list)):
        return type(t)(_select(pred, a, b) for a, b in zip(t, f))
    return t


def _structure(x):
    if isinstance(x, torch.Tensor):
        return ("T", tuple(x.shape), x.dtype)
    if isinstance(x, (tuple, list)):
        return (type(x).__name__,) + tuple(_structure(v) for v in x)
    return ("C", x)


def cond(pred, true_fn, false_fn, *operands):
    """``true_fn(*operands) if pred else false_fn(*operands)`` with ``pred`` a 0-d (or one-element) tensor.  Both
    functions must return the same structure of tensors (shapes and dtypes)."""
    session = _trace_state.current()
    if session is None:
        return true_fn(*operands) if bool(pred) else false_fn(*operands)
    from . import jit as _jit
    outer = session.rec
    if outer.depth > 0:           # inside a leaf that is recorded as one node: evaluate plainly
        return true_fn(*operands) if bool(pred) else false_fn(*operands)
    tg, t_out, t_caps = _jit.trace_branch(true_fn, operands, outer, "cond_true")
    fg, f_out, f_caps = _jit.trace_branch(false_fn, operands, outer, "cond_false")
    if _structure(t_out) != _structure(f_out):
        raise TypeError("For 'cond', both branches must return the same structure, got %s and %s"
                        % (_structure(t_out), _structure(f_out)))
    sw = Switch(tg, fg, len(operands), len(t_caps), len(f_caps))
    # (read through the plain tensor type: this Python branch only picks the example values of the trace)
    out = t_out if pred.detach().as_subclass(torch.Tensor).item() else f_out
    args = (pred,) + tuple(operands) + tuple(t_caps) + tuple(f_caps)
    node = outer.record(sw, args, {}, out)
    node.meta["primitive"] = "Switch"
    return out



# ---------------------------------------------------------------------------------------------------- loops
class While:
    """Target of a While node: the traced condition and body of ``while_loop``.  Each run evaluates the condition
    sub-graph on the current state, reads it on the host and runs the body sub-graph until it is false (the
    reference lowers ``while`` to a recursive Switch between the body-and-call-again graph and the exit graph:
    ccsrc/pipeline/jit/ps/parse/parse.cc ParseWhile; ops WhileLoop in ops/operations/_scalar_ops.py).  Reverse mode
    goes through the iterations that ran, like ``Switch``."""

    def __init__(self, cond_graph, body_graph, n_state, n_cond_caps, n_body_caps, max_iterations=None):
        from .executor import GraphExecutor
        self.graphs = (cond_graph, body_graph)
        self.executors = (GraphExecutor(cond_graph), GraphExecutor(body_graph))
        self.n_state, self.n_cond_caps, self.n_body_caps = n_state, n_cond_caps, n_body_caps
        self.max_iterations = max_iterations
        self.__name__ = "While"
        self.last_iterations = None

    def __call__(self, *vals):
        state = list(vals[:self.n_state])
        c_caps = list(vals[self.n_state:self.n_state + self.n_cond_caps])
        b_caps = list(vals[self.n_state + self.n_cond_caps:])
        cg, bg = self.graphs
        if any(isinstance(v, torch.Tensor) and v.is_cuda for v in state) and torch.cuda.is_current_stream_capturing():
            raise RuntimeError("a While node can not be captured into a CUDA graph: its trip count is read on the host")
        n = 0
        while True:
            pred = self.executors[0].run([state[i] for i in cg.operand_positions] + c_caps)
            if not bool(pred.detach().as_subclass(torch.Tensor).reshape(-1)[0].item()):
                break
            out = self.executors[1].run([state[i] for i in bg.operand_positions] + b_caps)
            state = list(out) if isinstance(out, (tuple, list)) else [out]
            n += 1
            if self.max_iterations is not None and n >= self.max_iterations:
                break
        self.last_iterations = n
        return tuple(state)


def while_loop(cond_fn, body_fn, init_val, max_iterations=None):
    """``state = init_val; while cond_fn(*state): state = body_fn(*state); return state`` with ``state`` a tuple of
    tensors (a single tensor is taken as a one-element state and returned as a tensor).  In graph mode the condition
    and the body become sub-graphs behind ONE While node whose trip count is decided at every run."""
    single = isinstance(init_val, torch.Tensor)
    state = (init_val,) if single else tuple(init_val)

    def plain():
        cur, n = state, 0
        while bool(cond_fn(*cur)):
            nxt = body_fn(*cur)
            cur = (nxt,) if isinstance(nxt, torch.Tensor) else tuple(nxt)
            n += 1
            if max_iterations is not None and n >= max_iterations:
                break
        return cur

    session = _trace_state.current()
    if session is None or session.rec.depth > 0 or not all(isinstance(v, torch.Tensor) for v in state):
        out = plain()
        return out[0] if single else out
    from . import jit as _jit
    outer = session.rec
    cg, c_out, c_caps = _jit.trace_branch(cond_fn, state, outer, "while_cond")
    bg, b_out, b_caps = _jit.trace_branch(body_fn, state, outer, "while_body")
    b_tuple = (b_out,) if isinstance(b_out, torch.Tensor) else tuple(b_out)
    if _structure(tuple(b_tuple)) != _structure(tuple(state)):
        raise TypeError("For 'while_loop', the body must return the structure of the loop state, got %s for %s"
                        % (_structure(tuple(b_tuple)), _structure(tuple(state))))
    if not isinstance(c_out, torch.Tensor) or c_out.numel() != 1:
        raise TypeError("For 'while_loop', the condition must return a one-element tensor")
    outer.depth += 1                                   # the example run of the trace itself is not recorded
    try:
        out = plain()
    finally:
        outer.depth -= 1
    node_target = While(cg, bg, len(state), len(c_caps), len(b_caps), max_iterations)
    args = tuple(state) + tuple(c_caps) + tuple(b_caps)
    node = outer.record(node_target, args, {}, tuple(out))
    node.meta["primitive"] = "While"
    return out[0] if single else tuple(out)


def fori_loop(lower, upper, body_fn, init_val, unroll=True):
    """``val = init_val; for i in range(lower, upper): val = body_fn(i, val)``.  Integer bounds unroll into the
    trace; tensor bounds run as a ``while_loop`` over (i, val)."""
    if isinstance(lower, int) and isinstance(upper, int):
        val = init_val
        for i in range(lower, upper):
            val = body_fn(i, val)
        return val
    lo = torch.as_tensor(lower)
    hi = torch.as_tensor(upper)
    single = isinstance(init_val, torch.Tensor)
    vals = (init_val,) if single else tuple(init_val)

    def c(i, *v):
        return i < hi

    def b(i, *v):
        out = body_fn(i, v[0] if single else tuple(v))
        out = (out,) if isinstance(out, torch.Tensor) else tuple(out)
        return (i + 1,) + out
    res = while_loop(c, b, (lo.clone(),) + vals)
    return res[1] if single else tuple(res[1:])


def scan(f, init, xs, length=None):
    """``carry, ys = init, []; for x in xs: carry, y = f(carry, x); ys.append(y)``; returns (carry, stacked ys).
    The steps unroll into the trace (the leading dimension is static)."""
    n = length if xs is None else (len(xs) if not isinstance(xs, torch.Tensor) else xs.shape[0])
    carry, ys = init, []
    for k in range(n):
        carry, y = f(carry, None if xs is None else xs[k])
        ys.append(y)
    if ys and isinstance(ys[0], torch.Tensor):
        return carry, torch.stack(ys)
    return carry, ys
