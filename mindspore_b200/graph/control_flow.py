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
