"""Source-level front end for data-dependent ``if`` statements in graph mode.

The tracer runs ``construct`` once and records what ran, so a plain Python ``if`` on a tensor value would be decided
at trace time.  This module rewrites the function's syntax tree before it is traced: every ``if`` / ``elif`` / ``else``
whose branches only bind local names becomes two local functions and one call of ``run_if``,

    if cond_expr:                       def __ms_true_0(a=<a, if bound>):  # names bound before are passed in
        a = f(a)                            a = f(a); b = g(a)
        b = g(a)              ==>           return (a, b)
    else:                               def __ms_false_0(a=<a, if bound>):
        b = h(a)                            b = h(a)
                                            return (a, b)
                                        (a, b) = __ms_run_if(cond_expr, __ms_true_0, __ms_false_0)

and ``run_if`` picks the plain Python branch for Python values (shape tests, flags, ``self.training``) and
``graph.control_flow.cond`` - both branches traced into sub-graphs under one ``Switch`` node - when the condition is a
tensor computed by the graph being traced.  This is the role of the reference's parser for ``if`` statements
(ccsrc/pipeline/jit/ps/parse/parse.cc: ParseIf builds the true / false / after blocks and a Switch).

Left as they are (and therefore decided at trace time, with the tracer's warning): branches that ``return``,
``break``, ``continue``, ``raise``, ``yield``, ``del`` or assign to attributes / subscripts, and functions whose source
is not available.

``while`` loops whose bodies only rebind local names that exist before the loop are rewritten the same way into a
condition function, a body function over the loop-carried names and one call of ``run_while``, which records a single
While node when the condition is a tensor of the graph (ParseWhile in the reference) and runs the plain Python loop
otherwise."""
from __future__ import annotations

import ast
import inspect
import textwrap
import types

import torch

_CACHE = {}
_UNDEFINED = type("Undefined", (), {"__repr__": lambda self: "<undefined in this branch>"})()


def run_if(test, true_fn, false_fn):
    """Runtime of a rewritten ``if``: see the module text."""
    from . import tracer as _trace_state
    if isinstance(test, torch.Tensor) and _trace_state.is_tracing():
        session = _trace_state.current()
        rec = getattr(session, "rec", None)
        if rec is not None and rec.depth == 0 and rec.knows(test) and test.numel() == 1:
            from .control_flow import cond
            return cond(test.reshape(()) if test.dim() else test, true_fn, false_fn)
    return true_fn() if test else false_fn()


def run_while(cond_fn, body_fn, state):
    """Runtime of a rewritten ``while``: a condition that is a tensor computed by the graph being traced makes the
    loop one While node (``graph.control_flow.while_loop``); anything else runs as the plain Python loop."""
    from . import tracer as _trace_state
    if _trace_state.is_tracing() and all(isinstance(v, torch.Tensor) for v in state):
        session = _trace_state.current()
        rec = getattr(session, "rec", None)
        if rec is not None and rec.depth == 0:
            rec.depth += 1                              # probe the condition without recording it
            try:
                first = cond_fn(*state)
            finally:
                rec.depth -= 1
            if isinstance(first, torch.Tensor) and first.numel() == 1 and \
                    any(rec.knows(v) for v in state):
                from .control_flow import while_loop
                return tuple(while_loop(cond_fn, body_fn, tuple(state)))
    while cond_fn(*state):
        state = body_fn(*state)
    return tuple(state)


def value_of(thunk):
    """Current value of a local name that may not be bound yet on this path (``thunk`` = ``lambda: name``)."""
    try:
        return thunk()
    except NameError:                      # UnboundLocalError and the free-variable form are both NameErrors
        return _UNDEFINED


class _Unsupported(Exception):
    pass


_BLOCKERS = (ast.Return, ast.Break, ast.Continue, ast.Raise, ast.Delete, ast.Global, ast.Nonlocal, ast.Yield,
             ast.YieldFrom, ast.Await, ast.Try, ast.With, ast.ClassDef, ast.Import, ast.ImportFrom)


def _stored_names(stmts):
    """Local names bound by the statements, in order of first binding; raises _Unsupported for constructs a branch
    function cannot hold."""
    names = []

    def target(t):
        if isinstance(t, ast.Name):
            if t.id not in names:
                names.append(t.id)
        elif isinstance(t, (ast.Tuple, ast.List)):
            for e in t.elts:
                target(e)
        elif isinstance(t, ast.Starred):
            target(t.value)
        else:
            raise _Unsupported("assignment to %s" % type(t).__name__)

    def visit(node):
        if isinstance(node, _BLOCKERS):
            raise _Unsupported(type(node).__name__)
        if isinstance(node, (ast.FunctionDef, ast.AsyncFunctionDef)):
            if node.name not in names and not node.name.startswith("__ms_"):   # not the helpers of an inner if
                names.append(node.name)
            return                                           # its body has its own scope
        if isinstance(node, (ast.Lambda, ast.ListComp, ast.SetComp, ast.DictComp, ast.GeneratorExp)):
            return
        if isinstance(node, ast.Assign):
            for t in node.targets:
                target(t)
        elif isinstance(node, (ast.AugAssign, ast.AnnAssign)):
            target(node.target)
        elif isinstance(node, ast.NamedExpr):
            target(node.target)
        elif isinstance(node, (ast.For, ast.AsyncFor)):
            target(node.target)
        for child in ast.iter_child_nodes(node):
            visit(child)

    for s in stmts:
        visit(s)
    return names


def _all_stores(node):
    """Every local name bound anywhere under ``node`` (nested function bodies excluded), for the bound-so-far set."""
    out = set()
    stack = [node]
    while stack:
        n = stack.pop()
        if isinstance(n, (ast.FunctionDef, ast.AsyncFunctionDef)):
            out.add(n.name)
            if n is not node:
                continue
        if isinstance(n, (ast.Lambda, ast.ListComp, ast.SetComp, ast.DictComp, ast.GeneratorExp)):
            continue
        if isinstance(n, ast.Name) and isinstance(n.ctx, ast.Store):
            out.add(n.id)
        stack.extend(ast.iter_child_nodes(n))
    return out


class _IfRewriter:
    """Walks statement lists in order, carrying the set of names that are bound when a statement is reached (names
    bound on some earlier path count; names bound only in a sibling branch do not)."""

    def __init__(self, func):
        self.counter = 0
        self.changed = False
        self.func = func
        bound = set(a.arg for a in func.args.args + func.args.posonlyargs + func.args.kwonlyargs)
        if func.args.vararg:
            bound.add(func.args.vararg.arg)
        if func.args.kwarg:
            bound.add(func.args.kwarg.arg)
        func.body = self.block(func.body, bound)

    def block(self, stmts, bound):
        out = []
        bound = set(bound)
        for st in stmts:
            if isinstance(st, ast.If):
                out.extend(self.convert_if(st, bound))
            elif isinstance(st, ast.While) and not st.orelse and self.convertible_while(st, bound):
                out.extend(self.convert_while(st, bound))
            else:
                for field in ("body", "orelse", "finalbody"):
                    sub = getattr(st, field, None)
                    if isinstance(sub, list) and sub and isinstance(sub[0], ast.stmt) and \
                            not isinstance(st, (ast.FunctionDef, ast.AsyncFunctionDef, ast.ClassDef)):
                        inner = set(bound)
                        if isinstance(st, (ast.For, ast.AsyncFor)):
                            inner |= _all_stores(st.target)
                        if isinstance(st, (ast.While, ast.For, ast.AsyncFor)):
                            inner |= _all_stores(st)          # a later iteration sees what an earlier one bound
                        setattr(st, field, self.block(sub, inner))
                for h in getattr(st, "handlers", []) or []:
                    h.body = self.block(h.body, set(bound) | ({h.name} if h.name else set()))
                out.append(st)
            bound |= _all_stores(st)
        return out

    def convertible_while(self, node, bound):
        try:
            names = _stored_names(node.body)
        except _Unsupported:
            return False
        # every loop-carried name must be bound before the loop (it is passed in as state)
        return bool(names) and all(n in bound for n in names)

    def convert_while(self, node, bound):
        names = _stored_names(node.body)
        inner = set(bound) | set(names)
        node.body = self.block(node.body, inner)
        k = self.counter
        self.counter += 1
        self.changed = True

        def fn(name, body):
            args = ast.arguments(posonlyargs=[], args=[ast.arg(arg=n) for n in names], vararg=None, kwonlyargs=[],
                                 kw_defaults=[], kwarg=None, defaults=[])
            return ast.FunctionDef(name=name, args=args, body=body, decorator_list=[], returns=None,
                                   type_comment=None, type_params=[])

        state = ast.Tuple(elts=[ast.Name(id=n, ctx=ast.Load()) for n in names], ctx=ast.Load())
        c_name, b_name = "__ms_wcond_%d" % k, "__ms_wbody_%d" % k
        cond_def = fn(c_name, [ast.Return(value=node.test)])
        body_def = fn(b_name, list(node.body) + [ast.Return(value=state)])
        call = ast.Call(func=ast.Name(id="__ms_run_while", ctx=ast.Load()),
                        args=[ast.Name(id=c_name, ctx=ast.Load()), ast.Name(id=b_name, ctx=ast.Load()), state],
                        keywords=[])
        assign = ast.Assign(targets=[ast.Tuple(elts=[ast.Name(id=n, ctx=ast.Store()) for n in names],
                                               ctx=ast.Store())], value=call)
        out = [cond_def, body_def, assign]
        for n in out:
            ast.copy_location(n, node)
        return out

    def convert_if(self, node, bound):
        node.body = self.block(node.body, bound)              # inner ifs first, each branch with its own view
        node.orelse = self.block(node.orelse, bound)
        try:
            names = _stored_names(node.body + node.orelse)
        except _Unsupported:
            return [node]
        k = self.counter
        self.counter += 1
        self.changed = True
        passed = [n for n in names if n in bound]

        def branch(name, stmts):
            body = list(stmts) or [ast.Pass()]
            bound_here = set(_stored_names(stmts)) | set(passed)
            ret = ast.Return(value=ast.Tuple(
                elts=[ast.Name(id=n, ctx=ast.Load()) if n in bound_here else ast.Name(id="__ms_undefined", ctx=ast.Load())
                      for n in names], ctx=ast.Load()))
            args = ast.arguments(posonlyargs=[], args=[ast.arg(arg=n) for n in passed], vararg=None, kwonlyargs=[],
                                 kw_defaults=[], kwarg=None,
                                 defaults=[ast.Call(func=ast.Name(id="__ms_value_of", ctx=ast.Load()), args=[
                                     ast.Lambda(args=ast.arguments(posonlyargs=[], args=[], vararg=None, kwonlyargs=[],
                                                                   kw_defaults=[], kwarg=None, defaults=[]),
                                                body=ast.Name(id=n, ctx=ast.Load()))], keywords=[]) for n in passed])
            return ast.FunctionDef(name=name, args=args, body=body + [ret], decorator_list=[], returns=None,
                                   type_comment=None, type_params=[])

        t_name, f_name = "__ms_true_%d" % k, "__ms_false_%d" % k
        call = ast.Call(func=ast.Name(id="__ms_run_if", ctx=ast.Load()),
                        args=[node.test, ast.Name(id=t_name, ctx=ast.Load()), ast.Name(id=f_name, ctx=ast.Load())],
                        keywords=[])
        if names:
            assign = ast.Assign(targets=[ast.Tuple(elts=[ast.Name(id=n, ctx=ast.Store()) for n in names],
                                                   ctx=ast.Store())], value=call)
        else:
            assign = ast.Expr(value=call)
        out = [branch(t_name, node.body), branch(f_name, node.orelse), assign]
        for n in out:
            ast.copy_location(n, node)
        return out


def convert_function(fn):
    """The function with its convertible ``if`` statements rewritten, or ``fn`` itself when nothing applies."""
    key = getattr(fn, "__code__", None)
    if key is None:
        return fn
    hit = _CACHE.get(key)
    if hit is not None:
        return hit if hit is not False else fn
    new = _convert(fn)
    _CACHE[key] = new if new is not None else False
    return new if new is not None else fn


def _convert(fn):
    try:
        src = textwrap.dedent(inspect.getsource(fn))
        tree = ast.parse(src)
    except (OSError, TypeError, SyntaxError, IndentationError):
        return None
    funcs = [n for n in tree.body if isinstance(n, (ast.FunctionDef,))]
    if len(funcs) != 1 or not any(isinstance(n, (ast.If, ast.While)) for n in ast.walk(funcs[0])):
        return None
    func = funcs[0]
    if any(isinstance(n, ast.Nonlocal) for n in ast.walk(func)):
        return None
    func.decorator_list = []
    rewriter = _IfRewriter(func)
    if not rewriter.changed:
        return None
    # The rewritten function is rebuilt inside a factory whose parameters are the original's free variables
    # (``__class__`` among them, which is what zero-argument ``super()`` reads).
    free = list(fn.__code__.co_freevars)
    factory = ast.FunctionDef(
        name="__ms_factory",
        args=ast.arguments(posonlyargs=[], args=[ast.arg(arg=v) for v in free], vararg=None, kwonlyargs=[],
                           kw_defaults=[], kwarg=None, defaults=[]),
        body=[func, ast.Return(value=ast.Name(id=func.name, ctx=ast.Load()))], decorator_list=[], returns=None,
        type_comment=None, type_params=[])
    module = ast.Module(body=[factory], type_ignores=[])
    ast.fix_missing_locations(module)
    try:
        code = compile(module, filename=inspect.getsourcefile(fn) or "<converted>", mode="exec")
    except (SyntaxError, ValueError, TypeError):
        return None
    glb = fn.__globals__                                      # the function keeps its module's live globals
    glb.setdefault("__ms_run_if", run_if)
    glb.setdefault("__ms_undefined", _UNDEFINED)
    glb.setdefault("__ms_value_of", value_of)
    glb.setdefault("__ms_run_while", run_while)
    ns = {}
    try:
        exec(code, glb, ns)                                   # noqa: S102  (our own rewritten source of fn)
        cells = [c.cell_contents for c in (fn.__closure__ or ())]
        new = ns["__ms_factory"](*cells)
    except Exception:  # noqa: BLE001  (an empty cell, a name clash ...: keep the original)
        return None
    new.__defaults__ = fn.__defaults__
    new.__kwdefaults__ = fn.__kwdefaults__
    new.__dict__.update(getattr(fn, "__dict__", {}))
    new.__ms_converted_from__ = fn
    new.__qualname__ = getattr(fn, "__qualname__", fn.__name__)
    return new


def converted_construct(cell):
    """``cell.construct`` bound to the rewritten function of its class (or the original bound method)."""
    fn = type(cell).construct
    new = convert_function(fn)
    if new is fn:
        return cell.construct
    return types.MethodType(new, cell)
