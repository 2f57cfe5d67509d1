"""Composite operators: ``GradOperation``, ``HyperMap``, ``Map``, ``MultitypeFuncGraph`` and the
functional autodiff API (``grad``, ``value_and_grad``, ``vjp``, ``jvp``, ``jacfwd``, ``jacrev``).

In PyNative mode gradients come from torch's tape; while a graph is being traced, ``GradOperation``
asks the tracer to differentiate the traced forward graph with the IR-level reverse-mode transform
(``graph.autodiff``), which is what lets communication primitives differentiate into their dual
collectives.

Parity: mindspore/python/mindspore/ops/composite/base.py:107 (GradOperation), :694
(MultitypeFuncGraph), :807 (HyperMap), :879 (Map); ops/function/grad/grad_func.py:93,233,659,874,
1073,1244.
"""
from __future__ import annotations

import torch

from ..common.parameter import Parameter
from ..common.tensor import Tensor, as_tensor


def _is_diff_tensor(x):
    return isinstance(x, torch.Tensor) and (x.is_floating_point() or x.is_complex())


def _flatten_outputs(out):
    if isinstance(out, torch.Tensor):
        return [out]
    if isinstance(out, (tuple, list)):
        res = []
        for o in out:
            res.extend(_flatten_outputs(o))
        return res
    return []


def _zeros_for(t):
    return torch.zeros_like(t.detach()).as_subclass(Tensor)


def _run_grad(fn, inputs, weights, sens, want_inputs, input_positions=None, has_aux=False, return_value=False):
    """Shared eager implementation: returns (value, input_grads, weight_grads)."""
    from ..graph import tracer as _tracer
    if _tracer.is_tracing():
        return _tracer.current().trace_grad(fn, inputs, weights, sens, want_inputs, input_positions, has_aux,
                                            return_value)
    work = []
    for i, x in enumerate(inputs):
        need = want_inputs and (input_positions is None or i in input_positions) and _is_diff_tensor(x)
        if need:
            work.append(x.detach().as_subclass(type(x) if isinstance(x, Tensor) else Tensor).requires_grad_(True))
        else:
            work.append(x)
    with torch.enable_grad():
        out = fn(*work)
    diff_out = out
    if has_aux:
        diff_out = out[0]
    outs = [o for o in _flatten_outputs(diff_out) if o.requires_grad]
    in_targets = [w for i, w in enumerate(work) if want_inputs and (input_positions is None or i in input_positions)
                  and _is_diff_tensor(w)]
    w_targets = [w for w in (weights or []) if w.requires_grad]
    targets = in_targets + w_targets
    grads = []
    if outs and targets:
        if sens is None:
            seeds = [torch.ones_like(o) for o in outs]
        else:
            seeds = [s if isinstance(s, torch.Tensor) else torch.full_like(o, float(s))
                     for s, o in zip(_flatten_outputs(sens) if not isinstance(sens, (int, float)) else [sens] * len(outs),
                                     outs)]
            seeds = [s.to(o.dtype).expand_as(o) if s.shape != o.shape else s.to(o.dtype) for s, o in zip(seeds, outs)]
        grads = list(torch.autograd.grad(outs, targets, seeds, allow_unused=True))
    else:
        grads = [None] * len(targets)
    grads = [(_zeros_for(t) if g is None else g.as_subclass(Tensor)) for g, t in zip(grads, targets)]
    in_grads = tuple(grads[:len(in_targets)])
    w_grads = []
    it = iter(grads[len(in_targets):])
    for w in (weights or []):
        w_grads.append(next(it) if w.requires_grad else _zeros_for(w))
    return out, in_grads, tuple(w_grads)


class GradOperation:
    def __init__(self, get_all=False, get_by_list=False, sens_param=False):
        for n, v in (("get_all", get_all), ("get_by_list", get_by_list), ("sens_param", sens_param)):
            if not isinstance(v, bool):
                raise TypeError("For 'GradOperation', the '%s' should be bool, but got %s" % (n, type(v).__name__))
        self.get_all, self.get_by_list, self.sens_param = get_all, get_by_list, sens_param

    def __call__(self, fn, weights=None):
        if self.get_by_list and weights is None:
            raise ValueError("GradOperation(get_by_list=True) needs the weights argument")
        wlist = list(weights) if weights is not None else None
        if isinstance(weights, Parameter):
            wlist = [weights]

        def grad_fn(*args):
            if self.sens_param:
                inputs, sens = args[:-1], args[-1]
            else:
                inputs, sens = args, None
            want_inputs = self.get_all or not self.get_by_list
            positions = None if self.get_all else ({0} if not self.get_by_list else set())
            _, ig, wg = _run_grad(fn, inputs, wlist if self.get_by_list else None, sens,
                                  want_inputs and (self.get_all or not self.get_by_list), positions)
            if self.get_by_list and self.get_all:
                return ig, wg
            if self.get_by_list:
                return wg if not isinstance(weights, Parameter) else wg[0]
            if self.get_all:
                return ig
            return ig[0] if ig else None

        return grad_fn


def _norm_position(grad_position, n):
    if grad_position is None:
        return set()
    if isinstance(grad_position, int):
        return {grad_position}
    return set(grad_position)


def grad(fn, grad_position=0, weights=None, has_aux=False, return_ids=False):
    def wrapped(*args):
        pos = _norm_position(grad_position, len(args))
        wl = [weights] if isinstance(weights, Parameter) else (list(weights) if weights is not None else None)
        out, ig, wg = _run_grad(fn, args, wl, None, bool(pos), pos, has_aux)
        res = _pack(ig, wg, grad_position, weights)
        if has_aux:
            return res, tuple(out[1:]) if len(out) > 2 else out[1]
        return res

    return wrapped


def _pack(ig, wg, grad_position, weights):
    parts = []
    if grad_position is not None:
        parts.append(ig[0] if isinstance(grad_position, int) else tuple(ig))
    if weights is not None:
        parts.append(wg[0] if isinstance(weights, Parameter) else tuple(wg))
    return parts[0] if len(parts) == 1 else tuple(parts)


def value_and_grad(fn, grad_position=0, weights=None, has_aux=False, return_ids=False):
    def wrapped(*args):
        pos = _norm_position(grad_position, len(args))
        wl = [weights] if isinstance(weights, Parameter) else (list(weights) if weights is not None else None)
        out, ig, wg = _run_grad(fn, args, wl, None, bool(pos), pos, has_aux, return_value=True)
        return out, _pack(ig, wg, grad_position, weights)

    return wrapped


def vjp(fn, *inputs, weights=None, has_aux=False):
    work = [x.detach().requires_grad_(True) if _is_diff_tensor(x) else x for x in inputs]
    with torch.enable_grad():
        out = fn(*work)
    primary = out[0] if has_aux else out

    def vjp_fn(*v):
        outs = _flatten_outputs(primary)
        targets = [w for w in work if _is_diff_tensor(w)]
        g = torch.autograd.grad(outs, targets, list(v), allow_unused=True, retain_graph=True)
        g = tuple(_zeros_for(t) if gi is None else gi.as_subclass(Tensor) for gi, t in zip(g, targets))
        return g if len(g) > 1 else g[0]

    return (primary, vjp_fn, out[1]) if has_aux else (primary, vjp_fn)


def jvp(fn, inputs, v, has_aux=False):
    inputs = inputs if isinstance(inputs, (tuple, list)) else (inputs,)
    v = v if isinstance(v, (tuple, list)) else (v,)
    out, tangent = torch.func.jvp(lambda *a: fn(*a), tuple(x.as_subclass(torch.Tensor) for x in inputs),
                                  tuple(t.as_subclass(torch.Tensor) for t in v))
    return as_tensor(out), as_tensor(tangent)


def jacrev(fn, grad_position=0, has_aux=False):
    def wrapped(*args):
        plain = tuple(a.as_subclass(torch.Tensor) if isinstance(a, torch.Tensor) else a for a in args)
        j = torch.func.jacrev(fn, argnums=grad_position, has_aux=has_aux)(*plain)
        return as_tensor(j) if isinstance(j, torch.Tensor) else j

    return wrapped


def jacfwd(fn, grad_position=0, has_aux=False):
    def wrapped(*args):
        plain = tuple(a.as_subclass(torch.Tensor) if isinstance(a, torch.Tensor) else a for a in args)
        j = torch.func.jacfwd(fn, argnums=grad_position, has_aux=has_aux)(*plain)
        return as_tensor(j) if isinstance(j, torch.Tensor) else j

    return wrapped


def stop_gradient(x):
    return x.detach() if isinstance(x, torch.Tensor) else x


# ------------------------------------------------------------------------------------ HyperMap & co
class MultitypeFuncGraph:
    """Function overloaded on argument kinds ('Tensor', 'Number', 'Tuple', ...)."""

    def __init__(self, name, read_value=False, need_raise=False):
        self.name = name
        self.entries = []

    def register(self, *type_names):
        def deco(fn):
            self.entries.append((tuple(type_names), fn))
            return fn
        return deco

    set_need_raise = lambda self: None  # noqa: E731

    @staticmethod
    def _kind(x):
        if isinstance(x, torch.Tensor):
            return "Tensor"
        if isinstance(x, bool):
            return "Bool"
        if isinstance(x, (int, float)):
            return "Number"
        if isinstance(x, tuple):
            return "Tuple"
        if isinstance(x, list):
            return "List"
        if x is None:
            return "None"
        if isinstance(x, str):
            return "String"
        if callable(x):
            return "Function"
        return type(x).__name__

    def __call__(self, *args):
        kinds = tuple(self._kind(a) for a in args)
        for sig, fn in self.entries:
            if len(sig) == len(kinds) and all(s == k or s in ("Any",) or (s == "RowTensor" and k == "Tensor")
                                              for s, k in zip(sig, kinds)):
                return fn(*args)
        raise ValueError("The '%s' operation does not support the type %s" % (self.name, list(kinds)))


class HyperMap:
    """Applies ``ops`` to every leaf of (possibly nested) tuples/lists of equal structure."""

    def __init__(self, ops=None, reverse=False):
        self.ops = ops
        self.reverse = reverse

    def __call__(self, *args):
        if self.ops is None:
            fn, args = args[0], args[1:]
        else:
            fn = self.ops
        return self._map(fn, *args)

    def _map(self, fn, *args):
        seq = [a for a in args if isinstance(a, (tuple, list))]
        if not seq:
            return fn(*args)
        n = len(seq[0])
        for s in seq:
            if len(s) != n:
                raise ValueError("HyperMap inputs must have the same length")
        idxs = range(n - 1, -1, -1) if self.reverse else range(n)
        out = [None] * n
        for i in idxs:
            out[i] = self._map(fn, *[a[i] if isinstance(a, (tuple, list)) else a for a in args])
        return tuple(out) if isinstance(seq[0], tuple) else out


class Map(HyperMap):
    def _map(self, fn, *args):
        seq = [a for a in args if isinstance(a, (tuple, list))]
        if not seq:
            return fn(*args)
        n = len(seq[0])
        out = [fn(*[a[i] if isinstance(a, (tuple, list)) else a for a in args]) for i in range(n)]
        return tuple(out) if isinstance(seq[0], tuple) else out


class _PartialFn:
    def __init__(self, fn, *args, **kwargs):
        self.fn, self.args, self.kwargs = fn, args, kwargs

    def __call__(self, *args, **kwargs):
        kw = dict(self.kwargs)
        kw.update(kwargs)
        return self.fn(*self.args, *args, **kw)


def partial(fn, *args, **kwargs):
    return _PartialFn(fn, *args, **kwargs)


class Partial:
    def __call__(self, fn, *args, **kwargs):
        return _PartialFn(fn, *args, **kwargs)


# clip_by_value / clip_by_global_norm (ops/composite/clip_ops.py)
def clip_by_value(x, clip_value_min=None, clip_value_max=None):
    if isinstance(x, (tuple, list)):
        return type(x)(clip_by_value(t, clip_value_min, clip_value_max) for t in x)
    lo = clip_value_min.item() if isinstance(clip_value_min, torch.Tensor) and clip_value_min.numel() == 1 else clip_value_min
    hi = clip_value_max.item() if isinstance(clip_value_max, torch.Tensor) and clip_value_max.numel() == 1 else clip_value_max
    return torch.clamp(x, min=lo, max=hi)


def clip_by_global_norm(x, clip_norm=1.0, use_norm=None):
    if use_norm is None:
        use_norm = torch.sqrt(sum((t.float() ** 2).sum() for t in x))
    scale = clip_norm / torch.maximum(use_norm, torch.as_tensor(float(clip_norm), device=use_norm.device))
    return tuple((t * scale.to(t.dtype)) for t in x)


# ------------------------------------------------------------------------------------------------ further composites
def _wrap_out(o):
    from .primitive import _wrap_out as w
    return w(o)


class ZipOperation:
    """``zip`` over tuples usable inside compiled code (ops/composite/base.py ``ZipOperation``)."""

    def __call__(self, *seqs):
        return tuple(zip(*seqs))


class UnpackCall:
    """``fn(*args_tuple, **kwargs_dict)`` (ops/composite/base.py ``UnpackCall``)."""

    def __call__(self, fn, *packs):
        args, kwargs = [], {}
        for p in packs:
            if isinstance(p, dict):
                kwargs.update(p)
            else:
                args += list(p)
        return fn(*args, **kwargs)


class Shard:
    """Functional form of ``ms.shard``: ``Shard()(fn, in_strategy, out_strategy, ...)``."""

    def __call__(self, fn, in_strategy, out_strategy=None, parameter_plan=None, device="Ascend", level=0):
        from ..parallel.shard import shard as _shard
        return _shard(fn, in_strategy, out_strategy, parameter_plan, device, level)


def count_nonzero(x, axis=(), keep_dims=False, dtype=torch.int32):
    x = _as_plain(x)
    axis = tuple(range(x.dim())) if axis in ((), None) else axis
    out = (x != 0).sum(axis, keepdim=keep_dims)
    return _wrap_out(out.to(dtype))


def _as_plain(x):
    return x if isinstance(x, torch.Tensor) else torch.as_tensor(x)


def tensor_dot(x1, x2, axes):
    return _wrap_out(torch.tensordot(_as_plain(x1), _as_plain(x2), dims=axes))


def dot(x1, x2):
    """Dot product over the last dim of ``x1`` and the second-to-last of ``x2`` (all leading dims kept, NumPy
    ``dot`` semantics for N-d inputs)."""
    a, b = _as_plain(x1), _as_plain(x2)
    if a.dim() <= 2 and b.dim() <= 2:
        return _wrap_out(a @ b)
    return _wrap_out(torch.tensordot(a, b, dims=([-1], [-2 if b.dim() > 1 else 0])))


def repeat_elements(x, rep, axis=0):
    return _wrap_out(torch.repeat_interleave(_as_plain(x), int(rep), dim=axis))


def sequence_mask(lengths, maxlen=None):
    lengths = _as_plain(lengths)
    n = int(lengths.max()) if maxlen is None else int(maxlen)
    return _wrap_out(torch.arange(n, device=lengths.device) < lengths.unsqueeze(-1))


def _seeded(seed):
    g = torch.Generator()
    if seed is not None:
        g.manual_seed(int(seed))
    else:
        g.seed()
    return g


def gamma(shape, alpha, beta, seed=None):
    a = _as_plain(alpha).float().expand(tuple(shape)).contiguous()
    g = _seeded(seed)
    return _wrap_out(torch._standard_gamma(a, generator=g) / _as_plain(beta).float())


def poisson(shape, mean, seed=None):
    m = _as_plain(mean).float().expand(tuple(shape)).contiguous()
    return _wrap_out(torch.poisson(m, generator=_seeded(seed)).to(torch.int32))


def laplace(shape, mean, lambda_param, seed=None):
    u = torch.rand(tuple(shape), generator=_seeded(seed)) - 0.5
    return _wrap_out(_as_plain(mean).float() - _as_plain(lambda_param).float() * torch.sign(u) *
                     torch.log1p(-2 * u.abs()))


def choice_with_mask(input_x, count=256, seed=None):
    x = _as_plain(input_x)
    idx = torch.nonzero(x)
    perm = torch.randperm(idx.shape[0], generator=_seeded(seed))[:count]
    chosen = idx[perm]
    out = torch.zeros((count, x.dim()), dtype=torch.int32)
    out[:chosen.shape[0]] = chosen.to(torch.int32)
    mask = torch.zeros(count, dtype=torch.bool)
    mask[:chosen.shape[0]] = True
    return _wrap_out(out), _wrap_out(mask)


def vmap(fn, in_axes=0, out_axes=0):
    from ..common.api import vmap as _vmap
    return _vmap(fn, in_axes, out_axes)


# ---------------------------------------------------------------------------------------------------- small helpers
def tail(seq):
    """Everything but the first element of a tuple / list (ops/composite/base.py Tail)."""
    if not isinstance(seq, (tuple, list)):
        raise TypeError("For 'tail', the input must be a tuple or a list, but got %s" % type(seq).__name__)
    return seq[1:]


def hyper_add(*values):
    """Elementwise sum over matching nested tuples / lists of tensors and numbers."""
    first = values[0]
    if isinstance(first, (tuple, list)):
        return type(first)(hyper_add(*parts) for parts in zip(*values))
    total = first
    for v in values[1:]:
        total = total + v
    return total


def zip_operation(*seqs):
    return ZipOperation()(*seqs)


def add_flags(fn=None, **flags):
    """Attaches compile flags to a function (``fn._func_graph_flags``); decorator with or without the function."""
    def deco(f):
        if not hasattr(f, "_func_graph_flags"):
            f._func_graph_flags = {}
        f._func_graph_flags.update(flags)
        return f
    return deco(fn) if fn is not None else deco


def env_get(env, parameter):
    """The gradient stored for ``parameter`` in an environment (a dict keyed by the parameter), zeros if absent."""
    if isinstance(env, dict):
        hit = env.get(parameter.name, env.get(id(parameter)))
        if hit is not None:
            return hit
    return _wrap_out(torch.zeros_like(_as_plain(parameter)))


def iter_converter(obj):
    """A cell list / dict / tuple as something ``ms_next`` can walk: dicts give their keys."""
    if isinstance(obj, dict):
        return tuple(obj.keys())
    if isinstance(obj, (tuple, list)):
        return obj
    return tuple(obj)


def ms_hasnext(seq):
    return len(seq) > 0


def ms_next(seq):
    """(first element, the rest): the functional form of a ``for`` loop over a sequence."""
    return seq[0], seq[1:]


_Grad = GradOperation


class _Vmap:
    """Callable form of ``vmap``: ``_Vmap()(fn, in_axes, out_axes)``."""

    def __call__(self, fn, in_axes=0, out_axes=0):
        return vmap(fn, in_axes, out_axes)


def __getattr__(name):
    # the tensor functions that the reference also lists under `composite` (zeros_like, normal, matmul, ...)
    from . import functional
    try:
        return getattr(functional, name)
    except AttributeError:
        from . import function_ext
        if hasattr(function_ext, name):
            return getattr(function_ext, name)
        raise AttributeError("module 'ops.composite' has no attribute %r" % name)
