"""Abstract values and shape / type inference without running a kernel.

An abstract value says what is known about a value before it exists: ``AbstractTensor`` (shape, dtype),
``AbstractScalar`` (type, and the value when it is a constant), ``AbstractSequence``, ``AbstractNone``.  A dimension of
an abstract tensor is an int, or a ``DimExpr``: an affine expression over *symbolic dimensions* (``SymVar``), each with
a range and a ``divisor * n + remainder`` form taken from the ``Symbol`` the user wrote in the input signature.

Inference evaluates the function on storage-less tensors (torch's ``meta`` device: shapes and dtypes propagate, no
memory, no kernel) at a few sample points of the symbolic dimensions and fits every output dimension as an affine
function of them: one base point, one point per symbol with that symbol moved by one admissible step, and one check
point with every symbol moved.  A dimension whose fit fails at the check point (a floor division, a data-dependent
size) is reported unknown (``None``, printed ``-1``).  Two input dimensions that the function needs equal (the rows of
both operands of an Add) are found by starting from one shared value for all symbols and splitting each symbol off
while the function still evaluates; the equalities that had to stay are returned as constraints.  The same engine
serves a single primitive (``Primitive.infer``), a function or cell (``infer``), and a traced graph
(``annotate_graph`` writes ``meta['abstract']`` on every forward node).

Parity (role): mindspore/core/abstract/abstract_value.h (AbstractTensor / AbstractScalar / AbstractTuple, Join and
Broaden), mindspore/core/abstract/dshape.h (dynamic dims -1, dynamic rank -2), mindspore/core/symbolic_shape/
(int symbols with range / divisor / remainder, symbol engine over a graph), mindspore/core/ops/*_infer
(``InferShape`` / ``InferType`` per primitive), mindspore/ccsrc/pipeline/jit/ps/static_analysis/ (evaluators).
"""
from fractions import Fraction

import torch
from torch.utils._python_dispatch import TorchDispatchMode
from torch.utils._pytree import tree_map

__all__ = ["SymVar", "DimExpr", "AbstractValue", "AbstractTensor", "AbstractScalar", "AbstractSequence",
           "AbstractNone", "InferenceError", "to_abstract", "infer", "infer_with_constraints", "check_signature",
           "annotate_graph", "DYNAMIC_DIM", "DYNAMIC_RANK"]

DYNAMIC_DIM = -1           # an unknown dimension in a shape list
DYNAMIC_RANK = -2          # the whole shape, rank included, is unknown: shape == [-2]


class InferenceError(RuntimeError):
    pass


# ------------------------------------------------------------------------------------------------ symbolic dimensions
class SymVar:
    """One symbolic dimension: ``value = divisor * n + remainder`` with ``min <= value`` (``<= max`` when set)."""

    def __init__(self, name, min=1, max=0, divisor=1, remainder=0):                       # noqa: A002
        self.name, self.min, self.max, self.divisor, self.remainder = name, int(min), int(max), int(divisor), \
            int(remainder)

    def sample(self, k):
        """The ``k``-th admissible value (k = 0 is the smallest), clipped to ``max``."""
        first = self.min + ((self.remainder - self.min) % self.divisor)
        v = first + k * self.divisor
        if self.max and v > self.max:
            last = self.max - ((self.max - self.remainder) % self.divisor)
            v = max(first, last)
        return v

    def admits(self, value):
        if value < self.min or (self.max and value > self.max):
            return False
        return value % self.divisor == self.remainder

    def __repr__(self):
        return self.name


class DimExpr:
    """``sum(coeff[v] * v) + const`` over symbolic dimensions; coefficients are exact fractions."""

    def __init__(self, coeffs, const=0):
        self.coeffs = {v: Fraction(c) for v, c in coeffs.items() if c != 0}
        self.const = Fraction(const)

    @classmethod
    def of(cls, var):
        return cls({var: 1}, 0)

    def evaluate(self, bindings):
        total = self.const
        for v, c in self.coeffs.items():
            total += c * bindings[v]
        if total.denominator != 1:
            raise InferenceError("dimension %r is not an integer for %r" % (self, bindings))
        return int(total)

    def is_static(self):
        return not self.coeffs

    def bounds(self):
        """(min, max) of the value over the ranges of the symbols; max is 0 when unbounded."""
        lo = hi = self.const
        unbounded = False
        for v, c in self.coeffs.items():
            vlo, vhi = v.sample(0), v.max
            if c > 0:
                lo += c * vlo
                unbounded |= not vhi
                hi += c * (vhi or 0)
            else:
                hi += c * vlo
                unbounded = True if not vhi else unbounded
                lo += c * (vhi or vlo)
        return int(lo), (0 if unbounded else int(hi))

    def divisor_remainder(self):
        """(divisor, remainder) of the value when it depends on one symbol by an integer factor, else (1, 0)."""
        if len(self.coeffs) == 1:
            (v, c), = self.coeffs.items()
            step, offset = c * v.divisor, c * v.remainder + self.const
            if c > 0 and step.denominator == 1 and offset.denominator == 1:
                return int(step), int(offset) % int(step)
        return 1, 0

    def to_symbol(self):
        """The same knowledge as a ``Symbol`` of the input-signature API."""
        from ..common.api import Symbol
        lo, hi = self.bounds()
        d, r = self.divisor_remainder()
        return Symbol(max=max(hi, 0), min=max(lo, 1), divisor=d, remainder=r)

    def __eq__(self, other):
        if isinstance(other, int):
            return self.is_static() and self.const == other
        return isinstance(other, DimExpr) and self.coeffs == other.coeffs and self.const == other.const

    def __hash__(self):
        return hash((tuple(sorted((v.name, c) for v, c in self.coeffs.items())), self.const))

    def __repr__(self):
        parts = []
        for v, c in sorted(self.coeffs.items(), key=lambda kv: kv[0].name):
            if c == 1:
                parts.append(v.name)
            elif c.denominator == 1:
                parts.append("%d*%s" % (c, v.name))
            else:
                parts.append("%s/%d" % (v.name if c.numerator == 1 else "%d*%s" % (c.numerator, v.name),
                                        c.denominator))
        if self.const or not parts:
            parts.append(str(self.const))
        return "+".join(parts).replace("+-", "-")


# ---------------------------------------------------------------------------------------------------- abstract values
class AbstractValue:
    def broaden(self):
        """The same type without a known value."""
        return self

    def join(self, other):
        """The least abstract value that covers both (used where two branches of a graph meet)."""
        raise NotImplementedError


class AbstractNone(AbstractValue):
    def join(self, other):
        if isinstance(other, AbstractNone):
            return self
        raise InferenceError("cannot join None with %r" % (other,))

    def __eq__(self, other):
        return isinstance(other, AbstractNone)

    def __hash__(self):
        return hash("AbstractNone")

    def __repr__(self):
        return "None"


class AbstractScalar(AbstractValue):
    """A Python number / bool / string: ``type`` and, for a compile-time constant, ``value`` (a ``DimExpr`` when it
    was computed from symbolic dimensions)."""

    def __init__(self, type, value=None):                                                  # noqa: A002
        self.type, self.value = type, value

    def broaden(self):
        return AbstractScalar(self.type, None)

    def join(self, other):
        if not isinstance(other, AbstractScalar) or other.type is not self.type:
            raise InferenceError("cannot join %r with %r" % (self, other))
        return self if self.value is not None and self.value == other.value else self.broaden()

    def __eq__(self, other):
        return isinstance(other, AbstractScalar) and self.type is other.type and self.value == other.value

    def __hash__(self):
        return hash((self.type, repr(self.value)))

    def __repr__(self):
        return "%s(%s)" % (self.type.__name__, "?" if self.value is None else self.value)


class AbstractTensor(AbstractValue):
    """``shape``: a tuple whose entries are ints, ``DimExpr`` or ``None`` (unknown); ``None`` instead of a tuple means
    the rank is unknown too.  Input signatures may also hold ``Symbol`` objects in it."""

    def __init__(self, shape, dtype):
        self.shape = None if shape is None else tuple(shape)
        self.dtype = dtype

    @property
    def shape_list(self):
        """The ``[-1, 128]`` form: -1 for every dimension that is not a fixed int, ``[-2]`` for an unknown rank."""
        if self.shape is None:
            return [DYNAMIC_RANK]
        return [int(d.const) if isinstance(d, DimExpr) and d.is_static() else d if isinstance(d, int) else DYNAMIC_DIM
                for d in self.shape]

    def is_dynamic(self):
        return self.shape is None or any(not isinstance(d, int) for d in self.shape)

    def join(self, other):
        if not isinstance(other, AbstractTensor) or other.dtype != self.dtype:
            raise InferenceError("cannot join %r with %r" % (self, other))
        if self.shape is None or other.shape is None or len(self.shape) != len(other.shape):
            return AbstractTensor(None, self.dtype)
        return AbstractTensor([a if _same_dim(a, b) else None for a, b in zip(self.shape, other.shape)], self.dtype)

    def __eq__(self, other):
        return isinstance(other, AbstractTensor) and self.dtype == other.dtype and (
            (self.shape is None) == (other.shape is None)) and (
            self.shape is None or (len(self.shape) == len(other.shape) and
                                   all(_same_dim(a, b) for a, b in zip(self.shape, other.shape))))

    def __hash__(self):
        return hash((self.dtype, repr(self.shape)))

    def __repr__(self):
        shape = "?" if self.shape is None else "(%s)" % ", ".join("-1" if d is None else str(d) for d in self.shape)
        return "Tensor[%s]%s" % (str(self.dtype).replace("torch.", ""), shape)


class AbstractSequence(AbstractValue):
    def __init__(self, elements, kind=tuple):
        self.elements, self.kind = list(elements), kind

    def broaden(self):
        return AbstractSequence([e.broaden() for e in self.elements], self.kind)

    def join(self, other):
        if not isinstance(other, AbstractSequence) or len(other.elements) != len(self.elements):
            raise InferenceError("cannot join sequences %r and %r" % (self, other))
        return AbstractSequence([a.join(b) for a, b in zip(self.elements, other.elements)], self.kind)

    def __len__(self):
        return len(self.elements)

    def __getitem__(self, i):
        return self.elements[i]

    def __eq__(self, other):
        return isinstance(other, AbstractSequence) and self.kind is other.kind and self.elements == other.elements

    def __hash__(self):
        return hash((self.kind, tuple(self.elements)))

    def __repr__(self):
        o, c = ("(", ")") if self.kind is tuple else ("[", "]")
        return o + ", ".join(repr(e) for e in self.elements) + c


def _same_dim(a, b):
    if a is None or b is None:
        return False
    return a == b


def _is_symbol(d):
    return type(d).__name__ == "Symbol" and hasattr(d, "divisor")


def to_abstract(v):
    """The abstract value of a runtime value, a placeholder tensor (``Tensor(shape=[None, 8], dtype=...)``) or an
    abstract value (returned as it is)."""
    if isinstance(v, AbstractValue):
        return v
    if isinstance(v, torch.Tensor):
        sym = getattr(v, "symbolic_shape", None)
        if sym is not None or getattr(v, "dynamic_rank", False):
            return AbstractTensor(None if getattr(v, "dynamic_rank", False) else sym, v.dtype)
        return AbstractTensor(tuple(v.shape), v.dtype)
    if v is None:
        return AbstractNone()
    if isinstance(v, (bool, int, float, str, complex)):
        return AbstractScalar(type(v), v)
    if isinstance(v, (tuple, list)):
        return AbstractSequence([to_abstract(e) for e in v], type(v) if type(v) in (tuple, list) else tuple)
    if isinstance(v, torch.dtype):
        return AbstractScalar(torch.dtype, v)
    return AbstractScalar(type(v), v)


# ------------------------------------------------------------------------------------------------------ the inference
class _Problem:
    """The symbolic dimensions of one call and the way to build concrete (meta) arguments for a sample point."""

    def __init__(self, abstracts):
        self.vars = []
        self._by_symbol = {}
        self.templates = [self._template(a) for a in abstracts]

    def _new_var(self, sym=None):
        name = "s%d" % len(self.vars)
        v = SymVar(name) if sym is None else SymVar(name, sym.min, sym.max, sym.divisor, sym.remainder)
        self.vars.append(v)
        return v

    def _dim(self, d):
        if d is None or (isinstance(d, int) and d == DYNAMIC_DIM):
            return self._new_var()
        if _is_symbol(d):
            if getattr(d, "unique", False):
                v = self._by_symbol.get(id(d))
                if v is None:
                    v = self._by_symbol[id(d)] = self._new_var(d)
                return v
            return self._new_var(d)
        if isinstance(d, DimExpr):
            if d.is_static():
                return int(d.const)
            raise InferenceError("an input dimension must be an int, None or a Symbol, but got %r" % (d,))
        return int(d)

    def _template(self, a):
        if isinstance(a, AbstractTensor):
            if a.shape is None:
                return ("rank", a.dtype)
            return ("tensor", tuple(self._dim(d) for d in a.shape), a.dtype)
        if isinstance(a, AbstractSequence):
            return ("seq", a.kind, [self._template(e) for e in a.elements])
        if isinstance(a, AbstractNone):
            return ("value", None)
        if isinstance(a, AbstractScalar):
            if a.value is None:
                return ("value", {bool: True, int: 1, float: 1.0, str: ""}.get(a.type, None))
            return ("value", a.value)
        return ("value", a)

    def materialize(self, bindings, rank=2):
        from ..common.tensor import Tensor

        def build(t):
            kind = t[0]
            if kind == "tensor":
                shape = [bindings[d] if isinstance(d, SymVar) else d for d in t[1]]
                return torch.Tensor._make_subclass(Tensor, torch.empty(shape, dtype=t[2], device="meta"), False)
            if kind == "rank":
                return torch.Tensor._make_subclass(Tensor, torch.empty([2] * rank, dtype=t[1], device="meta"), False)
            if kind == "seq":
                return t[1](build(e) for e in t[2])
            return t[1]
        return [build(t) for t in self.templates]

    def has_dynamic_rank(self):
        def any_rank(t):
            return t[0] == "rank" or (t[0] == "seq" and any(any_rank(e) for e in t[2]))
        return any(any_rank(t) for t in self.templates)


def _describe(out):
    """A structure of plain data for one evaluation: what `_fit` compares across sample points."""
    if isinstance(out, torch.Tensor):
        return ("tensor", tuple(int(d) for d in out.shape), out.dtype)
    if out is None:
        return ("none",)
    if isinstance(out, bool):
        return ("scalar", bool, out)
    if isinstance(out, int):
        return ("int", out)
    if isinstance(out, (float, str, complex, torch.dtype)):
        return ("scalar", type(out), out)
    if isinstance(out, torch.Size):
        return ("seq", tuple, [("int", int(d)) for d in out])
    if isinstance(out, (tuple, list)):
        return ("seq", list if isinstance(out, list) else tuple, [_describe(e) for e in out])
    if isinstance(out, dict):
        return ("seq", tuple, [_describe(e) for e in out.values()])
    return ("scalar", type(out), None)


def _fit_int(values, points, var_order, steps):
    """values[0] at the base point, values[1 + i] with symbol i moved by steps[i], values[-1] at the check point."""
    base = values[0]
    coeffs = {}
    for i, v in enumerate(var_order):
        delta = values[1 + i] - base
        if delta:
            coeffs[v] = Fraction(delta, steps[i])
    const = Fraction(base) - sum(c * points[0][v] for v, c in coeffs.items())
    expr = DimExpr(coeffs, const)
    predicted = expr.const + sum(c * points[-1][v] for v, c in expr.coeffs.items())
    if predicted != values[-1]:
        return None
    return int(base) if expr.is_static() else expr


def _fit(samples, points, var_order, steps):
    first = samples[0]
    kind = first[0]
    if any(s[0] != kind for s in samples):
        raise InferenceError("the kind of the result changes with the input shape")
    if kind == "tensor":
        if any(s[2] != first[2] for s in samples):
            raise InferenceError("the dtype of the result changes with the input shape")
        if any(len(s[1]) != len(first[1]) for s in samples):
            return AbstractTensor(None, first[2])
        dims = [_fit_int([s[1][k] for s in samples], points, var_order, steps) for k in range(len(first[1]))]
        return AbstractTensor(dims, first[2])
    if kind == "none":
        return AbstractNone()
    if kind == "int":
        return AbstractScalar(int, _fit_int([s[1] for s in samples], points, var_order, steps))
    if kind == "scalar":
        same = all(s[2] == first[2] for s in samples)
        return AbstractScalar(first[1], first[2] if same else None)
    if kind == "seq":
        if any(len(s[2]) != len(first[2]) for s in samples):
            raise InferenceError("the length of a result sequence changes with the input shape")
        return AbstractSequence([_fit([s[2][k] for s in samples], points, var_order, steps)
                                 for k in range(len(first[2]))], first[1])
    raise InferenceError("unknown result kind %r" % (kind,))


class _StoragelessMode(TorchDispatchMode):
    """Every operator sees storage-less operands: a real tensor that meets the evaluation (a parameter of the cell,
    a constant the function builds) is replaced by a ``meta`` tensor of its shape and dtype."""

    def __torch_dispatch__(self, func, types, args=(), kwargs=None):
        def strip(t):
            if isinstance(t, torch.Tensor) and t.device.type != "meta":
                return torch.empty_strided(t.shape, t.stride(), dtype=t.dtype, device="meta")
            return t
        args, kwargs = tree_map(strip, (args, kwargs or {}))
        return func(*args, **kwargs)


def _evaluate(fn, problem, bindings, kwargs, rank=2):
    args = problem.materialize(bindings, rank)
    with torch.no_grad(), _StoragelessMode():
        return _describe(fn(*args, **kwargs))


def _point(groups, offset):
    """One value per group of unified symbols: member symbols get the group's value.  Distinct groups get distinct
    sample indices so that two dimensions agree only when they are unified."""
    bindings = {}
    for gi, group in enumerate(groups):
        k = 1 + gi + offset.get(gi, 0)
        value = max(v.sample(k) for v in group)
        for v in group:
            bindings[v] = value if v.admits(value) else v.sample(k)
    return bindings


def _try(fn, problem, groups, kwargs):
    try:
        return _evaluate(fn, problem, _point([g for g in groups if g], {}), kwargs)
    except InferenceError:
        raise
    except Exception as e:                                                                  # noqa: BLE001
        return e


def _partition(fn, problem, kwargs):
    """Groups of symbols that must hold one value.  All independent if the function evaluates that way; otherwise
    start from one shared value and split symbols off one at a time while the evaluation still succeeds."""
    vs = problem.vars
    independent = [[v] for v in vs]
    if not vs:
        return independent
    r = _try(fn, problem, independent, kwargs)
    if not isinstance(r, Exception):
        return independent
    first_error = r
    groups = [list(vs)]
    r = _try(fn, problem, groups, kwargs)
    if isinstance(r, Exception):
        raise InferenceError("inference failed: %s: %s (with independent dynamic dimensions: %s)"
                             % (type(r).__name__, r, first_error)) from r
    moved = set()
    for v in vs:
        if v in moved:
            continue
        main = groups[0]
        # v on its own, v joined to a group split off earlier, or v with one partner (two pairs of equal
        # dimensions that are independent of each other come apart this way)
        options = [("new", [v])] + [("join", gi) for gi in range(1, len(groups))] + \
                  [("new", [v, w]) for w in main if w is not v]
        for kind, what in options:
            taken = [v] if kind == "join" else what
            rest = [x for x in main if x not in taken]
            if kind == "new":
                trial = [rest] + groups[1:] + [list(what)]
            else:
                trial = [rest] + [g + [v] if gi == what else g for gi, g in enumerate(groups) if gi >= 1]
            if not isinstance(_try(fn, problem, trial, kwargs), Exception):
                groups = trial
                moved.update(taken)
                break
    return [g for g in groups if g]


def infer_with_constraints(fn, *args, **kwargs):
    """``(abstract result, constraints)``: constraints is a list of tuples of symbol names that had to be equal for
    ``fn`` to accept the inputs (``[("s0", "s2")]``)."""
    abstracts = [to_abstract(a) for a in args]
    problem = _Problem(abstracts)
    if problem.has_dynamic_rank():
        outs = []
        for rank in (1, 2, 3, 4):
            try:
                outs.append(_evaluate(fn, problem, {v: v.sample(1) for v in problem.vars}, kwargs, rank))
            except Exception:                                                               # noqa: BLE001
                continue
        if not outs:
            raise InferenceError("inference failed for every rank from 1 to 4 of the dynamic-rank inputs")
        return _broaden_rank(outs), []
    groups = _partition(fn, problem, kwargs)
    reps = [g[0] for g in groups]                      # the fitted expressions are written over one symbol per group
    points = [_point(groups, {})]
    steps = []
    for gi, g in enumerate(groups):
        moved = _point(groups, {gi: 1})
        steps.append(moved[g[0]] - points[0][g[0]])
        points.append(moved)
    points.append(_point(groups, {gi: 2 + gi for gi in range(len(groups))}))
    usable = [i for i, s in enumerate(steps) if s != 0]   # a symbol whose range holds one value cannot move
    samples = []
    for p in points:
        try:
            samples.append(_evaluate(fn, problem, p, kwargs))
        except InferenceError:
            raise
        except Exception as e:                                                              # noqa: BLE001
            raise InferenceError("inference failed at %r: %s: %s" % (p, type(e).__name__, e)) from e
    keep = [0] + [1 + i for i in usable] + [len(points) - 1]
    out = _fit([samples[i] for i in keep], [points[i] for i in keep], [reps[i] for i in usable],
               [steps[i] for i in usable])
    constraints = [tuple(v.name for v in g) for g in groups if len(g) > 1]
    return out, constraints


def _broaden_rank(outs):
    first = outs[0]
    if first[0] == "tensor":
        same_shape = all(o[1] == first[1] for o in outs)
        return AbstractTensor(first[1] if same_shape else None, first[2])
    if first[0] == "seq":
        return AbstractSequence([_broaden_rank([o[2][k] for o in outs]) for k in range(len(first[2]))], first[1])
    if first[0] == "none":
        return AbstractNone()
    if first[0] == "int":
        return AbstractScalar(int, first[1] if all(o[1] == first[1] for o in outs) else None)
    return AbstractScalar(first[1], first[2] if all(o[2] == first[2] for o in outs) else None)


def infer(fn, *args, **kwargs):
    """The abstract result of ``fn(*args)``; ``args`` are abstract values, placeholder tensors or real values."""
    return infer_with_constraints(fn, *args, **kwargs)[0]


# ---------------------------------------------------------------------------------------------------- signature check
def check_signature(signature, args, what="input_signature"):
    """Check real arguments against a signature of placeholder tensors; returns the values of the unique symbols.
    Raises ``TypeError`` for a wrong kind or dtype and ``ValueError`` for a shape the signature does not admit."""
    signature = list(signature) if isinstance(signature, (tuple, list)) else [signature]
    if len(signature) != len(args):
        raise ValueError("For '%s', the number of arguments must be %d, but got %d"
                         % (what, len(signature), len(args)))
    bound = {}
    for i, (spec, arg) in enumerate(zip(signature, args)):
        _check_one(to_abstract(spec), arg, "%s[%d]" % (what, i), bound)
    return bound


def _check_one(spec, arg, where, bound):
    if isinstance(spec, AbstractSequence):
        if not isinstance(arg, (tuple, list)) or len(arg) != len(spec.elements):
            raise TypeError("For %s, a sequence of %d elements is expected, but got %r"
                            % (where, len(spec.elements), type(arg).__name__))
        for k, (s, a) in enumerate(zip(spec.elements, arg)):
            _check_one(s, a, "%s[%d]" % (where, k), bound)
        return
    if not isinstance(spec, AbstractTensor):
        return
    if not isinstance(arg, torch.Tensor):
        raise TypeError("For %s, a Tensor is expected, but got %s" % (where, type(arg).__name__))
    if arg.dtype != spec.dtype:
        raise TypeError("For %s, the dtype must be %s, but got %s" % (where, spec.dtype, arg.dtype))
    if spec.shape is None:
        return
    if len(spec.shape) != arg.dim():
        raise ValueError("For %s, the rank must be %d, but got shape %s" % (where, len(spec.shape), tuple(arg.shape)))
    for axis, (d, real) in enumerate(zip(spec.shape, arg.shape)):
        if d is None or (isinstance(d, int) and d == DYNAMIC_DIM):
            continue
        if _is_symbol(d):
            if not d.admits(int(real)):
                raise ValueError("For %s, dimension %d is %d, which %r does not admit" % (where, axis, real, d))
            if getattr(d, "unique", False):
                seen = bound.setdefault(id(d), int(real))
                if seen != int(real):
                    raise ValueError("For %s, dimension %d is %d, but the same unique Symbol was %d elsewhere"
                                     % (where, axis, real, seen))
            continue
        if int(d) != int(real):
            raise ValueError("For %s, dimension %d must be %d, but got shape %s"
                             % (where, axis, int(d), tuple(arg.shape)))


# ------------------------------------------------------------------------------------------------------- graph pass
def annotate_graph(fg, inputs):
    """Run the forward nodes of a traced graph on storage-less tensors and record every node's abstract value in
    ``node.meta['abstract']``.  Gradient nodes are skipped (their shapes are those of the values they differentiate).
    Returns the number of nodes annotated."""
    import torch.fx as fx

    from . import autodiff
    from ..common.tensor import Tensor

    def meta_of(t):
        if isinstance(t, torch.Tensor):
            return torch.Tensor._make_subclass(Tensor, torch.empty(tuple(t.shape), dtype=t.dtype, device="meta"), False)
        if isinstance(t, (tuple, list)):
            return type(t)(meta_of(e) for e in t)
        return t

    env = {}
    it = iter(inputs)
    done = 0
    for n in fg.graph.nodes:
        try:
            if n.op == "placeholder":
                env[n] = meta_of(next(it))
            elif n.op == "get_attr":
                env[n] = meta_of(n.meta["param"] if "param" in n.meta else n.meta["const"])
            elif n.op == "call_function":
                if n.target is autodiff.vjp or any(a not in env for a in n.all_input_nodes):
                    continue
                args = fx.node.map_arg(n.args, lambda a: env[a])
                kwargs = fx.node.map_arg(n.kwargs, lambda a: env[a])
                with torch.no_grad(), _StoragelessMode():
                    env[n] = n.target(*args, **kwargs)
            else:
                continue
        except Exception:                                                                   # noqa: BLE001
            continue                   # a node that needs real data (an index read on the host): left unannotated
        n.meta["abstract"] = to_abstract(env[n])
        done += 1
    return done
