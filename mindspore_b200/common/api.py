"""Top-level helpers of the ``mindspore`` namespace that are neither tensors nor cells: compile hints
(``mutable``, ``lazy_inline``, ``no_inline``, ``jit_class``, ``recompute``), ``Symbol`` for dynamic dimensions,
random ``Generator``, sparse tensor containers, ``vmap`` / ``hessian`` / ``get_grad``, ``data_sink``,
``ms_memory_recycle``, ``run_check`` and the strategy-search knobs.

Parity: python/mindspore/common/{mutable.py, lazy_inline.py, no_inline.py, jit_class (api.py:1040), recompute.py,
symbol.py, generator.py, sparse_tensor.py}, ops/composite (vmap), train/data_sink.py, run_check/_check_version.py,
parallel/algo_parameter_config.py."""
from __future__ import annotations

import functools
import gc

import numpy as np
import torch

from .tensor import Tensor

__all__ = ["mutable", "lazy_inline", "no_inline", "jit_class", "recompute", "Symbol", "Generator", "default_generator",
           "manual_seed", "initial_seed", "get_rng_state", "set_rng_state", "COOTensor", "CSRTensor", "RowTensor",
           "SparseTensor", "vmap", "hessian", "get_grad", "data_sink", "ms_memory_recycle", "run_check",
           "set_algo_parameters", "get_algo_parameters", "reset_algo_parameters", "set_cost_model_context", "get_cost_model_context", "reset_cost_model_context"]


# ------------------------------------------------------------------------------------------------ compile hints
def mutable(input_data, dynamic_len=False):
    """Marks a constant (scalar / tuple / list / dict of tensors) as a graph *input* rather than a compile-time
    constant.  The tracer here treats every tensor argument as an input already; Python scalars are turned into
    0-d tensors so that a new value does not force a recompile."""
    def conv(v):
        if isinstance(v, (bool, int, float)):
            return Tensor(torch.tensor(v))
        if isinstance(v, (list, tuple)):
            return type(v)(conv(x) for x in v)
        if isinstance(v, dict):
            return {k: conv(x) for k, x in v.items()}
        if isinstance(v, torch.Tensor) or v is None:
            return v
        raise TypeError("For 'mutable', the 'input_data' should be one of (bool, int, float, Tensor, tuple, list, "
                        "dict), but got %s" % type(v).__name__)
    out = conv(input_data)
    if dynamic_len and not isinstance(input_data, (list, tuple)):
        raise TypeError("For 'mutable', 'dynamic_len' can only be used with a tuple or list")
    return out


def lazy_inline(fn=None, attrs=None):
    """Marks a Cell's ``__init__``: identical sub-graphs of this cell type are compiled once and reused.  The tracer
    caches compiled sub-cells by (type, attrs) when this mark is present."""
    def wrap(f):
        @functools.wraps(f)
        def init(self, *args, **kwargs):
            f(self, *args, **kwargs)
            key = attrs if attrs is not None else tuple(list(args) + sorted(kwargs.items(), key=lambda kv: kv[0]))
            object.__setattr__(self, "_lazy_inline_key", (type(self).__name__, repr(key)))
        return init
    return wrap(fn) if callable(fn) else wrap


def no_inline(fn=None):
    """The function is kept as its own sub-graph (not inlined into the caller) by the tracer."""
    def wrap(f):
        f._no_inline = True
        return f
    return wrap(fn) if fn is not None else wrap


def jit_class(cls):
    """Instances of ``cls`` may be created and used inside compiled functions."""
    if not isinstance(cls, type):
        raise TypeError("Decorator jit_class can only be used for class type, but got %s." % (cls,))
    cls.__ms_class__ = True
    return cls


def recompute(block, *args, **kwargs):
    """Runs ``block(*args)`` without keeping its activations; they are recomputed during backward."""
    from torch.utils.checkpoint import checkpoint
    from ..nn.cell import Cell
    if not isinstance(block, Cell) and not callable(block):
        raise TypeError("For 'recompute', 'block' must be a Cell or a function")
    out = checkpoint(lambda *a: block(*a, **kwargs), *args, use_reentrant=False)
    return out


class Symbol:
    """A dimension whose value is only known at run time, with what is known about it: ``max`` / ``min`` bounds,
    ``divisor`` and ``remainder`` (dim = divisor * n + remainder), ``unique`` (all uses are the same value).  Used in
    ``Tensor(shape=(Symbol(divisor=8), 128), dtype=...)`` input signatures."""

    def __init__(self, max=0, min=1, divisor=1, remainder=0, unique=False, **kwargs):      # noqa: A002
        for name, v in (("max", max), ("min", min), ("divisor", divisor), ("remainder", remainder)):
            if not isinstance(v, int) or isinstance(v, bool):
                raise TypeError("For 'Symbol', '%s' must be an int, but got %s" % (name, type(v).__name__))
        if min <= 0:
            raise ValueError("For 'Symbol', 'min' must be positive, but got %d" % min)
        if divisor <= 0:
            raise ValueError("For 'Symbol', 'divisor' must be positive, but got %d" % divisor)
        if remainder < 0 or remainder >= divisor:
            raise ValueError("For 'Symbol', 'remainder' must be in [0, divisor), but got %d" % remainder)
        if max and max < min:
            raise ValueError("For 'Symbol', 'max' must not be less than 'min'")
        self.max, self.min, self.divisor, self.remainder, self.unique = max, min, divisor, remainder, unique
        self.id = id(self) if unique else None

    def admits(self, value):
        if value < self.min or (self.max and value > self.max):
            return False
        return value % self.divisor == self.remainder

    def to_dict(self):
        d = {"min": self.min, "divisor": self.divisor, "remainder": self.remainder}
        if self.max:
            d["max"] = self.max
        if self.unique:
            d["id"] = self.id
        return d

    def __repr__(self):
        return "Symbol(%s)" % ", ".join("%s=%s" % kv for kv in self.to_dict().items())


# ------------------------------------------------------------------------------------------------ random generator
class Generator:
    def __init__(self):
        self._cpu = torch.Generator()
        self._cuda = None

    def _gen(self, device="cpu"):
        if str(device).startswith("cuda"):
            if self._cuda is None:
                self._cuda = torch.Generator(device)
                self._cuda.manual_seed(self._cpu.initial_seed())
            return self._cuda
        return self._cpu

    def manual_seed(self, seed):
        self._cpu.manual_seed(int(seed))
        if self._cuda is not None:
            self._cuda.manual_seed(int(seed))
        return self

    def seed(self):
        s = self._cpu.seed()
        if self._cuda is not None:
            self._cuda.manual_seed(s)
        return s

    def initial_seed(self):
        return self._cpu.initial_seed()

    def get_state(self):
        return Tensor(self._cpu.get_state())

    def set_state(self, state):
        self._cpu.set_state(torch.as_tensor(state, dtype=torch.uint8).cpu())


default_generator = Generator()


def manual_seed(seed):
    torch.manual_seed(int(seed))
    return default_generator.manual_seed(seed)


def seed():
    """Seeds the default generator from the system's entropy and returns the seed (common/generator.py seed)."""
    return default_generator.seed()


class _no_grad:
    """Context manager / decorator: no gradient is recorded inside (common/_pijit_context ... ``_no_grad``)."""

    def __enter__(self):
        self._ctx = torch.no_grad()
        return self._ctx.__enter__()

    def __exit__(self, *exc):
        return self._ctx.__exit__(*exc)

    def __call__(self, fn):
        import functools

        @functools.wraps(fn)
        def wrapper(*args, **kwargs):
            with torch.no_grad():
                return fn(*args, **kwargs)
        return wrapper


class _NullType:
    """The type of ``_null``: a default that means "argument not given" where ``None`` is a legal value."""

    _instance = None

    def __new__(cls):
        if cls._instance is None:
            cls._instance = super().__new__(cls)
        return cls._instance

    def __repr__(self):
        return "null"

    def __bool__(self):
        return False


_null = _NullType()


def initial_seed():
    return default_generator.initial_seed()


def get_rng_state():
    return default_generator.get_state()


def set_rng_state(state):
    default_generator.set_state(state)


# ------------------------------------------------------------------------------------------------ sparse containers
class COOTensor:
    """Coordinate-format sparse tensor: ``indices`` [nnz, ndim] int, ``values`` [nnz], dense ``shape``."""

    def __init__(self, indices=None, values=None, shape=None, coo_tensor=None):
        if coo_tensor is not None:
            indices, values, shape = coo_tensor.indices, coo_tensor.values, coo_tensor.shape
        self.indices = Tensor(torch.as_tensor(indices))
        self.values = Tensor(torch.as_tensor(values))
        self.shape = tuple(int(s) for s in shape)
        if self.indices.dim() != 2 or self.indices.shape[1] != len(self.shape):
            raise ValueError("For COOTensor, 'indices' must be [nnz, %d], but got %s"
                             % (len(self.shape), tuple(self.indices.shape)))
        if self.indices.shape[0] != self.values.shape[0]:
            raise ValueError("For COOTensor, 'indices' and 'values' must have the same length")

    @property
    def dtype(self):
        return self.values.dtype

    @property
    def size(self):
        return int(self.values.numel())

    @property
    def ndim(self):
        return len(self.shape)

    def _torch(self):
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter("ignore", UserWarning)          # torch announces its invariant-check default once
            return torch.sparse_coo_tensor(self.indices.t().long(), self.values, self.shape, check_invariants=True)

    def to_dense(self):
        return Tensor(self._torch().to_dense())

    def coalesce(self):
        t = self._torch().coalesce()
        return COOTensor(t.indices().t(), t.values(), self.shape)

    def to_csr(self):
        if len(self.shape) != 2:
            raise ValueError("only 2-D COOTensor can be converted to CSRTensor")
        t = self._torch().coalesce()
        rows, cols = t.indices()[0], t.indices()[1]
        indptr = torch.zeros(self.shape[0] + 1, dtype=torch.int64, device=rows.device)
        indptr[1:] = torch.cumsum(torch.bincount(rows, minlength=self.shape[0]), 0)
        return CSRTensor(indptr, cols, t.values(), self.shape)

    def to_tuple(self):
        return self.indices, self.values, self.shape

    def astype(self, dtype):
        return COOTensor(self.indices, self.values.to(dtype), self.shape)

    def abs(self):
        return COOTensor(self.indices, self.values.abs(), self.shape)

    def add(self, other, thresh=0.0):
        t = (self._torch() + other._torch()).coalesce()
        keep = t.values().abs() > thresh if thresh else torch.ones_like(t.values(), dtype=torch.bool)
        return COOTensor(t.indices().t()[keep], t.values()[keep], self.shape)

    def __mul__(self, dense):
        d = torch.as_tensor(dense)
        if d.dim() == 0:
            return COOTensor(self.indices, self.values * d, self.shape)
        picked = d.expand(self.shape)[tuple(self.indices.long().t())]
        return COOTensor(self.indices, self.values * picked, self.shape)

    def __repr__(self):
        return "COOTensor(shape=%s, dtype=%s, nnz=%d)" % (self.shape, self.dtype, self.size)


SparseTensor = COOTensor


class CSRTensor:
    """Compressed-sparse-row matrix (optionally batched in trailing dense dims): ``indptr`` [rows + 1], ``indices``
    [nnz] column ids, ``values`` [nnz, ...]."""

    def __init__(self, indptr=None, indices=None, values=None, shape=None, csr_tensor=None):
        if csr_tensor is not None:
            indptr, indices, values, shape = csr_tensor.indptr, csr_tensor.indices, csr_tensor.values, csr_tensor.shape
        self.indptr = Tensor(torch.as_tensor(indptr))
        self.indices = Tensor(torch.as_tensor(indices))
        self.values = Tensor(torch.as_tensor(values))
        self.shape = tuple(int(s) for s in shape)
        if self.indptr.numel() != self.shape[0] + 1:
            raise ValueError("For CSRTensor, 'indptr' must have shape[0] + 1 = %d entries, but got %d"
                             % (self.shape[0] + 1, self.indptr.numel()))
        if self.indices.shape[0] != self.values.shape[0]:
            raise ValueError("For CSRTensor, 'indices' and 'values' must have the same length")

    @property
    def dtype(self):
        return self.values.dtype

    @property
    def size(self):
        return int(self.values.numel())

    @property
    def ndim(self):
        return len(self.shape)

    def _rows(self):
        counts = (self.indptr[1:] - self.indptr[:-1]).long()
        return torch.repeat_interleave(torch.arange(self.shape[0], device=counts.device), counts)

    @property
    def itemsize(self):
        return self.values.element_size()

    def add(self, b, alpha, beta):
        """``alpha * self + beta * b`` for two CSR matrices of one shape (CSRTensor.add)."""
        if not isinstance(b, CSRTensor) or tuple(b.shape) != tuple(self.shape):
            raise ValueError("For 'CSRTensor.add', 'b' must be a CSRTensor of the same shape")
        dense = float(torch.as_tensor(alpha)) * self.to_dense().as_subclass(torch.Tensor) + \
            float(torch.as_tensor(beta)) * b.to_dense().as_subclass(torch.Tensor)
        sp = dense.to_sparse_csr()
        return CSRTensor(sp.crow_indices().to(self.indptr.dtype), sp.col_indices().to(self.indices.dtype),
                         sp.values(), self.shape)

    def to_coo(self):
        return COOTensor(torch.stack([self._rows(), self.indices.long()], 1), self.values, self.shape)

    def to_dense(self):
        out = torch.zeros(self.shape, dtype=self.values.dtype, device=self.values.device)
        out.index_put_((self._rows(), self.indices.long()), self.values, accumulate=True)
        return Tensor(out)

    def to_tuple(self):
        return self.indptr, self.indices, self.values, self.shape

    def astype(self, dtype):
        return CSRTensor(self.indptr, self.indices, self.values.to(dtype), self.shape)

    def abs(self):
        return CSRTensor(self.indptr, self.indices, self.values.abs(), self.shape)

    def mv(self, dense_vector):
        v = torch.as_tensor(dense_vector).reshape(-1)
        prod = self.values * v[self.indices.long()]
        out = torch.zeros(self.shape[0], dtype=prod.dtype, device=prod.device)
        return Tensor(out.index_add_(0, self._rows(), prod).reshape(-1, 1))

    def mm(self, dense):
        d = torch.as_tensor(dense)
        prod = self.values.unsqueeze(-1) * d[self.indices.long()]
        out = torch.zeros(self.shape[0], d.shape[1], dtype=prod.dtype, device=prod.device)
        return Tensor(out.index_add_(0, self._rows(), prod))

    def sum(self, axis):
        if axis not in (1, -1):
            raise ValueError("CSRTensor.sum supports axis=1")
        out = torch.zeros(self.shape[0], dtype=self.values.dtype, device=self.values.device)
        return Tensor(out.index_add_(0, self._rows(), self.values).reshape(-1, 1))

    def __mul__(self, dense):
        d = torch.as_tensor(dense)
        if d.dim() == 0:
            return CSRTensor(self.indptr, self.indices, self.values * d, self.shape)
        picked = d.expand(self.shape)[self._rows(), self.indices.long()]
        return CSRTensor(self.indptr, self.indices, self.values * picked, self.shape)

    def __repr__(self):
        return "CSRTensor(shape=%s, dtype=%s, nnz=%d)" % (self.shape, self.dtype, self.size)


class RowTensor:
    """Rows ``indices`` of a dense tensor of ``dense_shape`` with their ``values`` (sparse gradient of an embedding)."""

    def __init__(self, indices=None, values=None, shape=None, row_tensor=None):
        if row_tensor is not None:
            indices, values, shape = row_tensor.indices, row_tensor.values, row_tensor.dense_shape
        self.indices = Tensor(torch.as_tensor(indices))
        self.values = Tensor(torch.as_tensor(values))
        self.dense_shape = tuple(int(s) for s in shape)

    def to_dense(self):
        out = torch.zeros(self.dense_shape, dtype=self.values.dtype, device=self.values.device)
        return Tensor(out.index_add_(0, self.indices.long().reshape(-1), self.values))

    def __repr__(self):
        return "RowTensor(dense_shape=%s, rows=%d)" % (self.dense_shape, self.indices.numel())


# ------------------------------------------------------------------------------------------------ function transforms
def vmap(fn, in_axes=0, out_axes=0):
    """Vectorising map over ``in_axes`` of the inputs (``None``: broadcast the argument)."""
    from ..ops.primitive import _wrap_out
    mapped = torch.func.vmap(lambda *a: fn(*a), in_dims=in_axes, out_dims=out_axes)

    @functools.wraps(fn)
    def run(*args):
        return _wrap_out(mapped(*args))
    return run


def hessian(fn, grad_position=0):
    from ..ops.composite import jacfwd, jacrev
    return jacfwd(jacrev(fn, grad_position), grad_position)


def get_grad(gradients, identifier):
    """Picks one gradient out of the result of ``grad(..., return_ids=True)``: by input position (int) or by
    Parameter."""
    def walk(g):
        if isinstance(g, (tuple, list)) and len(g) == 2 and not isinstance(g[0], (tuple, list)):
            return [g]
        out = []
        if isinstance(g, (tuple, list)):
            for x in g:
                out += walk(x)
        return out
    for key, value in walk(gradients):
        if isinstance(identifier, int) and key == identifier:
            return value
        if not isinstance(identifier, int) and key == getattr(identifier, "name", None):
            return value
    raise RuntimeError("Can not find the gradient for position or Parameter %r" % (identifier,))


def data_sink(fn, dataset, sink_size=1, jit_config=None, input_signature=None):
    """Returns a function that, per call, pulls ``sink_size`` batches from ``dataset`` and runs ``fn`` on each (the
    host loop the reference moves onto the device queue); the iterator restarts when the dataset is exhausted."""
    state = {"it": None}

    def run():
        out = None
        for _ in range(int(sink_size)):
            if state["it"] is None:
                state["it"] = iter(dataset.create_tuple_iterator())
            try:
                batch = next(state["it"])
            except StopIteration:
                state["it"] = iter(dataset.create_tuple_iterator())
                batch = next(state["it"])
            out = fn(*batch)
        return out
    return run


def ms_memory_recycle():
    """Drops compiled-graph caches and returns cached device memory to the driver."""
    gc.collect()
    if torch.cuda.is_available():
        torch.cuda.empty_cache()


def run_check():
    """Prints the version and checks that a small computation runs on the configured device."""
    from .. import __version__, context
    target = context.get_context("device_target")
    dev = "cuda" if target == "GPU" and torch.cuda.is_available() else "cpu"
    x = torch.ones(3, 3, device=dev)
    ok = bool(torch.allclose(x @ x, torch.full((3, 3), 3.0, device=dev)))
    print("MindSpore-B200 version: ", __version__)
    if ok:
        print("The result of multiplication calculation is correct, mindspore_b200 has been installed on platform "
              "[%s] successfully!" % target)
    else:
        raise RuntimeError("device check failed on %s" % dev)


# ------------------------------------------------------------------------------------------------ strategy-search knobs
_ALGO_DEFAULTS = {"fully_use_devices": True, "elementwise_op_strategy_follow": False, "enable_algo_approxi": False,
                  "algo_approxi_epsilon": 0.1, "tensor_slice_align_enable": False, "tensor_slice_align_size": 16}
_algo = dict(_ALGO_DEFAULTS)


def set_algo_parameters(**kwargs):
    for k, v in kwargs.items():
        if k not in _ALGO_DEFAULTS:
            raise ValueError("Set context keyword %s is not recognized!" % k)
        if not isinstance(v, type(_ALGO_DEFAULTS[k])) and not (isinstance(_ALGO_DEFAULTS[k], float) and isinstance(v, int)):
            raise TypeError("For 'set_algo_parameters', '%s' must be %s" % (k, type(_ALGO_DEFAULTS[k]).__name__))
        if k == "tensor_slice_align_size" and not 1 <= v <= 1024:
            raise ValueError("tensor_slice_align_size must be in [1, 1024]")
        _algo[k] = v


def get_algo_parameters(attr_key):
    if attr_key not in _algo:
        raise ValueError("Get context keyword %s is not recognized!" % attr_key)
    return _algo[attr_key]


from ..parallel.cost_model import (get_cost_model_context, reset_cost_model_context,  # noqa: E402,F401
                                   set_cost_model_context)


def reset_algo_parameters():
    _algo.clear()
    _algo.update(_ALGO_DEFAULTS)


def __getattr__(name):
    # the reference keeps jit / ms_function / ms_class / flops_collection in common.api; they live in graph.jit here
    if name in ("jit", "ms_function"):
        from ..graph import jit as _jit
        return getattr(_jit, name)
    if name == "ms_class":
        return jit_class
    if name == "flops_collection":
        from ..graph.flops import flops_collection
        return flops_collection
    raise AttributeError("module %r has no attribute %r" % (__name__, name))


COOTensor.itemsize = property(lambda self: self.values.element_size())
