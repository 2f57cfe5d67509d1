"""``nn.Cell``: the module base class.

Attribute assignment registers ``Parameter`` and child ``Cell`` objects; ``__call__`` runs
``construct`` eagerly in PYNATIVE mode and, in GRAPH mode, compiles the outermost cell once per
input signature (trace -> passes -> auto-parallel -> executor) and replays the compiled graph.

Parity: mindspore/python/mindspore/nn/cell.py:110 (class), :685-723 (__call__), :841 (__setattr__),
:1045-1074 (compile / compile_and_run), :574 (shard), :1246-1503 (parameter APIs), :1819 (to_float),
:1887 (set_grad), :1903 (set_train), :2301 (set_comm_fusion), :2373 (recompute), :318 (pipeline_stage).
"""
from __future__ import annotations

from collections import OrderedDict

import torch

from .. import context
from ..common import dtype as mstype
from ..common.parameter import Parameter, ParameterTuple
from ..common.tensor import Tensor


class Cell:
    _graph_depth = 0  # >0 while some outer Cell is already executing (nested calls run inline)

    def __init__(self, auto_prefix=True, flags=None):
        object.__setattr__(self, "_params", OrderedDict())
        object.__setattr__(self, "_cells", OrderedDict())
        object.__setattr__(self, "_params_list", OrderedDict())
        self.training = False
        self.requires_grad = False
        self._auto_prefix = auto_prefix
        self._param_prefix = ""
        self._phase = "train"
        self._forward_pre_hook = OrderedDict()
        self._forward_hook = OrderedDict()
        self._backward_hook = OrderedDict()
        self._cell_tag = None
        self._scope = None
        self._mixed_precision_type = None
        self._to_float_dtype = None
        self._pipeline_stage = None
        self._recompute = False
        self._recompute_kwargs = {}
        self._shard_fn = None
        self._in_strategy = None
        self._out_strategy = None
        self._jit_config = None
        self._compiled = {}
        self._use_graph = None
        self._has_config_recompute = False
        self.parameter_layout_dict = {}
        self.parallel_parameter_name_list = []
        self.cls_name = self.__class__.__name__
        self._attrs = {}
        if flags:
            self.add_flags(**flags)

    # ------------------------------------------------------------------ attribute interception
    def __setattr__(self, name, value):
        params = self.__dict__.get("_params")
        cells = self.__dict__.get("_cells")
        if isinstance(value, Parameter):
            if params is None:
                raise AttributeError("Can not assign params before Cell.__init__() call.")
            if name in self.__dict__:
                del self.__dict__[name]
            if cells is not None and name in cells:
                raise TypeError("For 'Cell', the %r must be Cell, but got Parameter." % name)
            if value.name == "Parameter" or not value.name:
                value.name = name
            params[name] = value
        elif isinstance(value, Cell):
            if cells is None:
                raise AttributeError("Can not assign cells before Cell.__init__() call.")
            if name in self.__dict__:
                del self.__dict__[name]
            if params is not None and name in params:
                raise TypeError("For 'Cell', the %r must be Parameter, but got Cell." % name)
            if self._auto_prefix:
                value.update_parameters_name(name + ".")
            cells[name] = value
        elif isinstance(value, ParameterTuple):
            self._params_list[name] = value
            object.__setattr__(self, name, value)
        elif params is not None and name in params:
            if value is None:
                params[name] = None
            elif isinstance(value, torch.Tensor):
                params[name].set_data(value)
            else:
                raise TypeError("For 'Cell', the %r must be Parameter or Tensor, but got %s" % (name, type(value)))
        elif cells is not None and name in cells:
            if value is not None:
                raise TypeError("For 'Cell', the %r must be Cell or None, but got %s" % (name, type(value)))
            cells[name] = None
        else:
            object.__setattr__(self, name, value)

    def __getattr__(self, name):
        d = self.__dict__
        if "_params" in d and name in d["_params"]:
            return d["_params"][name]
        if "_cells" in d and name in d["_cells"]:
            return d["_cells"][name]
        raise AttributeError("The '%s' object has no attribute '%s'." % (type(self).__name__, name))

    def __delattr__(self, name):
        if name in self._params:
            del self._params[name]
        elif name in self._cells:
            del self._cells[name]
        else:
            object.__delattr__(self, name)

    def __repr__(self):
        extra = self.extend_repr()
        lines = []
        for k, c in self._cells.items():
            sub = repr(c).replace("\n", "\n  ")
            lines.append("(%s): %s" % (k, sub))
        body = extra
        if lines:
            body += ("\n  " if not extra else "\n  ") + "\n  ".join(lines) + "\n"
        return "%s<%s>" % (type(self).__name__, body)

    def extend_repr(self):
        return ""

    # ------------------------------------------------------------------ call
    def construct(self, *inputs, **kwargs):
        raise NotImplementedError("%s must implement construct()" % type(self).__name__)

    def _cast_inputs(self, inputs):
        dt = self._to_float_dtype
        if dt is None:
            return inputs
        return tuple(x.to(dt) if isinstance(x, torch.Tensor) and x.is_floating_point() and x.dtype != dt else x
                     for x in inputs)

    def _run_construct(self, inputs, kwargs):
        for hook in self._forward_pre_hook.values():
            res = hook(self, inputs)
            if res is not None:
                inputs = res if isinstance(res, tuple) else (res,)
        inputs = self._cast_inputs(inputs)
        if self._recompute and torch.is_grad_enabled() and Cell._recompute_enabled:
            from torch.utils.checkpoint import checkpoint
            out = checkpoint(lambda *a: self.construct(*a, **kwargs), *inputs, use_reentrant=False)
        else:
            construct = self.construct
            if Cell._graph_depth > 0:
                from ..graph.ast_transform import converted_construct
                construct = converted_construct(self)          # data-dependent ifs become Switch nodes
            out = construct(*inputs, **kwargs)
        for hook in self._forward_hook.values():
            res = hook(self, inputs, out)
            if res is not None:
                out = res
        if self._backward_hook and isinstance(out, torch.Tensor) and out.requires_grad:
            hooks = list(self._backward_hook.values())
            cell = self

            def _bw(grad):
                g = grad
                for h in hooks:
                    r = h(cell, g, g)
                    if r is not None:
                        g = r[0] if isinstance(r, tuple) else r
                return g
            out.register_hook(_bw)
        return out

    _recompute_enabled = True

    # set by parallel.pipeline while a pipeline stage runs: callable(cell, inputs, kwargs) deciding whether a
    # cell tagged with ``pipeline_stage`` runs here, is skipped, or ends this stage's part of the forward pass
    _stage_hook = None

    def __call__(self, *inputs, **kwargs):
        if Cell._stage_hook is not None and self._pipeline_stage is not None:
            return Cell._stage_hook(self, inputs, kwargs)
        return self._call_impl(inputs, kwargs)

    def _call_impl(self, inputs, kwargs):
        from ..graph import tracer as _tracer
        if Cell._graph_depth > 0 or _tracer.is_tracing():
            return self._run_construct(inputs, kwargs)
        use_graph = context.get_context("mode") == context.GRAPH_MODE and self._use_graph is not False
        Cell._graph_depth += 1
        try:
            if use_graph:
                from ..graph import jit as _jit
                return _jit.compile_and_run_cell(self, inputs, kwargs)
            return self._run_construct(inputs, kwargs)
        finally:
            Cell._graph_depth -= 1

    def compile(self, *inputs, **kwargs):
        from ..graph import jit as _jit
        return _jit.compile_cell(self, inputs, kwargs)

    def compile_and_run(self, *inputs, **kwargs):
        from ..graph import jit as _jit
        return _jit.compile_and_run_cell(self, inputs, kwargs)

    def set_inputs(self, *inputs, **kwargs):
        self._dynamic_inputs = inputs

    def get_inputs(self):
        return getattr(self, "_dynamic_inputs", None)

    def infer_outputs(self, *inputs):
        """Abstract outputs (shapes with symbolic dimensions, dtypes) of ``construct`` for abstract / placeholder
        inputs, without running a kernel; the ``set_inputs`` declaration when no inputs are given."""
        from ..graph.abstract import infer
        if not inputs:
            inputs = getattr(self, "_dynamic_inputs", None) or ()
        return infer(lambda *a: self._run_construct(a, {}), *inputs)

    def set_jit_config(self, jit_config):
        self._jit_config = jit_config

    # ------------------------------------------------------------------ hierarchy
    def insert_param_to_cell(self, param_name, param, check_name_contain_dot=True):
        if not param_name:
            raise KeyError("The name of parameter should not be null.")
        if check_name_contain_dot and "." in param_name:
            raise KeyError("The name of parameter should not contain \".\"")
        if "_params" not in self.__dict__:
            raise AttributeError("You need call init() first.")
        if hasattr(self, param_name) and param_name not in self._params:
            raise KeyError("Duplicated parameter name '%s'." % param_name)
        if not isinstance(param, Parameter) and param is not None:
            raise TypeError("The type of parameter should be 'Parameter' if not None.")
        if isinstance(param, Parameter) and param.name == "Parameter":
            param.name = param_name
        self._params[param_name] = param

    def insert_child_to_cell(self, child_name, child_cell):
        if not isinstance(child_cell, Cell) and child_cell is not None:
            raise TypeError("Child cell type is incorrect.")
        if not child_name or "." in child_name:
            raise KeyError("Child cell name is incorrect.")
        if hasattr(self, child_name) and child_name not in self._cells:
            raise KeyError("Duplicate child name '%s'." % child_name)
        self._cells[child_name] = child_cell

    def cells(self):
        return self._cells.values()

    def name_cells(self):
        return OrderedDict((k, v) for k, v in self._cells.items() if v is not None)

    def cells_and_names(self, cells=None, name_prefix=""):
        seen = cells if cells is not None else set()
        if id(self) in seen:
            return
        seen.add(id(self))
        yield name_prefix, self
        for name, cell in self._cells.items():
            if cell is None:
                continue
            pre = name if not name_prefix else name_prefix + "." + name
            yield from cell.cells_and_names(seen, pre)

    def update_parameters_name(self, prefix="", recurse=True):
        for _, p in self.parameters_and_names(expand=recurse):
            p.name = prefix + p.name
            p.is_init = False

    def _param_walk(self, prefix="", expand=True, seen=None):
        seen = seen if seen is not None else set()
        for name, p in self._params.items():
            if p is not None and id(p) not in seen:
                seen.add(id(p))
                yield (prefix + name, p)
        for _, plist in self._params_list.items():
            for p in plist:
                if id(p) not in seen:
                    seen.add(id(p))
                    yield (p.name, p)
        if expand:
            for cname, cell in self._cells.items():
                if cell is not None:
                    yield from cell._param_walk(prefix + cname + ".", expand, seen)

    def parameters_and_names(self, name_prefix="", expand=True):
        yield from self._param_walk(name_prefix + "." if name_prefix else "", expand)

    def get_parameters(self, expand=True):
        for _, p in self.parameters_and_names(expand=expand):
            yield p

    def parameters_dict(self, recurse=True):
        out = OrderedDict()
        for _, p in self.parameters_and_names(expand=recurse):
            out[p.name] = p
        return out

    def trainable_params(self, recurse=True):
        return [p for p in self.get_parameters(expand=recurse) if p._ms_requires_grad]

    def untrainable_params(self, recurse=True):
        return [p for p in self.get_parameters(expand=recurse) if not p._ms_requires_grad]

    def parameters_broadcast_dict(self, recurse=True):
        return OrderedDict((p.name, p) for p in self.get_parameters(expand=recurse) if not p.layerwise_parallel)

    def init_parameters_data(self, auto_parallel_mode=False):
        replace = {}
        for p in self.get_parameters():
            layout = self.parameter_layout_dict.get(p.name) if auto_parallel_mode else None
            p.init_data(layout, set_sliced=layout is not None)
        return replace

    def load_parameter_slice(self, params):
        return None

    # ------------------------------------------------------------------ modes and flags
    def set_train(self, mode=True):
        self._phase = "train" if mode else "predict"
        for _, c in self.cells_and_names():
            c.training = mode
        return self

    def set_grad(self, requires_grad=True):
        for _, c in self.cells_and_names():
            c.requires_grad = requires_grad
        return self

    def set_data_parallel(self):
        self.add_flags(defer_inline=True)

    @property
    def phase(self):
        return self._phase

    @phase.setter
    def phase(self, v):
        self._phase = v

    def add_flags(self, **flags):
        self._attrs.update(flags)
        for k, v in flags.items():
            object.__setattr__(self, "_flag_" + k, v)
        return self

    def add_flags_recursive(self, **flags):
        for _, c in self.cells_and_names():
            c.add_flags(**flags)
        return self

    def get_flags(self):
        return dict(self._attrs)

    def to_float(self, dst_type):
        """Marks this subtree to compute in ``dst_type``: float inputs are cast on entry and the
        subtree's floating parameters are held in that dtype (fp32 master copies are the optimizer's job)."""
        if dst_type not in (mstype.float16, mstype.float32, mstype.bfloat16):
            raise ValueError("For 'to_float', the argument 'dst_type' must be float16, float32 or bfloat16, got %s"
                             % (dst_type,))
        for _, c in self.cells_and_names():
            c._to_float_dtype = dst_type
            for p in c._params.values():
                if p is not None and p.is_floating_point() and p.dtype != dst_type and \
                        not getattr(c, "_keep_fp32_params", False):
                    p.set_data(p.detach().as_subclass(torch.Tensor).to(dst_type))
        return self

    def set_boost(self, boost_type):
        self._boost_type = boost_type
        return self

    def set_comm_fusion(self, fusion_type, recurse=True):
        for p in self.trainable_params(recurse):
            p.comm_fusion = fusion_type
        return self

    def set_broadcast_flag(self, mode=True):
        self.add_flags(broadcast_flag=mode)
        return self

    def set_auto_parallel(self):
        self._auto_parallel = True

    # ------------------------------------------------------------------ parallel annotations
    def shard(self, in_strategy, out_strategy=None, parameter_plan=None, device="Ascend", level=0):
        from ..parallel.shard import Shard
        fn = Shard()(self, in_strategy, out_strategy, parameter_plan, device, level)
        self._shard_fn = fn
        self._in_strategy, self._out_strategy = in_strategy, out_strategy
        return fn

    @property
    def pipeline_stage(self):
        return self._pipeline_stage

    @pipeline_stage.setter
    def pipeline_stage(self, value):
        if not isinstance(value, int) or isinstance(value, bool):
            raise TypeError("For 'Cell', the property 'pipeline_stage' must be int type, but got %s" % type(value))
        if value < 0:
            raise ValueError("For 'Cell', the property 'pipeline_stage' can not be less than 0, but got %d" % value)
        self._pipeline_stage = value
        for p in self.trainable_params():
            p.add_pipeline_stage(value)

    def recompute(self, **kwargs):
        """Activation checkpointing for this cell (mp_comm_recompute, parallel_optimizer_comm_recompute,
        recompute_slice_activation accepted like the reference, nn/cell.py:2373)."""
        for k in kwargs:
            if k not in ("mp_comm_recompute", "parallel_optimizer_comm_recompute", "recompute_slice_activation",
                         "mode"):
                raise ValueError("For 'recompute', keyword %r is not recognized" % k)
        self._recompute = kwargs.pop("mode", True)
        self._recompute_kwargs = kwargs
        self._has_config_recompute = True
        if "parallel_optimizer_comm_recompute" in kwargs:
            for p in self.trainable_params():
                p.parallel_optimizer_comm_recompute = kwargs["parallel_optimizer_comm_recompute"]
        return self

    def place(self, role, rank_id):
        """Pins this cell to process ``rank_id`` of ``role`` for MPMD execution (``parallel.mpmd.run_placed``)."""
        if role not in ("MS_WORKER", "MS_SERVER", "MS_SCHED", "MS_PSERVER"):
            raise ValueError("For 'Cell.place', 'role' must be MS_WORKER, MS_SERVER, MS_SCHED or MS_PSERVER, got %r"
                             % (role,))
        if not isinstance(rank_id, int) or isinstance(rank_id, bool) or rank_id < 0:
            raise ValueError("For 'Cell.place', 'rank_id' must be a non-negative int, got %r" % (rank_id,))
        self.add_flags(ms_role=role, rank_id=rank_id)
        object.__setattr__(self, "_placement", (role, rank_id))
        return self

    # ------------------------------------------------------------------ hooks
    def register_forward_pre_hook(self, hook_fn):
        return _HookHandle(self._forward_pre_hook, hook_fn)

    def register_forward_hook(self, hook_fn):
        return _HookHandle(self._forward_hook, hook_fn)

    def register_backward_hook(self, hook_fn):
        return _HookHandle(self._backward_hook, hook_fn)

    def register_backward_pre_hook(self, hook_fn):
        """``hook_fn(cell, grad_output)`` runs before the cell's backward; it may return a replacement gradient."""
        return _HookHandle(self._backward_hook, lambda cell, gin, gout: hook_fn(cell, gout))

    def register_state_dict_post_hook(self, hook_fn):
        hooks = self.__dict__.setdefault("_state_dict_hooks", OrderedDict())
        return _HookHandle(hooks, hook_fn)

    def register_load_state_dict_post_hook(self, hook_fn):
        hooks = self.__dict__.setdefault("_load_state_dict_hooks", OrderedDict())
        return _HookHandle(hooks, hook_fn)

    # ------------------------------------------------------------------ torch-style state access (mint / experimental)
    def state_dict(self):
        out = OrderedDict((p.name, p) for p in self.get_parameters())
        for h in self.__dict__.get("_state_dict_hooks", {}).values():
            r = h(self, out)
            out = r if r is not None else out
        return out

    def load_state_dict(self, state_dict, strict=True):
        own = {p.name: p for p in self.get_parameters()}
        missing = [k for k in own if k not in state_dict]
        unexpected = [k for k in state_dict if k not in own]
        if strict and (missing or unexpected):
            raise RuntimeError("load_state_dict: missing keys %s, unexpected keys %s" % (missing, unexpected))
        import torch as _torch
        with _torch.no_grad():
            for k, p in own.items():
                if k in state_dict:
                    src = _torch.as_tensor(state_dict[k]).reshape(p.shape)
                    p.copy_(src.to(p.dtype))
                    from ..common.parameter import sync_master
                    sync_master(p, src)
        for h in self.__dict__.get("_load_state_dict_hooks", {}).values():
            h(self, (missing, unexpected))
        return missing, unexpected

    def named_parameters(self, name_prefix="", recurse=True):
        return self.parameters_and_names(name_prefix)

    def parameters(self, recurse=True):
        return self.get_parameters()

    def train(self, mode=True):
        return self.set_train(mode)

    def eval(self):
        return self.set_train(False)

    # ------------------------------------------------------------------ misc
    @property
    def param_prefix(self):
        return getattr(self, "_param_prefix", "")

    @property
    def create_time(self):
        """Nanosecond timestamp taken when this property (or the compile cache key) first needed it."""
        t = self.__dict__.get("_create_time")
        if t is None:
            import time as _time
            t = _time.time_ns()
            object.__setattr__(self, "_create_time", t)
        return t

    @property
    def pipeline_segment(self):
        return self.__dict__.get("_pipeline_segment", -1)

    @pipeline_segment.setter
    def pipeline_segment(self, value):
        if not isinstance(value, int) or isinstance(value, bool):
            raise TypeError("'pipeline_segment' must be int type, but got type : %s" % type(value))
        if value < 0:
            raise ValueError("'pipeline_segment' can not be less than 0, but got %d" % value)
        object.__setattr__(self, "_pipeline_segment", value)

    @property
    def parallel_parameter_merge_net_dict(self):
        return self.__dict__.setdefault("_parallel_parameter_merge_net_dict", {})

    @parallel_parameter_merge_net_dict.setter
    def parallel_parameter_merge_net_dict(self, value):
        if not isinstance(value, dict):
            raise TypeError("'parallel_parameter_merge_net_dict' must be dict type, but got %s" % type(value))
        object.__setattr__(self, "_parallel_parameter_merge_net_dict", value)

    @property
    def jit_config_dict(self):
        return self.__dict__.get("_jit_config_dict", {})

    def set_parallel_input_with_inputs(self, *inputs):
        from ..utils.log import logger
        logger.warning("'set_parallel_input_with_inputs' function is deprecated.")

    def auto_parallel_compile_and_run(self):
        from ..utils.log import logger
        logger.warning("'auto_parallel_compile_and_run' function is deprecated.")
        return False

    def check_names_and_refresh_name(self):
        """Parameter names must be unique within a network; raises otherwise."""
        names = [p.name for _, p in self.parameters_and_names()]
        dup = sorted({n for n in names if names.count(n) > 1})
        if dup:
            raise ValueError("The value of parameter names %s duplicate; parameter names must be unique" % dup)

    def set_param_fl(self, push_to_server=False, pull_from_server=False, requires_aggr=True):
        """Federated-learning flags on every parameter of the cell."""
        for p in self.get_parameters():
            p.set_param_fl(push_to_server, pull_from_server, requires_aggr)

    @property
    def bprop_debug(self):
        return getattr(self, "_bprop_debug", False)

    @bprop_debug.setter
    def bprop_debug(self, value):
        object.__setattr__(self, "_bprop_debug", bool(value))

    @property
    def cell_init_args(self):
        return getattr(self, "_cell_init_args", type(self).__name__)

    def get_scope(self):
        return getattr(self, "_scope", None)

    def generate_scope(self):
        """Scope names (``Default/<attr>-<Class>``) for this cell's children, used in graph dumps."""
        base = self.get_scope() or "Default"
        for name, cell in self._cells.items():
            if cell is not None:
                object.__setattr__(cell, "_scope", "%s/%s-%s" % (base, name, type(cell).__name__))
                cell.generate_scope()

    def update_cell_prefix(self):
        for name, cell in self.cells_and_names():
            object.__setattr__(cell, "_param_prefix", name)

    def update_cell_type(self, cell_type):
        object.__setattr__(self, "cell_type", cell_type)

    def check_names(self):
        seen = set()
        for _, p in self.parameters_and_names():
            if p.name in seen:
                raise ValueError("The value of %s is duplicated in this cell: parameter names must be unique" % p.name)
            seen.add(p.name)

    def cast_inputs(self, inputs, dst_type):
        import torch as _torch
        return tuple(x.to(dst_type) if isinstance(x, _torch.Tensor) and x.is_floating_point() else x for x in inputs)

    def auto_cast_inputs(self, inputs):
        dt = getattr(self, "_mixed_precision_type", None)
        return self.cast_inputs(inputs, dt) if dt is not None else tuple(inputs)

    def run_construct(self, cast_inputs, kwargs):
        return self._run_construct(tuple(cast_inputs), kwargs or {})

    def infer_param_pipeline_stage(self):
        """Parameters that belong to this process's pipeline stage."""
        from .. import context as _ctx
        stages = _ctx.get_auto_parallel_context("pipeline_stages")
        if stages <= 1:
            return list(self.get_parameters())
        per = max(1, _ctx.get_auto_parallel_context("device_num") // stages)
        mine = _ctx.get_auto_parallel_context("global_rank") // per
        out = []
        for _, cell in self.cells_and_names():
            st = getattr(cell, "_pipeline_stage", None)
            if st is None or st == mine:
                out += [p for p in cell._params.values() if p is not None]
        return out

    def remove_redundant_parameters(self):
        """Drops parameters of cells that belong to other pipeline stages (their memory is freed)."""
        keep = {id(p) for p in self.infer_param_pipeline_stage()}
        for _, cell in self.cells_and_names():
            for name in [n for n, p in cell._params.items() if p is not None and id(p) not in keep]:
                del cell._params[name]

    def set_param_ps(self, recurse=True, init_in_server=False):
        for p in (self.get_parameters() if recurse else self._params.values()):
            if p is not None:
                p.set_param_ps(init_in_server)

    def get_func_graph_proto(self):
        """Text of the compiled graph of this cell (empty before the first graph-mode call)."""
        cg = getattr(self, "_compiled_graph", None)
        return cg.fg.to_text() if cg is not None and hasattr(cg, "fg") else ""

    def cast_param(self, param):
        return param

    def flatten_weights(self, fusion_size=0):
        return None

    def exec_checkpoint_graph(self):
        return None

    def apply(self, fn):
        for c in self.cells():
            if c is not None:
                c.apply(fn)
        fn(self)
        return self


class _HookHandle:
    _next = 0

    def __init__(self, table, fn):
        self.table = table
        self.key = _HookHandle._next
        _HookHandle._next += 1
        table[self.key] = fn

    def remove(self):
        self.table.pop(self.key, None)


class GraphCell(Cell):
    """Runs a compiled / loaded graph (``load()`` result) as a Cell.  Parity: nn/cell.py:2554."""

    def __init__(self, graph, params_init=None, obf_random_seed=None):
        super().__init__(auto_prefix=True)
        self.graph = graph
        self._use_graph = False
        for name, p in getattr(graph, "params", {}).items():     # the weights of the file train like a cell's own
            self.insert_param_to_cell(name, p, check_name_contain_dot=False)
        if params_init:
            for name, value in params_init.items():
                graph.set_param(name, value)

    def construct(self, *inputs):
        return self.graph(*inputs)
