"""``mindspore_b200.ops``: primitive classes, the functional API and composite operators."""
from . import composite, functional, operations
from .composite import (GradOperation, HyperMap, Map, MultitypeFuncGraph, Partial, clip_by_global_norm,
                        clip_by_value, grad, jacfwd, jacrev, jvp, stop_gradient, value_and_grad, vjp)
from .functional import *  # noqa: F401,F403
from .operations import *  # noqa: F401,F403
from . import function_ext as _function_ext
globals().update({_n: getattr(_function_ext, _n) for _n in _function_ext.__all__ if _n not in globals()})
from .primitive import (Primitive, PrimitiveWithCheck, PrimitiveWithInfer, constexpr, prim_attr_register)
from . import functional as F  # noqa: N812
from . import operations as P  # noqa: N812
from . import composite as C  # noqa: N812
from .composite import (Shard, UnpackCall, ZipOperation, choice_with_mask, count_nonzero, dot, gamma, laplace,  # noqa: E402,F401
                        poisson, repeat_elements, sequence_mask, tensor_dot, vmap)

from .op_info_register import (AiCPURegOp, AkgAscendRegOp, AkgGpuRegOp, CpuRegOp, CustomRegOp, DataType,  # noqa: E402,F401
                               TBERegOp, custom_info_register, get_vm_impl_fn, op_info_register, vm_impl_registry)


def reshard(tensor, layout):
    """Redistributes ``tensor`` to ``layout`` (a ``parallel.Layout`` with its tensor map applied): the dispatcher's
    redistribution - all-gather / slice / all-to-all as the two layouts require - inserted by hand at this point of
    the network (python/mindspore/ops/function/reshard_func.py).  Outside semi-auto / auto parallel mode, or for a
    tensor whose layout the dispatcher does not know, the tensor is taken as replicated."""
    from .. import context
    from ..parallel import spmd
    from ..parallel.layout import Layout, TensorLayout
    if not isinstance(layout, Layout):
        raise TypeError("Reshard only support type mindspore.Layout, but got %s" % type(layout))
    d = layout.to_dict()
    if len(d["tensor_map"]) != tensor.dim():
        raise ValueError("reshard: the layout has %d dims, the tensor %d" % (len(d["tensor_map"]), tensor.dim()))
    mode = context.get_auto_parallel_context("parallel_mode")
    if mode not in (context.ParallelMode.SEMI_AUTO_PARALLEL, context.ParallelMode.AUTO_PARALLEL):
        return tensor
    cur = spmd.get_layout(tensor)
    full = cur.shape if cur is not None else tuple(tensor.shape)
    need = TensorLayout(d["device_matrix"], d["tensor_map"], full)
    if cur is None:
        cur = TensorLayout(d["device_matrix"], (-1,) * tensor.dim(), full)
    out = spmd._redistribute(tensor, cur, need)
    return spmd.set_layout(_wrap_reshard(out), need)


def _wrap_reshard(t):
    from .primitive import _wrap_out
    return _wrap_out(t)


from .operations import _COMM_NAMES  # noqa: E402
_SPARSE_PREFIXES = ("coo_", "csr_", "make_", "row_tensor_", "dense_to_sparse_")
_SPARSE_NAMES = ("coo2csr", "csr2coo", "coalesce")


def __getattr__(name):
    # the sparse functions need common.api (COOTensor / CSRTensor), which itself imports ops: resolved on first use
    if name in _COMM_NAMES:
        # the communication primitives import the communication package, which imports ops: resolved on first use
        import importlib
        return getattr(importlib.import_module(__name__ + ".comm_ops"), name)
    if name.startswith(_SPARSE_PREFIXES) or name in _SPARSE_NAMES:
        import importlib
        mod = importlib.import_module(__name__ + ".sparse_func")
        if name in mod.__all__:
            return getattr(mod, name)
    raise AttributeError("module %r has no attribute %r" % (__name__, name))
