from . import dtype
from .dtype import *  # noqa: F401,F403
from . import initializer  # noqa: F401  (the module: `common.initializer.Normal`, `common.initializer.initializer`)
from .parameter import Parameter, ParameterTuple
from .seed import get_seed, set_seed
from .tensor import Tensor, as_tensor
from . import tensor_ext  # noqa: E402,F401  (attaches the MindSpore-only Tensor methods)


# ---- names the reference exposes from `mindspore.common` as well as from the top level
_FROM_API = {"COOTensor": "COOTensor", "CSRTensor": "CSRTensor", "RowTensor": "RowTensor", "Symbol": "Symbol",
             "jit_class": "jit_class", "ms_class": "jit_class", "lazy_inline": "lazy_inline",
             "ms_memory_recycle": "ms_memory_recycle", "mutable": "mutable", "no_inline": "no_inline",
             "recompute": "recompute", "SparseTensor": "COOTensor", "RowTensorInner": "RowTensor",
             "_no_grad": "_no_grad", "_null": "_null", "_NullType": "_NullType", "flops_collection": "flops_collection"}


from .jit_config import JitConfig  # noqa: E402,F401


def __getattr__(name):
    # resolved lazily: these live in modules that import `common` themselves
    if name in _FROM_API:
        from . import api as _api
        return getattr(_api, _FROM_API[name])
    if name in ("jit", "ms_function"):
        from ..graph import jit as _jit
        return _jit.jit
    if name in ("load_mindir", "save_mindir"):
        from ..train import serialization as _ser
        return _ser.load if name == "load_mindir" else _ser.export
    if name == "set_dump":
        from ..utils.dump import set_dump
        return set_dump
    raise AttributeError("module 'common' has no attribute %r" % name)
