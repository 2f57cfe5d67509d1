"""``mindspore_b200.mint``: the torch-like functional / module namespace (python/mindspore/mint/__init__.py).
Functions take and return ``Tensor``; they are thin forwards to the tensor substrate, and ``mint.nn`` /
``mint.optim`` re-export the matching layers and optimizers."""
from __future__ import annotations

import types

import torch

from .common.tensor import as_tensor as _T


def _wrap(fn):
    def f(*args, **kwargs):
        out = fn(*args, **kwargs)
        if isinstance(out, torch.Tensor):
            return _T(out)
        if isinstance(out, tuple):
            return tuple(_T(o) if isinstance(o, torch.Tensor) else o for o in out)
        return out
    f.__name__ = getattr(fn, "__name__", "fn")
    f.__doc__ = "Forward of torch.%s returning framework tensors." % f.__name__
    return f


_NAMES = """abs add all any arange argmax argmin baddbmm bmm cat ceil chunk clamp cos cosh cumsum div eq erf exp
flatten flip floor gather ge greater gt index_select isclose isfinite le less log log1p logical_and logical_not
logical_or lt matmul max maximum mean min minimum mul ne neg nonzero normal ones ones_like permute pow prod rand
rand_like reciprocal repeat_interleave reshape rsqrt scatter_add searchsorted sigmoid sign sin sinh softmax sort
split sqrt square squeeze stack sub sum tanh tile topk tril triu unique unsqueeze where zeros zeros_like narrow
broadcast_to cumprod atan2 tan asin acos atan erfinv logsumexp roll median var std isnan isinf linspace eye full
full_like masked_select nan_to_num remainder fmod round trunc bitwise_and bitwise_or bitwise_xor outer einsum""".split()

for _n in _NAMES:
    if hasattr(torch, _n):
        globals()[_n] = _wrap(getattr(torch, _n))
concat = _wrap(torch.cat)
greater_equal = _wrap(torch.ge)
less_equal = _wrap(torch.le)
not_equal = _wrap(torch.ne)
divide = _wrap(torch.div)
multiply = _wrap(torch.mul)
subtract = _wrap(torch.sub)
negative = _wrap(torch.neg)
absolute = _wrap(torch.abs)
for _n in """addbmm addmm addmv clone randn randn_like randint randint_like randperm transpose swapaxes t mm mv dot
cross diag trace kron argsort bincount cummax cummin diff count_nonzero histc kthvalue msort nansum amax amin
aminmax allclose equal exp2 expm1 log2 log10 logaddexp hypot floor_divide true_divide ldexp lerp frac xlogy sinc
deg2rad rad2deg asinh acosh atanh bernoulli multinomial empty empty_like arange meshgrid tensor_split hsplit vsplit
dsplit unbind movedim squeeze unflatten triu_indices tril_indices select index_add scatter masked_fill take
take_along_dim clamp_min clamp_max logical_xor bitwise_not floor_divide isreal signbit heaviside""".split():
    if hasattr(torch, _n) and _n not in globals():
        globals()[_n] = _wrap(getattr(torch, _n))
special = types.ModuleType("mindspore_b200.mint.special")
for _n in ("erfc", "expm1", "exp2", "round", "sinc", "log1p", "log_softmax", "digamma", "gammaln", "erfinv", "i0",
           "i0e", "i1", "i1e", "logit", "expit", "xlogy", "zeta", "bessel_j0", "bessel_j1", "ndtr", "ndtri", "entr"):
    if hasattr(torch.special, _n):
        setattr(special, _n, _wrap(getattr(torch.special, _n)))
distributed = types.ModuleType("mindspore_b200.mint.distributed")


def _fill_distributed():
    from .communication import comm_func as _cf
    from .communication import management as _m
    distributed.init_process_group = lambda backend="nccl", **kw: _m.init(backend if backend != "hccl" else None)
    distributed.destroy_process_group = lambda group=None: _m.release()
    distributed.get_rank = _m.get_rank
    distributed.get_world_size = _m.get_group_size
    distributed.new_group = lambda ranks=None, **kw: (_m.create_group(_m.stage_rank_list_name(ranks), list(ranks)),
                                                     _m.stage_rank_list_name(ranks))[1]
    distributed.get_backend = lambda group=None: _m.GlobalComm.BACKEND
    for _name in ("all_reduce", "all_gather_into_tensor", "reduce_scatter_tensor", "reduce", "broadcast", "barrier",
                  "isend", "irecv", "batch_isend_irecv", "scatter_tensor", "gather_into_tensor"):
        if hasattr(_cf, _name):
            setattr(distributed, _name, getattr(_cf, _name))
    distributed.P2POp = getattr(_cf, "P2POp", None)

nn = types.ModuleType("mindspore_b200.mint.nn")
optim = types.ModuleType("mindspore_b200.mint.optim")
linalg = types.ModuleType("mindspore_b200.mint.linalg")
linalg.norm = _wrap(torch.linalg.norm)
linalg.inv = _wrap(torch.linalg.inv)
for _n in ("det", "slogdet", "qr", "svd", "eigh", "eig", "cholesky", "solve", "lstsq", "pinv", "matrix_norm",
           "vector_norm", "matrix_rank", "cross", "matrix_power", "cond", "vander"):
    if hasattr(torch.linalg, _n):
        setattr(linalg, _n, _wrap(getattr(torch.linalg, _n)))


def _fill_submodules():
    from . import nn as _nn
    for name in ("Linear", "Dropout", "Embedding", "LayerNorm", "GroupNorm", "ReLU", "GELU", "SiLU", "Sigmoid", "Tanh",
                 "Softmax", "LogSoftmax", "Conv2d", "BatchNorm2d", "MaxPool2d", "AvgPool2d", "CrossEntropyLoss",
                 "MSELoss", "L1Loss", "BCEWithLogitsLoss", "Identity", "Flatten", "Cell", "CellList",
                 "SequentialCell"):
        if hasattr(_nn, name):
            setattr(nn, name, getattr(_nn, name))
    if not hasattr(nn, "Linear") and hasattr(_nn, "Dense"):
        nn.Linear = _nn.Dense
    functional = types.ModuleType("mindspore_b200.mint.nn.functional")
    for name in ("relu", "gelu", "silu", "softmax", "log_softmax", "dropout", "layer_norm", "linear", "embedding",
                 "cross_entropy", "mse_loss", "l1_loss", "sigmoid", "tanh", "one_hot", "pad", "max_pool2d",
                 "avg_pool2d", "batch_norm", "group_norm", "normalize", "softplus", "leaky_relu", "elu",
                 "binary_cross_entropy_with_logits", "interpolate", "unfold", "fold", "grid_sample",
                 "binary_cross_entropy", "conv_transpose2d", "conv2d", "max_unpool2d", "hardswish", "hardsigmoid",
                 "mish", "prelu", "selu", "softshrink", "hardshrink", "logsigmoid", "adaptive_avg_pool2d"):
        if hasattr(torch.nn.functional, name):
            setattr(functional, name, _wrap(getattr(torch.nn.functional, name)))
    nn.functional = functional
    optim.AdamW = _nn.AdamWeightDecay
    optim.Adam = _nn.Adam
    optim.SGD = _nn.SGD
    for name in ("Fold", "Unfold", "PixelShuffle", "Conv3d", "ConvTranspose2d", "L1Loss", "Softplus", "ELU", "PReLU",
                 "LeakyReLU", "Hardtanh", "GLU", "AdaptiveAvgPool2d", "AdaptiveMaxPool2d", "Upsample"):
        if hasattr(_nn, name) and not hasattr(nn, name):
            setattr(nn, name, getattr(_nn, name))
    if hasattr(_nn, "Conv2dTranspose"):
        nn.ConvTranspose2d = _nn.Conv2dTranspose
    _fill_distributed()
    globals()["functional"] = functional


_fill_submodules()

arctan2 = _wrap(torch.arctan2)
inverse = _wrap(torch.linalg.inv)



def _register_submodules():
    import sys
    for m in (special, distributed, nn, optim, linalg, functional):
        sys.modules.setdefault(m.__name__, m)
    globals().setdefault("__path__", [])                  # `import mindspore_b200.mint.nn.functional` resolves
    nn.__dict__.setdefault("__path__", [])


_register_submodules()
