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

nn = types.ModuleType("mindspore_b200.mint.nn")
optim = types.ModuleType("mindspore_b200.mint.optim")
linalg = types.ModuleType("mindspore_b200.mint.linalg")
linalg.norm = _wrap(torch.linalg.norm)
linalg.inv = _wrap(torch.linalg.inv)


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
                 "binary_cross_entropy_with_logits", "interpolate", "unfold", "fold", "grid_sample"):
        if hasattr(torch.nn.functional, name):
            setattr(functional, name, _wrap(getattr(torch.nn.functional, name)))
    nn.functional = functional
    optim.AdamW = _nn.AdamWeightDecay
    optim.Adam = _nn.Adam
    optim.SGD = _nn.SGD


_fill_submodules()
