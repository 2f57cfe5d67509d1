"""Layers: Dense, convolutions, normalisation, embedding, dropout, activations, pooling, containers,
recurrent layers.

Parity: mindspore/python/mindspore/nn/layer/{basic,conv,normalization,embedding,activation,pooling,
container,rnns}.py.  Hot layers (Dense, LayerNorm, RMSNorm, Embedding, GELU/SiLU, Conv2d, BatchNorm2d)
route to the sm_100a kernels through ``ops.fused`` / ``ops.conv`` for CUDA bf16 tensors.
"""
from __future__ import annotations

import math
from collections import OrderedDict

import torch
import torch.nn.functional as F

from ..common import dtype as mstype
from ..common.initializer import HeUniform, Uniform, initializer
from ..common.parameter import Parameter
from ..common.tensor import Tensor
from ..ops import conv as _conv
from ..ops import fused
from ..ops import operations as P
from ..ops.primitive import _wrap_out
from .cell import Cell


# ------------------------------------------------------------------------------------ activations
def _act_cell(name, fn, doc=None):
    def construct(self, x):
        return _wrap_out(fn(x))
    return type(name, (Cell,), {"construct": construct, "__doc__": doc or name})


ReLU = _act_cell("ReLU", torch.relu)
ReLU6 = _act_cell("ReLU6", F.relu6)
Sigmoid = _act_cell("Sigmoid", torch.sigmoid)
Tanh = _act_cell("Tanh", torch.tanh)
SiLU = _act_cell("SiLU", F.silu)
Mish = _act_cell("Mish", F.mish)
HSwish = _act_cell("HSwish", F.hardswish)
HSigmoid = _act_cell("HSigmoid", F.hardsigmoid)
Softsign = _act_cell("Softsign", F.softsign)
LogSigmoid = _act_cell("LogSigmoid", F.logsigmoid)
SeLU = _act_cell("SeLU", F.selu)
Tanhshrink = _act_cell("Tanhshrink", F.tanhshrink)
FastGelu = _act_cell("FastGelu", fused.gelu_tanh)


class GELU(Cell):
    def __init__(self, approximate=True):
        super().__init__()
        self.approximate = approximate

    def construct(self, x):
        return _wrap_out(fused.gelu_tanh(x) if self.approximate else F.gelu(x))


class LeakyReLU(Cell):
    def __init__(self, alpha=0.2):
        super().__init__()
        self.alpha = alpha

    def construct(self, x):
        return _wrap_out(F.leaky_relu(x, self.alpha))


class ELU(Cell):
    def __init__(self, alpha=1.0):
        super().__init__()
        self.alpha = alpha

    def construct(self, x):
        return _wrap_out(F.elu(x, self.alpha))


class PReLU(Cell):
    def __init__(self, channel=1, w=0.25):
        super().__init__()
        self.w = Parameter(initializer(w, (channel,), mstype.float32), name="a")

    def construct(self, x):
        return _wrap_out(F.prelu(x, self.w))


class Softmax(Cell):
    def __init__(self, axis=-1):
        super().__init__()
        self.axis = axis

    def construct(self, x):
        return _wrap_out(torch.softmax(x, self.axis))


class LogSoftmax(Softmax):
    def construct(self, x):
        return _wrap_out(torch.log_softmax(x, self.axis))


class Softplus(Cell):
    def __init__(self, beta=1, threshold=20):
        super().__init__()
        self.beta, self.threshold = beta, threshold

    def construct(self, x):
        return _wrap_out(F.softplus(x, self.beta, self.threshold))


class Hardtanh(Cell):
    def __init__(self, min_val=-1.0, max_val=1.0):
        super().__init__()
        self.lo, self.hi = min_val, max_val

    def construct(self, x):
        return _wrap_out(F.hardtanh(x, self.lo, self.hi))


class GLU(Cell):
    def __init__(self, axis=-1):
        super().__init__()
        self.axis = axis

    def construct(self, x):
        return _wrap_out(F.glu(x, self.axis))


class Threshold(Cell):
    def __init__(self, threshold, value):
        super().__init__()
        self.threshold, self.value = threshold, value

    def construct(self, x):
        return _wrap_out(F.threshold(x, self.threshold, self.value))


_ACTIVATIONS = {
    "relu": ReLU, "relu6": ReLU6, "sigmoid": Sigmoid, "tanh": Tanh, "gelu": GELU, "fast_gelu": FastGelu,
    "silu": SiLU, "swish": SiLU, "mish": Mish, "hswish": HSwish, "hsigmoid": HSigmoid, "leakyrelu": LeakyReLU,
    "elu": ELU, "softmax": Softmax, "logsoftmax": LogSoftmax, "logsigmoid": LogSigmoid, "softplus": Softplus,
    "prelu": PReLU, "selu": SeLU, "hardtanh": Hardtanh, "softsign": Softsign,
}


def get_activation(name, prim_name=None):
    if name is None:
        return None
    if isinstance(name, Cell):
        return name
    if name not in _ACTIVATIONS:
        raise KeyError("For '%s', the 'name' must be in %s, but got %r." % (prim_name or "get_activation",
                                                                            sorted(_ACTIVATIONS), name))
    return _ACTIVATIONS[name]()


# ------------------------------------------------------------------------------------ basic
class Dense(Cell):
    def __init__(self, in_channels, out_channels, weight_init=None, bias_init=None, has_bias=True, activation=None,
                 dtype=mstype.float32):
        super().__init__()
        if not isinstance(in_channels, int) or in_channels <= 0 or not isinstance(out_channels, int) or \
                out_channels <= 0:
            raise ValueError("For 'Dense', in_channels and out_channels must be positive ints")
        self.in_channels, self.out_channels, self.has_bias = in_channels, out_channels, has_bias
        if isinstance(weight_init, torch.Tensor) and tuple(weight_init.shape) != (out_channels, in_channels):
            raise ValueError("For 'Dense', weight init shape error: expected %s, got %s"
                             % ((out_channels, in_channels), tuple(weight_init.shape)))
        if weight_init is None:
            weight_init = HeUniform(math.sqrt(5))
        self.weight = Parameter(initializer(weight_init, (out_channels, in_channels), dtype), name="weight")
        self.bias = None
        if has_bias:
            if isinstance(bias_init, torch.Tensor) and tuple(bias_init.shape) != (out_channels,):
                raise ValueError("For 'Dense', bias init shape error")
            if bias_init is None:
                bound = 1 / math.sqrt(in_channels)
                bias_init = Uniform(bound)
            self.bias = Parameter(initializer(bias_init, (out_channels,), dtype), name="bias")
        self.activation = get_activation(activation) if isinstance(activation, str) else activation
        self.matmul = P.MatMul(transpose_b=True)
        self.bias_add = P.BiasAdd()

    def construct(self, x):
        w, b = self.weight, self.bias
        if self._to_float_dtype is not None and w.dtype != x.dtype:
            w = w.to(x.dtype)
            b = b.to(x.dtype) if b is not None else None
        if self.matmul.in_strategy is not None or self.matmul.in_layout is not None:
            shp = x.shape
            y = self.matmul(x.reshape(-1, shp[-1]), w)
            if b is not None:
                y = self.bias_add(y, b)
            y = y.reshape(shp[:-1] + (self.out_channels,))
        else:
            y = _wrap_out(fused.linear(x, w, b))
        if self.activation is not None:
            y = self.activation(y)
        return y

    def extend_repr(self):
        return "input_channels=%d, output_channels=%d, has_bias=%s" % (self.in_channels, self.out_channels,
                                                                       self.has_bias)


class Flatten(Cell):
    def __init__(self, start_dim=1, end_dim=-1):
        super().__init__()
        self.start_dim, self.end_dim = start_dim, end_dim

    def construct(self, x):
        return _wrap_out(torch.flatten(x, self.start_dim, self.end_dim))


class Identity(Cell):
    def construct(self, x):
        return x


class Dropout(Cell):
    def __init__(self, keep_prob=0.5, p=None, dtype=mstype.float32):
        super().__init__()
        if p is None:
            if keep_prob <= 0 or keep_prob > 1:
                raise ValueError("For 'Dropout', 'keep_prob' must be in (0, 1], got %s" % keep_prob)
            p = 1.0 - keep_prob
        elif p < 0 or p >= 1:
            raise ValueError("For 'Dropout', 'p' must be in [0, 1), got %s" % p)
        self.p = p

    def construct(self, x):
        if not self.training or self.p == 0:
            return x
        return _wrap_out(F.dropout(x, self.p, True))


class Embedding(Cell):
    def __init__(self, vocab_size, embedding_size, use_one_hot=False, embedding_table="normal", dtype=mstype.float32,
                 padding_idx=None):
        super().__init__()
        self.vocab_size, self.embedding_size, self.padding_idx = vocab_size, embedding_size, padding_idx
        table = initializer(embedding_table, (vocab_size, embedding_size), dtype)
        if padding_idx is not None:
            table[padding_idx] = 0
        self.embedding_table = Parameter(table, name="embedding_table")

    def construct(self, ids):
        return _wrap_out(fused.embedding(self.embedding_table, ids))


class EmbeddingLookup(Embedding):
    def __init__(self, vocab_size, embedding_size, param_init="normal", target="CPU", slice_mode="batch_slice",
                 manual_shapes=None, max_norm=None, sparse=True, vocab_cache_size=0, dtype=mstype.float32):
        super().__init__(vocab_size, embedding_size, embedding_table=param_init, dtype=dtype)


# ------------------------------------------------------------------------------------ convolution
def _pair(v):
    return (v, v) if isinstance(v, int) else tuple(v)


class Conv2d(Cell):
    def __init__(self, in_channels, out_channels, kernel_size, stride=1, pad_mode="same", padding=0, dilation=1,
                 group=1, has_bias=False, weight_init=None, bias_init=None, data_format="NCHW", dtype=mstype.float32):
        super().__init__()
        if pad_mode not in ("same", "valid", "pad"):
            raise ValueError("For 'Conv2d', 'pad_mode' must be same, valid or pad, got %r" % pad_mode)
        if in_channels % group or out_channels % group:
            raise ValueError("For 'Conv2d', channels must be divisible by group")
        self.in_channels, self.out_channels = in_channels, out_channels
        self.kernel_size, self.stride, self.dilation = _pair(kernel_size), _pair(stride), _pair(dilation)
        self.pad_mode, self.padding, self.group, self.has_bias = pad_mode, padding, group, has_bias
        if weight_init is None:
            weight_init = HeUniform(math.sqrt(5))
        self.weight = Parameter(initializer(weight_init, (out_channels, in_channels // group) + self.kernel_size,
                                            dtype), name="weight")
        self.bias = None
        if has_bias:
            if bias_init is None:
                fan_in = in_channels // group * self.kernel_size[0] * self.kernel_size[1]
                bias_init = Uniform(1 / math.sqrt(fan_in))
            self.bias = Parameter(initializer(bias_init, (out_channels,), dtype), name="bias")

    def construct(self, x):
        w, b = self.weight, self.bias
        if w.dtype != x.dtype:
            w = w.to(x.dtype)
            b = b.to(x.dtype) if b is not None else None
        return _wrap_out(_conv.conv2d(x, w, self.stride, self.pad_mode, self.padding, self.dilation, self.group, b))

    def extend_repr(self):
        return "input_channels=%d, output_channels=%d, kernel_size=%s, stride=%s, pad_mode=%s" % (
            self.in_channels, self.out_channels, self.kernel_size, self.stride, self.pad_mode)


class Conv1d(Cell):
    def __init__(self, in_channels, out_channels, kernel_size, stride=1, pad_mode="same", padding=0, dilation=1,
                 group=1, has_bias=False, weight_init=None, bias_init=None, dtype=mstype.float32):
        super().__init__()
        self.conv = Conv2d(in_channels, out_channels, (1, kernel_size), (1, stride), pad_mode,
                           (0, 0, padding, padding) if pad_mode == "pad" else 0, (1, dilation), group, has_bias,
                           weight_init, bias_init, dtype=dtype)

    def construct(self, x):
        return self.conv(x.unsqueeze(2)).squeeze(2)


class Conv2dTranspose(Cell):
    def __init__(self, in_channels, out_channels, kernel_size, stride=1, pad_mode="same", padding=0,
                 output_padding=0, dilation=1, group=1, has_bias=False, weight_init=None, bias_init=None,
                 dtype=mstype.float32):
        super().__init__()
        self.kernel_size, self.stride, self.dilation = _pair(kernel_size), _pair(stride), _pair(dilation)
        self.pad_mode, self.padding, self.group = pad_mode, padding, group
        self.output_padding = output_padding
        if weight_init is None:
            weight_init = HeUniform(math.sqrt(5))
        self.weight = Parameter(initializer(weight_init, (in_channels, out_channels // group) + self.kernel_size,
                                            dtype), name="weight")
        self.bias = Parameter(initializer(bias_init or "zeros", (out_channels,), dtype), name="bias") if has_bias \
            else None

    def construct(self, x):
        k, s, d = self.kernel_size, self.stride, self.dilation
        if self.pad_mode == "pad":
            p = _pair(self.padding)[:2] if not isinstance(self.padding, int) else (self.padding, self.padding)
            return _wrap_out(F.conv_transpose2d(x, self.weight.to(x.dtype), self.bias, s, p,
                                                _pair(self.output_padding), self.group, d))
        y = F.conv_transpose2d(x, self.weight.to(x.dtype), self.bias, s, 0, 0, self.group, d)
        if self.pad_mode == "same":
            th, tw = x.shape[-2] * s[0], x.shape[-1] * s[1]
            oh, ow = (y.shape[-2] - th) // 2, (y.shape[-1] - tw) // 2
            y = y[..., oh:oh + th, ow:ow + tw]
        return _wrap_out(y)


# ------------------------------------------------------------------------------------ normalisation
class _BatchNorm(Cell):
    _keep_fp32_params = True

    def __init__(self, num_features, eps=1e-5, momentum=0.9, affine=True, gamma_init="ones", beta_init="zeros",
                 moving_mean_init="zeros", moving_var_init="ones", use_batch_statistics=None, data_format="NCHW",
                 dtype=mstype.float32):
        super().__init__()
        if num_features < 1:
            raise ValueError("For BatchNorm, 'num_features' must be at least 1")
        if momentum < 0 or momentum > 1:
            raise ValueError("For BatchNorm, 'momentum' must be in [0, 1]")
        self.num_features, self.eps, self.momentum = num_features, eps, momentum
        self.use_batch_statistics = use_batch_statistics
        self.gamma = Parameter(initializer(gamma_init, (num_features,), dtype), name="gamma", requires_grad=affine)
        self.beta = Parameter(initializer(beta_init, (num_features,), dtype), name="beta", requires_grad=affine)
        self.moving_mean = Parameter(initializer(moving_mean_init, (num_features,), dtype), name="moving_mean",
                                     requires_grad=False)
        self.moving_variance = Parameter(initializer(moving_var_init, (num_features,), dtype),
                                         name="moving_variance", requires_grad=False)

    def construct(self, x):
        training = self.training if self.use_batch_statistics is None else self.use_batch_statistics
        # reference momentum convention: moving = moving*momentum + batch*(1-momentum)
        return _wrap_out(_conv.batch_norm(x, self.gamma, self.beta, self.moving_mean, self.moving_variance,
                                          training, 1.0 - self.momentum, self.eps))

    def extend_repr(self):
        return "num_features=%d, eps=%g, momentum=%g" % (self.num_features, self.eps, self.momentum)


class BatchNorm1d(_BatchNorm):
    pass


class BatchNorm2d(_BatchNorm):
    pass


class BatchNorm3d(_BatchNorm):
    pass


class SyncBatchNorm(_BatchNorm):
    """Cross-replica batch norm: per-channel sum / sum-of-squares are all-reduced over ``process_groups``."""

    def __init__(self, num_features, eps=1e-5, momentum=0.9, affine=True, gamma_init="ones", beta_init="zeros",
                 moving_mean_init="zeros", moving_var_init="ones", use_batch_statistics=None, process_groups=None,
                 dtype=mstype.float32):
        super().__init__(num_features, eps, momentum, affine, gamma_init, beta_init, moving_mean_init,
                         moving_var_init, use_batch_statistics, dtype=dtype)
        self.process_groups = process_groups

    def construct(self, x):
        import torch.distributed as dist
        training = self.training if self.use_batch_statistics is None else self.use_batch_statistics
        if not training or not (dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1):
            return super().construct(x)
        dims = [0] + list(range(2, x.dim()))
        xf = x.float()
        n = torch.tensor([xf.numel() / xf.shape[1]], device=x.device)
        stats = torch.cat([xf.sum(dims), (xf * xf).sum(dims), n])
        from ..communication.comm_func import all_reduce_autograd
        stats = all_reduce_autograd(stats)
        C = x.shape[1]
        cnt = stats[-1]
        mean = stats[:C] / cnt
        var = stats[C:2 * C] / cnt - mean * mean
        with torch.no_grad():
            m = 1.0 - self.momentum
            torch.Tensor.mul_(self.moving_mean, 1 - m).add_(mean.detach() * m)
            torch.Tensor.mul_(self.moving_variance, 1 - m).add_(var.detach() * cnt / (cnt - 1).clamp(min=1) * m)
        shape = [1, C] + [1] * (x.dim() - 2)
        y = (xf - mean.view(shape)) * torch.rsqrt(var.view(shape) + self.eps)
        return _wrap_out((y * self.gamma.view(shape) + self.beta.view(shape)).to(x.dtype))


class LayerNorm(Cell):
    _keep_fp32_params = False

    def __init__(self, normalized_shape, begin_norm_axis=-1, begin_params_axis=-1, gamma_init="ones",
                 beta_init="zeros", epsilon=1e-7, dtype=mstype.float32):
        super().__init__()
        if isinstance(normalized_shape, int):
            normalized_shape = (normalized_shape,)
        if not isinstance(normalized_shape, (tuple, list)):
            raise TypeError("For 'LayerNorm', 'normalized_shape' must be tuple[int] or list[int]")
        self.normalized_shape = tuple(normalized_shape)
        self.begin_norm_axis, self.epsilon = begin_norm_axis, epsilon
        self.gamma = Parameter(initializer(gamma_init, self.normalized_shape, dtype), name="gamma")
        self.beta = Parameter(initializer(beta_init, self.normalized_shape, dtype), name="beta")
        self.layer_norm = P.LayerNorm(begin_norm_axis, begin_params_axis, epsilon)

    def construct(self, x):
        g, b = self.gamma, self.beta
        if g.dtype != x.dtype:
            g, b = g.to(x.dtype), b.to(x.dtype)
        if self.layer_norm.in_strategy is not None:
            return self.layer_norm(x, g, b)[0]
        if len(self.normalized_shape) == 1:
            return _wrap_out(fused.layer_norm(x, g, b, self.epsilon))
        return _wrap_out(F.layer_norm(x, self.normalized_shape, g, b, self.epsilon))


class RMSNorm(Cell):
    def __init__(self, dim, eps=1e-6, dtype=mstype.float32):
        super().__init__()
        self.eps = eps
        self.weight = Parameter(initializer("ones", (dim,), dtype), name="weight")
        self.rms_norm = P.RmsNorm(eps)

    def construct(self, x, residual=None):
        w = self.weight if self.weight.dtype == x.dtype else self.weight.to(x.dtype)
        if residual is None:
            return _wrap_out(fused.rms_norm(x, w, self.eps)[0])
        y, stream = fused.rms_norm(x, w, self.eps, residual)
        return _wrap_out(y), _wrap_out(stream)


class GroupNorm(Cell):
    def __init__(self, num_groups, num_channels, eps=1e-5, affine=True, gamma_init="ones", beta_init="zeros",
                 dtype=mstype.float32):
        super().__init__()
        if num_channels % num_groups:
            raise ValueError("For 'GroupNorm', 'num_channels' must be divided by 'num_groups'")
        self.num_groups, self.eps = num_groups, eps
        self.gamma = Parameter(initializer(gamma_init, (num_channels,), dtype), name="gamma", requires_grad=affine)
        self.beta = Parameter(initializer(beta_init, (num_channels,), dtype), name="beta", requires_grad=affine)

    def construct(self, x):
        return _wrap_out(F.group_norm(x, self.num_groups, self.gamma.to(x.dtype), self.beta.to(x.dtype), self.eps))


class InstanceNorm2d(Cell):
    def __init__(self, num_features, eps=1e-5, momentum=0.1, affine=True, gamma_init="ones", beta_init="zeros",
                 dtype=mstype.float32):
        super().__init__()
        self.eps = eps
        self.gamma = Parameter(initializer(gamma_init, (num_features,), dtype), name="gamma", requires_grad=affine)
        self.beta = Parameter(initializer(beta_init, (num_features,), dtype), name="beta", requires_grad=affine)

    def construct(self, x):
        return _wrap_out(F.instance_norm(x, None, None, self.gamma.to(x.dtype), self.beta.to(x.dtype), True, 0.1,
                                         self.eps))


# ------------------------------------------------------------------------------------ pooling
class _Pool2d(Cell):
    def __init__(self, kernel_size=1, stride=1, pad_mode="valid", padding=0, dilation=1, return_indices=False,
                 ceil_mode=False, count_include_pad=True, divisor_override=None, data_format="NCHW"):
        super().__init__()
        if pad_mode.lower() not in ("valid", "same", "pad"):
            raise ValueError("pad_mode must be valid, same or pad")
        self.kernel_size, self.stride = _pair(kernel_size), _pair(stride)
        self.pad_mode, self.padding, self.ceil_mode = pad_mode.lower(), padding, ceil_mode
        self.count_include_pad = count_include_pad


class MaxPool2d(_Pool2d):
    def construct(self, x):
        if self.pad_mode == "same":
            x = P._same_pad(x, self.kernel_size, self.stride, float("-inf"))
            return _wrap_out(F.max_pool2d(x, self.kernel_size, self.stride))
        pad = self.padding if self.pad_mode == "pad" else 0
        return _wrap_out(F.max_pool2d(x, self.kernel_size, self.stride, pad, ceil_mode=self.ceil_mode))


class AvgPool2d(_Pool2d):
    def construct(self, x):
        if self.pad_mode == "same":
            x = P._same_pad(x, self.kernel_size, self.stride, 0.0)
            return _wrap_out(F.avg_pool2d(x, self.kernel_size, self.stride))
        pad = self.padding if self.pad_mode == "pad" else 0
        return _wrap_out(F.avg_pool2d(x, self.kernel_size, self.stride, pad, self.ceil_mode, self.count_include_pad))


class MaxPool1d(Cell):
    def __init__(self, kernel_size=1, stride=1, pad_mode="valid"):
        super().__init__()
        self.k, self.s = kernel_size, stride

    def construct(self, x):
        return _wrap_out(F.max_pool1d(x, self.k, self.s))


class AvgPool1d(MaxPool1d):
    def construct(self, x):
        return _wrap_out(F.avg_pool1d(x, self.k, self.s))


class AdaptiveAvgPool2d(Cell):
    def __init__(self, output_size):
        super().__init__()
        self.output_size = output_size

    def construct(self, x):
        return _wrap_out(F.adaptive_avg_pool2d(x, self.output_size))


class AdaptiveMaxPool2d(AdaptiveAvgPool2d):
    def construct(self, x):
        return _wrap_out(F.adaptive_max_pool2d(x, self.output_size))


# ------------------------------------------------------------------------------------ containers
class SequentialCell(Cell):
    def __init__(self, *args):
        super().__init__()
        self._is_dynamic_name = []
        if len(args) == 1 and isinstance(args[0], (list, tuple)):
            for i, c in enumerate(args[0]):
                self.insert_child_to_cell(str(i), c)
                c.update_parameters_name(str(i) + ".")
        elif len(args) == 1 and isinstance(args[0], OrderedDict):
            for name, c in args[0].items():
                self.insert_child_to_cell(name, c)
                c.update_parameters_name(name + ".")
        else:
            for i, c in enumerate(args):
                self.insert_child_to_cell(str(i), c)
                c.update_parameters_name(str(i) + ".")
        self.cell_list = list(self._cells.values())

    def __getitem__(self, index):
        if isinstance(index, slice):
            return SequentialCell(OrderedDict(list(self._cells.items())[index]))
        return list(self._cells.values())[index]

    def __len__(self):
        return len(self._cells)

    def __iter__(self):
        return iter(self._cells.values())

    def append(self, cell):
        name = str(len(self))
        self.insert_child_to_cell(name, cell)
        cell.update_parameters_name(name + ".")
        self.cell_list = list(self._cells.values())
        return self

    def construct(self, x):
        for c in self._cells.values():
            x = c(x)
        return x


class CellList(Cell):
    def __init__(self, *args, **kwargs):
        auto_prefix = kwargs.pop("auto_prefix", True)
        super().__init__(auto_prefix=auto_prefix)
        if len(args) == 1:
            self.extend(args[0])

    def __getitem__(self, index):
        if isinstance(index, slice):
            return CellList(list(self._cells.values())[index])
        return list(self._cells.values())[index]

    def __setitem__(self, index, cell):
        key = list(self._cells.keys())[index]
        self._cells[key] = cell

    def __len__(self):
        return len(self._cells)

    def __iter__(self):
        return iter(self._cells.values())

    def append(self, cell):
        if not isinstance(cell, Cell):
            raise TypeError("CellList elements must be Cell, got %s" % type(cell))
        name = str(len(self))
        if self._auto_prefix:
            cell.update_parameters_name(name + ".")
        self._cells[name] = cell
        return self

    def extend(self, cells):
        for c in cells:
            self.append(c)
        return self

    def insert(self, index, cell):
        items = list(self._cells.values())
        items.insert(index, cell)
        self._cells.clear()
        for i, c in enumerate(items):
            self._cells[str(i)] = c

    def construct(self, *inputs):
        raise NotImplementedError("CellList is a container and can not be called")


class CellDict(Cell):
    def __init__(self, *args, **kwargs):
        super().__init__()
        if args:
            items = args[0].items() if isinstance(args[0], dict) else args[0]
            for k, v in items:
                self[k] = v

    def __getitem__(self, key):
        return self._cells[key]

    def __setitem__(self, key, cell):
        cell.update_parameters_name(key + ".")
        self._cells[key] = cell

    def __len__(self):
        return len(self._cells)

    def __iter__(self):
        return iter(self._cells)

    def __contains__(self, key):
        return key in self._cells

    def keys(self):
        return self._cells.keys()

    def values(self):
        return self._cells.values()

    def items(self):
        return self._cells.items()

    def construct(self, *inputs):
        raise NotImplementedError("CellDict is a container and can not be called")


# ------------------------------------------------------------------------------------ recurrent
class _RNNBase(Cell):
    _mode = "LSTM"

    def __init__(self, input_size, hidden_size, num_layers=1, has_bias=True, batch_first=False, dropout=0.0,
                 bidirectional=False, dtype=mstype.float32):
        super().__init__()
        self.input_size, self.hidden_size, self.num_layers = input_size, hidden_size, num_layers
        self.batch_first, self.dropout, self.bidirectional, self.has_bias = batch_first, dropout, bidirectional, has_bias
        gate = {"LSTM": 4, "GRU": 3, "RNN_TANH": 1, "RNN_RELU": 1}[self._mode]
        ndir = 2 if bidirectional else 1
        k = 1 / math.sqrt(hidden_size)
        self._flat_names = []
        for layer in range(num_layers):
            for d in range(ndir):
                suf = "_l%d%s" % (layer, "_reverse" if d else "")
                isz = input_size if layer == 0 else hidden_size * ndir
                names = [("weight_ih" + suf, (gate * hidden_size, isz)), ("weight_hh" + suf, (gate * hidden_size, hidden_size))]
                if has_bias:
                    names += [("bias_ih" + suf, (gate * hidden_size,)), ("bias_hh" + suf, (gate * hidden_size,))]
                for n, shp in names:
                    setattr(self, n, Parameter(initializer(Uniform(k), shp, dtype), name=n))
                    self._flat_names.append(n)

    def construct(self, x, hx=None, seq_length=None):
        flat = [getattr(self, n) for n in self._flat_names]
        B = x.shape[0] if self.batch_first else x.shape[1]
        ndir = 2 if self.bidirectional else 1
        if hx is None:
            z = torch.zeros(self.num_layers * ndir, B, self.hidden_size, dtype=x.dtype, device=x.device)
            hx = (z, z.clone()) if self._mode == "LSTM" else z
        vf = torch._VF
        if self._mode == "LSTM":
            out, h, c = vf.lstm(x, hx, flat, self.has_bias, self.num_layers, self.dropout, self.training,
                                self.bidirectional, self.batch_first)
            return _wrap_out(out), (_wrap_out(h), _wrap_out(c))
        fn = {"GRU": vf.gru, "RNN_TANH": vf.rnn_tanh, "RNN_RELU": vf.rnn_relu}[self._mode]
        out, h = fn(x, hx, flat, self.has_bias, self.num_layers, self.dropout, self.training, self.bidirectional,
                    self.batch_first)
        return _wrap_out(out), _wrap_out(h)


class LSTM(_RNNBase):
    _mode = "LSTM"


class GRU(_RNNBase):
    _mode = "GRU"


class RNN(_RNNBase):
    _mode = "RNN_TANH"

    def __init__(self, *args, nonlinearity="tanh", **kwargs):
        self._mode = "RNN_TANH" if nonlinearity == "tanh" else "RNN_RELU"
        super().__init__(*args, **kwargs)


# ------------------------------------------------------------------------------------ misc layers
class Pad(Cell):
    def __init__(self, paddings, mode="CONSTANT"):
        super().__init__()
        self.paddings, self.mode = paddings, mode.lower()

    def construct(self, x):
        flat = []
        for lo, hi in reversed(self.paddings):
            flat += [lo, hi]
        mode = {"constant": "constant", "reflect": "reflect", "symmetric": "replicate"}[self.mode]
        return _wrap_out(F.pad(x, flat, mode=mode))


class Upsample(Cell):
    def __init__(self, size=None, scale_factor=None, mode="nearest", align_corners=None):
        super().__init__()
        self.size, self.scale_factor, self.mode, self.align_corners = size, scale_factor, mode, align_corners

    def construct(self, x):
        return _wrap_out(F.interpolate(x, self.size, self.scale_factor, self.mode, self.align_corners))


class OneHot(Cell):
    def __init__(self, axis=-1, depth=1, on_value=1.0, off_value=0.0, dtype=mstype.float32):
        super().__init__()
        self.depth, self.on, self.off, self.dtype, self.axis = depth, on_value, off_value, dtype, axis

    def construct(self, idx):
        oh = F.one_hot(idx.long(), self.depth).to(self.dtype)
        return _wrap_out(oh * (self.on - self.off) + self.off)


class MultiheadAttention(Cell):
    """torch-like multi-head attention (nn/layer/transformer.py:60).  Inputs are (L, N, E) or (N, L, E)."""

    def __init__(self, embed_dim, num_heads, dropout=0.0, has_bias=True, add_bias_kv=False, add_zero_attn=False,
                 kdim=None, vdim=None, batch_first=False, dtype=mstype.float32):
        super().__init__()
        if embed_dim % num_heads:
            raise ValueError("embed_dim must be divisible by num_heads")
        self.embed_dim, self.num_heads, self.batch_first = embed_dim, num_heads, batch_first
        self.in_proj = Dense(embed_dim, 3 * embed_dim, has_bias=has_bias, dtype=dtype)
        self.out_proj = Dense(embed_dim, embed_dim, has_bias=has_bias, dtype=dtype)

    def construct(self, query, key, value, key_padding_mask=None, need_weights=False, attn_mask=None):
        if not self.batch_first:
            query, key, value = (t.transpose(1, 0, 2) for t in (query, key, value))
        w, b = self.in_proj.weight, self.in_proj.bias
        E = self.embed_dim
        q = fused.linear(query, w[:E], b[:E] if b is not None else None)
        k = fused.linear(key, w[E:2 * E], b[E:2 * E] if b is not None else None)
        v = fused.linear(value, w[2 * E:], b[2 * E:] if b is not None else None)
        B, L, _ = q.shape
        H = self.num_heads
        q, k, v = (t.reshape(B, t.shape[1], H, E // H).permute(0, 2, 1, 3) for t in (q, k, v))
        mask = None
        if attn_mask is not None:
            mask = ~attn_mask.bool() if attn_mask.dtype == torch.bool else attn_mask
        if key_padding_mask is not None:
            kp = ~key_padding_mask.bool()[:, None, None, :]
            mask = kp if mask is None else (mask & kp if mask.dtype == torch.bool else mask)
        o = F.scaled_dot_product_attention(q, k, v, attn_mask=mask)
        o = o.permute(0, 2, 1, 3).reshape(B, L, E)
        out = self.out_proj(_wrap_out(o))
        if not self.batch_first:
            out = out.transpose(1, 0, 2)
        return out, None
