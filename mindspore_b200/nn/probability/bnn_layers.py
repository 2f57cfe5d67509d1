"""Bayesian layers: weights are distributions, the forward pass samples them, the training loss adds the KL
divergence from a prior.

``NormalPosterior`` holds a trainable mean and an unconstrained scale (``sd = 1e-6 + softplus(untransformed_std)``);
``NormalPrior`` is a fixed normal.  ``DenseReparam`` / ``ConvReparam`` sample one weight per call with the
reparameterisation trick (``w = mean + sd * eps``), ``DenseLocalReparam`` samples the pre-activation instead
(``N(x @ mean.T, sqrt(x**2 @ sd**2.T))``), which lowers the gradient variance for the same cost.
``WithBNNLossCell`` walks a network, collects ``compute_kl_loss`` of every Bayesian layer and returns
``dnn_factor * loss + bnn_factor * sum(kl)``.

Parity: mindspore/python/mindspore/nn/probability/bnn_layers/{layer_distribution,dense_variational,
conv_variational,bnn_cell_wrapper}.py.
"""
import math

import numpy as np
import torch
import torch.nn.functional as F

from ...common.parameter import Parameter
from ...common.tensor import Tensor
from ..cell import Cell
from ..layer import get_activation

__all__ = ["NormalPrior", "NormalPosterior", "DenseReparam", "DenseLocalReparam", "ConvReparam", "WithBNNLossCell"]


def _number(value, name, non_negative=False):
    if isinstance(value, bool) or not isinstance(value, (int, float)):
        raise TypeError("The type of `%s` must be `int` or `float`" % name)
    if non_negative and value < 0:
        raise TypeError("The type of `%s` must be `int` or `float` and its value must > 0" % name)
    return float(value)


class _LayerDistribution(Cell):
    """What both ends of the KL term offer: ``mean()`` / ``sd()`` tensors, ``sample()``, and the reference's
    call-by-name form (``dist("sample")``, ``dist("kl_loss", "Normal", mean, sd)``)."""

    def mean_value(self):
        raise NotImplementedError

    def sd_value(self):
        raise NotImplementedError

    def sample(self, shape=None):
        mean, sd = self.mean_value(), self.sd_value()
        if shape is not None:
            mean, sd = mean.expand(tuple(shape) + tuple(mean.shape)), sd.expand(tuple(shape) + tuple(sd.shape))
        return mean + sd * torch.randn_like(mean + sd)

    def kl_loss(self, dist_type, mean_b, sd_b):
        """KL(N(mean_b, sd_b) || self), elementwise."""
        if dist_type != "Normal":
            raise ValueError("kl_loss is defined between Normal distributions, but got %r" % (dist_type,))
        mean_a, sd_a = self.mean_value(), self.sd_value()
        ratio = sd_b / sd_a
        return 0.5 * (ratio * ratio + ((mean_b - mean_a) / sd_a) ** 2 - 1.0) - torch.log(ratio)

    def construct(self, name="sample", *args, **kwargs):
        if name == "sample":
            return self.sample(*args, **kwargs)
        if name == "mean":
            return self.mean_value()
        if name == "sd":
            return self.sd_value()
        if name == "var":
            return self.sd_value() ** 2
        if name == "get_dist_type":
            return "Normal"
        if name == "get_dist_args":
            return self.mean_value(), self.sd_value()
        if name == "kl_loss":
            return self.kl_loss(*args)
        raise ValueError("unknown distribution function %r" % (name,))


class NormalPrior(_LayerDistribution):
    def __init__(self, dtype=torch.float32, mean=0, std=0.1):
        super().__init__()
        self._mean = torch.tensor(_number(mean, "mean"), dtype=dtype)
        self._sd = torch.tensor(_number(std, "std"), dtype=dtype)

    def mean_value(self):
        return self._mean

    def sd_value(self):
        return self._sd


class NormalPosterior(_LayerDistribution):
    def __init__(self, name, shape, dtype=torch.float32, loc_mean=0, loc_std=0.1, untransformed_scale_mean=-5,
                 untransformed_scale_std=0.1):
        super().__init__()
        if not isinstance(name, str):
            raise TypeError("The type of `name` must be `str`")
        if not isinstance(shape, (tuple, list)):
            raise TypeError("The type of `shape` must be `tuple` or `list`")
        _number(loc_mean, "loc_mean")
        _number(untransformed_scale_mean, "untransformed_scale_mean")
        _number(loc_std, "loc_std", non_negative=True)
        _number(untransformed_scale_std, "untransformed_scale_std", non_negative=True)
        self.mean = Parameter(Tensor(np.random.normal(loc_mean, loc_std, shape), dtype=dtype), name=name + "_mean")
        self.untransformed_std = Parameter(
            Tensor(np.random.normal(untransformed_scale_mean, untransformed_scale_std, shape), dtype=dtype),
            name=name + "_untransformed_std")

    def mean_value(self):
        return self.mean

    def sd_value(self):
        return 1e-6 + F.softplus(self.untransformed_std)


def normal_post_fn(name, shape):
    return NormalPosterior(name=name, shape=shape)


def _prior(fn, arg_name):
    prior = fn() if isinstance(fn, type) or not isinstance(fn, Cell) and callable(fn) else fn
    if not isinstance(prior, Cell):
        raise TypeError("The type of `%s` must be `Cell` or a function that returns one" % arg_name)
    return prior


def _posterior(fn, shape, param_name, arg_name):
    try:
        post = fn(shape=shape, name=param_name)
    except TypeError:
        raise TypeError("The type of `%s` must be a function with `name` and `shape` arguments" % arg_name)
    if not isinstance(post, Cell):
        raise TypeError("`%s` must return a Cell" % arg_name)
    for p in post.get_parameters():
        if not p.requires_grad:
            raise ValueError("The parameters of `%s` must be trainable" % arg_name)
    return post


class _Variational(Cell):
    """The KL bookkeeping that dense and convolutional layers share."""

    has_bias = False

    def compute_kl_loss(self):
        kl = self.weight_prior.kl_loss("Normal", *self.weight_posterior("get_dist_args")).sum()
        if self.has_bias:
            kl = kl + self.bias_prior.kl_loss("Normal", *self.bias_posterior("get_dist_args")).sum()
        return kl

    def _set_activation(self, activation):
        if not activation:
            self.activation, self.activation_flag = None, False
            return
        self.activation_flag = True
        if isinstance(activation, str):
            self.activation = get_activation(activation)
        elif isinstance(activation, Cell):
            self.activation = activation
        else:
            raise ValueError("The type of `activation` is wrong.")


class _DenseVariational(_Variational):
    def __init__(self, in_channels, out_channels, activation=None, has_bias=True, weight_prior_fn=NormalPrior,
                 weight_posterior_fn=normal_post_fn, bias_prior_fn=NormalPrior, bias_posterior_fn=normal_post_fn):
        super().__init__()
        for v, n in ((in_channels, "in_channels"), (out_channels, "out_channels")):
            if isinstance(v, bool) or not isinstance(v, int) or v <= 0:
                raise ValueError("`%s` must be a positive int, but got %r" % (n, v))
        self.in_channels, self.out_channels, self.has_bias = in_channels, out_channels, bool(has_bias)
        self.weight_prior = _prior(weight_prior_fn, "weight_prior_fn")
        self.weight_posterior = _posterior(weight_posterior_fn, [out_channels, in_channels], "bnn_weight",
                                           "weight_posterior_fn")
        if self.has_bias:
            self.bias_prior = _prior(bias_prior_fn, "bias_prior_fn")
            self.bias_posterior = _posterior(bias_posterior_fn, [out_channels], "bnn_bias", "bias_posterior_fn")
        self._set_activation(activation)

    def construct(self, x):
        out = self._apply_variational_weight(x)
        if self.has_bias:
            out = out + self.bias_posterior("sample")
        return self.activation(out) if self.activation_flag else out


class DenseReparam(_DenseVariational):
    def _apply_variational_weight(self, x):
        return x @ self.weight_posterior("sample").t()


class DenseLocalReparam(_DenseVariational):
    def _apply_variational_weight(self, x):
        mean = x @ self.weight_posterior("mean").t()
        sd = torch.sqrt((x * x) @ (self.weight_posterior("sd") ** 2).t())
        return mean + sd * torch.randn_like(mean)


class _ConvVariational(_Variational):
    def __init__(self, in_channels, out_channels, kernel_size, stride=1, pad_mode="same", padding=0, dilation=1,
                 group=1, has_bias=False, weight_prior_fn=NormalPrior, weight_posterior_fn=normal_post_fn,
                 bias_prior_fn=NormalPrior, bias_posterior_fn=normal_post_fn):
        super().__init__()
        pair = lambda v: (v, v) if isinstance(v, int) else tuple(v)                          # noqa: E731
        if pad_mode not in ("valid", "same", "pad"):
            raise ValueError("`pad_mode` must be one of valid, same, pad, but got %r" % (pad_mode,))
        if in_channels % group or out_channels % group:
            raise ValueError("`in_channels` and `out_channels` must be divisible by `group`")
        self.in_channels, self.out_channels, self.group = in_channels, out_channels, group
        self.kernel_size, self.stride, self.dilation = pair(kernel_size), pair(stride), pair(dilation)
        self.pad_mode, self.padding, self.has_bias = pad_mode, padding, bool(has_bias)
        self.shape = [out_channels, in_channels // group, *self.kernel_size]
        self.weight_prior = _prior(weight_prior_fn, "weight_prior_fn")
        self.weight_posterior = _posterior(weight_posterior_fn, self.shape, "bnn_weight", "weight_posterior_fn")
        if self.has_bias:
            self.bias_prior = _prior(bias_prior_fn, "bias_prior_fn")
            self.bias_posterior = _posterior(bias_posterior_fn, [out_channels], "bnn_bias", "bias_posterior_fn")

    def _conv(self, x, weight):
        if self.pad_mode == "same":
            if self.stride == (1, 1):
                return F.conv2d(x, weight, None, 1, "same", self.dilation, self.group)
            pads = []
            for size, k, s, d in zip(x.shape[-2:], self.kernel_size, self.stride, self.dilation):
                total = max((math.ceil(size / s) - 1) * s + (k - 1) * d + 1 - size, 0)
                pads = [total // 2, total - total // 2] + pads           # F.pad takes the last axis first
            return F.conv2d(F.pad(x, pads), weight, None, self.stride, 0, self.dilation, self.group)
        if self.pad_mode == "pad":
            p = self.padding
            if isinstance(p, int):
                return F.conv2d(x, weight, None, self.stride, p, self.dilation, self.group)
            top, bottom, left, right = p
            return F.conv2d(F.pad(x, [left, right, top, bottom]), weight, None, self.stride, 0, self.dilation,
                            self.group)
        return F.conv2d(x, weight, None, self.stride, 0, self.dilation, self.group)

    def construct(self, x):
        out = self._apply_variational_weight(x)
        if self.has_bias:
            out = out + self.bias_posterior("sample").reshape(1, -1, 1, 1)
        return out


class ConvReparam(_ConvVariational):
    def _apply_variational_weight(self, x):
        return self._conv(x, self.weight_posterior("sample"))


class WithBNNLossCell(Cell):
    def __init__(self, backbone, loss_fn, dnn_factor=1, bnn_factor=1):
        super().__init__(auto_prefix=False)
        for v, n in ((dnn_factor, "dnn_factor"), (bnn_factor, "bnn_factor")):
            if isinstance(v, bool) or not isinstance(v, (int, float)):
                raise TypeError("The type of `%s` must be `int` or `float`" % n)
            if v < 0:
                raise ValueError("The value of `%s` must >= 0" % n)
        self._backbone, self._loss_fn = backbone, loss_fn
        self.dnn_factor, self.bnn_factor = dnn_factor, bnn_factor
        self.kl_loss = []
        self._collect(backbone)

    def _collect(self, net):
        for _, layer in net.name_cells().items():
            if isinstance(layer, _Variational):
                self.kl_loss.append(layer.compute_kl_loss)
            else:
                self._collect(layer)

    def construct(self, x, label):
        loss = self._loss_fn(self._backbone(x), label) * self.dnn_factor
        kl = 0
        for term in self.kl_loss:
            kl = kl + term()
        return loss + kl * self.bnn_factor

    @property
    def backbone_network(self):
        return self._backbone
