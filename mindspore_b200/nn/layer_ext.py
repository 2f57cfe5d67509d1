"""Less common layers: 3-D and transposed convolutions, RNN cells, the ``nn.Transformer`` family, pixel shuffle,
unfold / fold, multi-field embedding lookup, InstanceNorm1d.

Parity: python/mindspore/nn/layer/{conv.py (Conv3d :700, Conv1dTranspose :1190, Conv3dTranspose :900),
rnn_cells.py, transformer.py, channel_shuffle.py / pixel shuffle in basic.py, embedding.py
(MultiFieldEmbeddingLookup :560), normalization.py}."""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F

from ..common import dtype as mstype
from ..common.initializer import HeUniform, Uniform, initializer
from ..common.parameter import Parameter
from ..ops.primitive import _wrap_out
from .cell import Cell
from .layer import CellList, Dense, Dropout, LayerNorm, MultiheadAttention

__all__ = ["Conv3d", "Conv1dTranspose", "Conv3dTranspose", "InstanceNorm1d", "InstanceNorm3d", "LSTMCell", "GRUCell",
           "RNNCell", "TransformerEncoderLayer", "TransformerDecoderLayer", "TransformerEncoder", "TransformerDecoder",
           "Transformer", "PixelShuffle", "PixelUnshuffle", "Unfold", "Fold", "MultiFieldEmbeddingLookup",
           "ChannelShuffle"]


def _tuple(v, n):
    return (v,) * n if isinstance(v, int) else tuple(v)


def _same_pads(size, k, s, d):
    out = []
    for i in range(len(size)):
        eff = (k[i] - 1) * d[i] + 1
        total = max((math.ceil(size[i] / s[i]) - 1) * s[i] + eff - size[i], 0)
        out.append((total // 2, total - total // 2))
    return out


class Conv3d(Cell):
    def __init__(self, in_channels, out_channels, kernel_size, stride=1, pad_mode="same", padding=0, dilation=1,
                 group=1, has_bias=False, weight_init=None, bias_init=None, data_format="NCDHW", dtype=mstype.float32):
        super().__init__()
        self.kernel_size, self.stride, self.dilation = _tuple(kernel_size, 3), _tuple(stride, 3), _tuple(dilation, 3)
        self.pad_mode, self.padding, self.group = pad_mode, padding, group
        self.weight = Parameter(initializer(weight_init or HeUniform(math.sqrt(5)),
                                            (out_channels, in_channels // group) + self.kernel_size, dtype), name="weight")
        fan_in = in_channels // group * self.kernel_size[0] * self.kernel_size[1] * self.kernel_size[2]
        self.bias = Parameter(initializer(bias_init or Uniform(1 / math.sqrt(fan_in)), (out_channels,), dtype),
                              name="bias") if has_bias else None

    def construct(self, x):
        w = self.weight.to(x.dtype)
        b = self.bias.to(x.dtype) if self.bias is not None else None
        pad = 0
        if self.pad_mode == "same":
            pads = _same_pads(x.shape[2:], self.kernel_size, self.stride, self.dilation)
            x = F.pad(x, [p for pr in reversed(pads) for p in pr])
        elif self.pad_mode == "pad":
            p = self.padding
            if isinstance(p, int):
                pad = p
            else:
                x = F.pad(x, [p[4], p[5], p[2], p[3], p[0], p[1]])
        return _wrap_out(F.conv3d(x, w, b, self.stride, pad, self.dilation, self.group))


class _ConvTransposeNd(Cell):
    _nd = 2

    def __init__(self, in_channels, out_channels, kernel_size, stride=1, pad_mode="same", padding=0, dilation=1,
                 group=1, output_padding=0, has_bias=False, weight_init=None, bias_init=None, dtype=mstype.float32):
        super().__init__()
        n = self._nd
        self.kernel_size, self.stride, self.dilation = _tuple(kernel_size, n), _tuple(stride, n), _tuple(dilation, n)
        self.pad_mode, self.padding, self.group, self.output_padding = pad_mode, padding, group, output_padding
        self.weight = Parameter(initializer(weight_init or HeUniform(math.sqrt(5)),
                                            (in_channels, out_channels // group) + self.kernel_size, dtype), name="weight")
        self.bias = Parameter(initializer(bias_init or "zeros", (out_channels,), dtype), name="bias") if has_bias else None

    def construct(self, x):
        fn = {1: F.conv_transpose1d, 3: F.conv_transpose3d}[self._nd]
        w = self.weight.to(x.dtype)
        b = self.bias.to(x.dtype) if self.bias is not None else None
        if self.pad_mode == "pad":
            p = self.padding if isinstance(self.padding, int) else tuple(self.padding)[::2]
            return _wrap_out(fn(x, w, b, self.stride, p, self.output_padding, self.group, self.dilation))
        y = fn(x, w, b, self.stride, 0, 0, self.group, self.dilation)
        if self.pad_mode == "same":
            for i in range(self._nd):
                target = x.shape[2 + i] * self.stride[i]
                off = (y.shape[2 + i] - target) // 2
                y = y.narrow(2 + i, off, target)
        return _wrap_out(y)


class Conv1dTranspose(_ConvTransposeNd):
    _nd = 1


class Conv3dTranspose(_ConvTransposeNd):
    _nd = 3


class _InstanceNorm(Cell):
    def __init__(self, num_features, eps=1e-5, momentum=0.1, affine=True, gamma_init="ones", beta_init="zeros",
                 dtype=mstype.float32):
        super().__init__()
        self.eps, self.affine = eps, affine
        self.gamma = Parameter(initializer(gamma_init, (num_features,), dtype), name="gamma", requires_grad=affine)
        self.beta = Parameter(initializer(beta_init, (num_features,), dtype), name="beta", requires_grad=affine)

    def construct(self, x):
        return _wrap_out(F.instance_norm(x, None, None, self.gamma.to(x.dtype), self.beta.to(x.dtype), True, 0.1,
                                         self.eps))


class InstanceNorm1d(_InstanceNorm):
    pass


class InstanceNorm3d(_InstanceNorm):
    pass


# ------------------------------------------------------------------------------------------------ RNN cells
class _RNNCellBase(Cell):
    _gates = 1

    def __init__(self, input_size, hidden_size, has_bias=True, dtype=mstype.float32):
        super().__init__()
        self.input_size, self.hidden_size, self.has_bias = input_size, hidden_size, has_bias
        k = 1 / math.sqrt(hidden_size)
        g = self._gates * hidden_size
        self.weight_ih = Parameter(initializer(Uniform(k), (g, input_size), dtype), name="weight_ih")
        self.weight_hh = Parameter(initializer(Uniform(k), (g, hidden_size), dtype), name="weight_hh")
        self.bias_ih = Parameter(initializer(Uniform(k), (g,), dtype), name="bias_ih") if has_bias else None
        self.bias_hh = Parameter(initializer(Uniform(k), (g,), dtype), name="bias_hh") if has_bias else None


class RNNCell(_RNNCellBase):
    def __init__(self, input_size, hidden_size, has_bias=True, nonlinearity="tanh", dtype=mstype.float32):
        super().__init__(input_size, hidden_size, has_bias, dtype)
        if nonlinearity not in ("tanh", "relu"):
            raise ValueError("For 'RNNCell', 'nonlinearity' must be tanh or relu, got %r" % nonlinearity)
        self.nonlinearity = nonlinearity

    def construct(self, x, hx):
        pre = F.linear(x, self.weight_ih, self.bias_ih) + F.linear(hx, self.weight_hh, self.bias_hh)
        return _wrap_out(torch.tanh(pre) if self.nonlinearity == "tanh" else F.relu(pre))


class LSTMCell(_RNNCellBase):
    _gates = 4

    def construct(self, x, hx):
        h, c = hx
        gates = F.linear(x, self.weight_ih, self.bias_ih) + F.linear(h, self.weight_hh, self.bias_hh)
        i, f, g, o = gates.chunk(4, -1)
        c2 = torch.sigmoid(f) * c + torch.sigmoid(i) * torch.tanh(g)
        h2 = torch.sigmoid(o) * torch.tanh(c2)
        return _wrap_out(h2), _wrap_out(c2)


class GRUCell(_RNNCellBase):
    _gates = 3

    def construct(self, x, hx):
        gi = F.linear(x, self.weight_ih, self.bias_ih)
        gh = F.linear(hx, self.weight_hh, self.bias_hh)
        ir, iz, in_ = gi.chunk(3, -1)
        hr, hz, hn = gh.chunk(3, -1)
        r, z = torch.sigmoid(ir + hr), torch.sigmoid(iz + hz)
        n = torch.tanh(in_ + r * hn)
        return _wrap_out((1 - z) * n + z * hx)


# ------------------------------------------------------------------------------------------------ nn.Transformer
def _activation(name):
    if callable(name):
        return name
    return {"relu": F.relu, "gelu": F.gelu}[name]


class TransformerEncoderLayer(Cell):
    def __init__(self, d_model, nhead, dim_feedforward=2048, dropout=0.1, activation="relu", layer_norm_eps=1e-5,
                 batch_first=False, norm_first=False, dtype=mstype.float32):
        super().__init__()
        self.self_attn = MultiheadAttention(d_model, nhead, dropout=dropout, batch_first=batch_first, dtype=dtype)
        self.dense1, self.dense2 = Dense(d_model, dim_feedforward, dtype=dtype), Dense(dim_feedforward, d_model, dtype=dtype)
        self.norm1, self.norm2 = LayerNorm((d_model,), epsilon=layer_norm_eps), LayerNorm((d_model,), epsilon=layer_norm_eps)
        self.dropout, self.dropout1, self.dropout2 = Dropout(p=dropout), Dropout(p=dropout), Dropout(p=dropout)
        self.act, self.norm_first = _activation(activation), norm_first

    def _sa(self, x, mask, kpm):
        return self.dropout1(self.self_attn(x, x, x, attn_mask=mask, key_padding_mask=kpm, need_weights=False)[0])

    def _ff(self, x):
        return self.dropout2(self.dense2(self.dropout(_wrap_out(self.act(self.dense1(x))))))

    def construct(self, src, src_mask=None, src_key_padding_mask=None):
        x = src
        if self.norm_first:
            x = x + self._sa(self.norm1(x), src_mask, src_key_padding_mask)
            return x + self._ff(self.norm2(x))
        x = self.norm1(x + self._sa(x, src_mask, src_key_padding_mask))
        return self.norm2(x + self._ff(x))


class TransformerDecoderLayer(Cell):
    def __init__(self, d_model, nhead, dim_feedforward=2048, dropout=0.1, activation="relu", layer_norm_eps=1e-5,
                 batch_first=False, norm_first=False, dtype=mstype.float32):
        super().__init__()
        self.self_attn = MultiheadAttention(d_model, nhead, dropout=dropout, batch_first=batch_first, dtype=dtype)
        self.multihead_attn = MultiheadAttention(d_model, nhead, dropout=dropout, batch_first=batch_first, dtype=dtype)
        self.dense1, self.dense2 = Dense(d_model, dim_feedforward, dtype=dtype), Dense(dim_feedforward, d_model, dtype=dtype)
        self.norm1, self.norm2, self.norm3 = (LayerNorm((d_model,), epsilon=layer_norm_eps) for _ in range(3))
        self.dropout, self.dropout1, self.dropout2, self.dropout3 = (Dropout(p=dropout) for _ in range(4))
        self.act, self.norm_first = _activation(activation), norm_first

    def construct(self, tgt, memory, tgt_mask=None, memory_mask=None, tgt_key_padding_mask=None,
                  memory_key_padding_mask=None):
        def sa(x):
            return self.dropout1(self.self_attn(x, x, x, attn_mask=tgt_mask, key_padding_mask=tgt_key_padding_mask,
                                                need_weights=False)[0])

        def ca(x):
            return self.dropout2(self.multihead_attn(x, memory, memory, attn_mask=memory_mask,
                                                     key_padding_mask=memory_key_padding_mask, need_weights=False)[0])

        def ff(x):
            return self.dropout3(self.dense2(self.dropout(_wrap_out(self.act(self.dense1(x))))))
        x = tgt
        if self.norm_first:
            x = x + sa(self.norm1(x))
            x = x + ca(self.norm2(x))
            return x + ff(self.norm3(x))
        x = self.norm1(x + sa(x))
        x = self.norm2(x + ca(x))
        return self.norm3(x + ff(x))


class TransformerEncoder(Cell):
    def __init__(self, encoder_layer, num_layers, norm=None):
        super().__init__()
        import copy
        self.layers = CellList([encoder_layer] + [copy.deepcopy(encoder_layer) for _ in range(num_layers - 1)])
        self.norm = norm

    def construct(self, src, src_mask=None, src_key_padding_mask=None):
        x = src
        for layer in self.layers:
            x = layer(x, src_mask, src_key_padding_mask)
        return self.norm(x) if self.norm is not None else x


class TransformerDecoder(Cell):
    def __init__(self, decoder_layer, num_layers, norm=None):
        super().__init__()
        import copy
        self.layers = CellList([decoder_layer] + [copy.deepcopy(decoder_layer) for _ in range(num_layers - 1)])
        self.norm = norm

    def construct(self, tgt, memory, tgt_mask=None, memory_mask=None, tgt_key_padding_mask=None,
                  memory_key_padding_mask=None):
        x = tgt
        for layer in self.layers:
            x = layer(x, memory, tgt_mask, memory_mask, tgt_key_padding_mask, memory_key_padding_mask)
        return self.norm(x) if self.norm is not None else x


class Transformer(Cell):
    def __init__(self, d_model=512, nhead=8, num_encoder_layers=6, num_decoder_layers=6, dim_feedforward=2048,
                 dropout=0.1, activation="relu", custom_encoder=None, custom_decoder=None, layer_norm_eps=1e-5,
                 batch_first=False, norm_first=False, dtype=mstype.float32):
        super().__init__()
        self.encoder = custom_encoder or TransformerEncoder(
            TransformerEncoderLayer(d_model, nhead, dim_feedforward, dropout, activation, layer_norm_eps, batch_first,
                                    norm_first, dtype), num_encoder_layers, LayerNorm((d_model,), epsilon=layer_norm_eps))
        self.decoder = custom_decoder or TransformerDecoder(
            TransformerDecoderLayer(d_model, nhead, dim_feedforward, dropout, activation, layer_norm_eps, batch_first,
                                    norm_first, dtype), num_decoder_layers, LayerNorm((d_model,), epsilon=layer_norm_eps))
        self.d_model, self.nhead, self.batch_first = d_model, nhead, batch_first

    def construct(self, src, tgt, src_mask=None, tgt_mask=None, memory_mask=None, src_key_padding_mask=None,
                  tgt_key_padding_mask=None, memory_key_padding_mask=None):
        memory = self.encoder(src, src_mask, src_key_padding_mask)
        return self.decoder(tgt, memory, tgt_mask, memory_mask, tgt_key_padding_mask, memory_key_padding_mask)


# ------------------------------------------------------------------------------------------------ layout shuffles
class PixelShuffle(Cell):
    def __init__(self, upscale_factor):
        super().__init__()
        self.upscale_factor = upscale_factor

    def construct(self, x):
        return _wrap_out(F.pixel_shuffle(x, self.upscale_factor))


class PixelUnshuffle(Cell):
    def __init__(self, downscale_factor):
        super().__init__()
        self.downscale_factor = downscale_factor

    def construct(self, x):
        return _wrap_out(F.pixel_unshuffle(x, self.downscale_factor))


class ChannelShuffle(Cell):
    def __init__(self, groups):
        super().__init__()
        self.groups = groups

    def construct(self, x):
        return _wrap_out(F.channel_shuffle(x, self.groups))


class Unfold(Cell):
    """Sliding local blocks: [N, C, H, W] -> [N, C * kh * kw, L] (``ksizes`` / ``strides`` / ``rates`` given as
    [1, h, w, 1] like the reference's ``nn.Unfold``, or plain ints / pairs)."""

    def __init__(self, ksizes, strides=1, rates=1, padding="valid"):
        super().__init__()
        def hw(v):
            v = list(v) if isinstance(v, (list, tuple)) else [v, v]
            return tuple(v[1:3]) if len(v) == 4 else tuple(v)
        self.k, self.s, self.d = hw(ksizes), hw(strides), hw(rates)
        self.padding = padding

    def construct(self, x):
        if isinstance(self.padding, str) and self.padding.lower() == "same":
            pads = _same_pads(x.shape[2:], self.k, self.s, self.d)
            x = F.pad(x, [pads[1][0], pads[1][1], pads[0][0], pads[0][1]])
            pad = 0
        else:
            pad = 0 if isinstance(self.padding, str) else self.padding
        return _wrap_out(F.unfold(x, self.k, self.d, pad, self.s))


class Fold(Cell):
    def __init__(self, output_size, kernel_size, dilation=1, padding=0, stride=1):
        super().__init__()
        self.args = (output_size, kernel_size, dilation, padding, stride)

    def construct(self, x):
        return _wrap_out(F.fold(x, *self.args))


class MultiFieldEmbeddingLookup(Cell):
    """Embedding lookup whose ids are grouped into fields: (ids [B, L], weights [B, L], field_ids [B, L]) ->
    [B, field_size, D], combining the embeddings of one field by SUM / MEAN / MAX."""

    def __init__(self, vocab_size, embedding_size, field_size, param_init="normal", target="CPU", slice_mode="batch_slice",
                 feature_num_list=None, max_norm=None, sparse=True, operator="SUM", dtype=mstype.float32):
        super().__init__()
        if operator not in ("SUM", "MEAN", "MAX"):
            raise ValueError("For 'MultiFieldEmbeddingLookup', 'operator' must be SUM, MEAN or MAX, got %r" % operator)
        self.field_size, self.operator, self.max_norm = field_size, operator, max_norm
        self.embedding_table = Parameter(initializer(param_init, (vocab_size, embedding_size), dtype),
                                         name="embedding_table")

    def construct(self, input_indices, input_values, field_ids):
        emb = F.embedding(input_indices.long(), self.embedding_table, max_norm=self.max_norm)
        emb = emb * input_values.unsqueeze(-1).to(emb.dtype)
        B, L, D = emb.shape
        onehot = F.one_hot(field_ids.long().clamp_min(0), self.field_size).to(emb.dtype)        # [B, L, F]
        valid = (field_ids >= 0).unsqueeze(-1).to(emb.dtype)
        onehot = onehot * valid
        if self.operator == "MAX":
            big = emb.unsqueeze(2).expand(B, L, self.field_size, D)
            masked = torch.where(onehot.unsqueeze(-1) > 0, big, torch.full_like(big, float("-inf")))
            out = masked.amax(1)
            return _wrap_out(torch.where(torch.isinf(out), torch.zeros_like(out), out))
        out = torch.einsum("blf,bld->bfd", onehot, emb)
        if self.operator == "MEAN":
            cnt = torch.einsum("blf,bl->bf", onehot, input_values.to(emb.dtype)).clamp_min(1e-12)
            out = out / cnt.unsqueeze(-1)
        return _wrap_out(out)


# ------------------------------------------------------------------------------------------------ simple functional layers
def _fn_cell(name, fn, arg_names=(), defaults=(), doc=None):
    """Cell whose constructor stores ``arg_names`` and whose construct calls ``fn(x, *stored)``."""
    def __init__(self, *args, **kwargs):
        Cell.__init__(self)
        vals = dict(zip(arg_names, defaults))
        vals.update(dict(zip(arg_names, args)))
        for k, v in kwargs.items():
            if k not in arg_names:
                raise TypeError("%s got an unexpected keyword argument %r" % (name, k))
            vals[k] = v
        missing = [a for a in arg_names if a not in vals]
        if missing:
            raise TypeError("%s missing required arguments: %s" % (name, ", ".join(missing)))
        for k, v in vals.items():
            object.__setattr__(self, k, v)

    def construct(self, x, *more):
        return _wrap_out(fn(x, *more, *[getattr(self, a) for a in arg_names]))

    cls = type(name, (Cell,), {"__init__": __init__, "construct": construct, "__doc__": doc or "%s layer." % name})
    globals()[name] = cls
    __all__.append(name)
    return cls


def _pad_cell(name, nd, mode):
    def __init__(self, padding, value=0.0):
        Cell.__init__(self)
        p = (padding,) * (2 * nd) if isinstance(padding, int) else tuple(padding)
        if len(p) != 2 * nd:
            raise ValueError("%s needs an int or %d padding values, got %r" % (name, 2 * nd, padding))
        self.padding, self.value = p, value

    def construct(self, x):
        if mode == "constant":
            return _wrap_out(F.pad(x, self.padding, value=self.value))
        return _wrap_out(F.pad(x, self.padding, mode=mode))

    cls = type(name, (Cell,), {"__init__": __init__, "construct": construct,
                               "__doc__": "%s padding of the last %d dims." % (mode, nd)})
    globals()[name] = cls
    __all__.append(name)


for _nd in (1, 2, 3):
    _pad_cell("ReflectionPad%dd" % _nd, _nd, "reflect")
    _pad_cell("ReplicationPad%dd" % _nd, _nd, "replicate")
    _pad_cell("ConstantPad%dd" % _nd, _nd, "constant")


class ZeroPad2d(ConstantPad2d):      # noqa: F821
    def __init__(self, padding):
        super().__init__(padding, 0.0)


__all__.append("ZeroPad2d")

_fn_cell("MaxPool3d", lambda x, k, s, p, d, c: F.max_pool3d(x, k, s if s is not None else k, p, d, c),
         ("kernel_size", "stride", "padding", "dilation", "ceil_mode"), (1, None, 0, 1, False))
_fn_cell("AvgPool3d", lambda x, k, s, p, c, cip: F.avg_pool3d(x, k, s if s is not None else k, p, c, cip),
         ("kernel_size", "stride", "padding", "ceil_mode", "count_include_pad"), (1, None, 0, False, True))
_fn_cell("AdaptiveAvgPool1d", F.adaptive_avg_pool1d, ("output_size",))
_fn_cell("AdaptiveAvgPool3d", F.adaptive_avg_pool3d, ("output_size",))
_fn_cell("AdaptiveMaxPool1d", F.adaptive_max_pool1d, ("output_size",))
_fn_cell("AdaptiveMaxPool3d", F.adaptive_max_pool3d, ("output_size",))
_fn_cell("LPPool1d", lambda x, n, k, s, c: F.lp_pool1d(x, n, k, s, c), ("norm_type", "kernel_size", "stride", "ceil_mode"),
         (2, 1, None, False))
_fn_cell("LPPool2d", lambda x, n, k, s, c: F.lp_pool2d(x, n, k, s, c), ("norm_type", "kernel_size", "stride", "ceil_mode"),
         (2, 1, None, False))
_fn_cell("LRN", lambda x, r, b, a, be, nr="ACROSS_CHANNELS": F.local_response_norm(x, 2 * r + 1, a * (2 * r + 1), be, b),
         ("depth_radius", "bias", "alpha", "beta", "norm_region"), (5, 1.0, 1.0, 0.5, "ACROSS_CHANNELS"))
_fn_cell("Softmin", lambda x, axis: F.softmin(x, axis), ("axis",), (-1,))
_fn_cell("Softmax2d", lambda x: F.softmax(x, -3))
_fn_cell("Hardswish", F.hardswish)
_fn_cell("Hardsigmoid", F.hardsigmoid)
_fn_cell("SELU", F.selu)
_fn_cell("CELU", lambda x, alpha: F.celu(x, alpha), ("alpha",), (1.0,))
_fn_cell("Swish", F.silu)
_fn_cell("HShrink", lambda x, lambd: F.hardshrink(x, lambd), ("lambd",), (0.5,))
_fn_cell("SoftShrink", lambda x, lambd: F.softshrink(x, lambd), ("lambd",), (0.5,))
Hardshrink, Softshrink = HShrink, SoftShrink      # noqa: F821
__all__ += ["Hardshrink", "Softshrink"]
_fn_cell("Roll", lambda x, shift, axis: torch.roll(x, shift, axis), ("shift", "axis"))
_fn_cell("Tril", lambda x, k=0: torch.tril(x, k))
_fn_cell("Triu", lambda x, k=0: torch.triu(x, k))
_fn_cell("Unflatten", lambda x, axis, unflattened_size: torch.unflatten(x, axis, tuple(unflattened_size)),
         ("axis", "unflattened_size"))
_fn_cell("Norm", lambda x, axis, keep_dims: torch.linalg.vector_norm(x, 2, axis if axis != () else None, keep_dims),
         ("axis", "keep_dims"), ((), False))
_fn_cell("CosineSimilarity", lambda a, b, dim, eps: F.cosine_similarity(a, b, dim, eps), ("dim", "eps"), (1, 1e-8))
_fn_cell("PairwiseDistance", lambda a, b, p, eps, keepdim: F.pairwise_distance(a, b, p, eps, keepdim),
         ("p", "eps", "keepdim"), (2.0, 1e-6, False))
_fn_cell("MaxUnpool2d", lambda x, idx, k, s, p: F.max_unpool2d(x, idx.long(), k, s, p), ("kernel_size", "stride", "padding"),
         (1, None, 0))


class RReLU(Cell):
    def __init__(self, lower=1 / 8, upper=1 / 3):
        super().__init__()
        self.lower, self.upper = lower, upper

    def construct(self, x):
        return _wrap_out(F.rrelu(x, self.lower, self.upper, self.training))


class _DropoutNd(Cell):
    _fn = staticmethod(F.dropout2d)

    def __init__(self, p=0.5):
        super().__init__()
        if not 0 <= p < 1:
            raise ValueError("dropout probability must be in [0, 1), got %r" % (p,))
        self.p = p

    def construct(self, x):
        return _wrap_out(type(self)._fn(x, self.p, self.training))


class Dropout1d(_DropoutNd):
    _fn = staticmethod(F.dropout1d)


class Dropout2d(_DropoutNd):
    _fn = staticmethod(F.dropout2d)


class Dropout3d(_DropoutNd):
    _fn = staticmethod(F.dropout3d)


class ResizeBilinear(Cell):
    def __init__(self, half_pixel_centers=False):
        super().__init__()
        self.half_pixel_centers = half_pixel_centers

    def construct(self, x, size=None, scale_factor=None, align_corners=False):
        return _wrap_out(F.interpolate(x, size=size, scale_factor=scale_factor, mode="bilinear",
                                       align_corners=align_corners))


class FractionalMaxPool2d(Cell):
    def __init__(self, kernel_size, output_size=None, output_ratio=None, return_indices=False, _random_samples=None):
        super().__init__()
        self.args = (kernel_size, output_size, output_ratio, return_indices, _random_samples)

    def construct(self, x):
        k, o, r, ri, rs = self.args
        return _wrap_out(F.fractional_max_pool2d(x, k, o, r, ri, rs))


class ClipByNorm(Cell):
    def __init__(self, axis=None):
        super().__init__()
        self.axis = axis

    def construct(self, x, clip_norm):
        n = torch.linalg.vector_norm(x.float(), 2, self.axis, keepdim=self.axis is not None)
        c = torch.as_tensor(clip_norm, dtype=torch.float32, device=x.device)
        return _wrap_out((x.float() * (c / torch.maximum(n, c))).to(x.dtype))


class L1Regularizer(Cell):
    def __init__(self, scale):
        super().__init__()
        if scale <= 0:
            raise ValueError("For 'L1Regularizer', 'scale' must be positive, got %r" % (scale,))
        self.scale = scale

    def construct(self, weights):
        return _wrap_out(self.scale * weights.abs().sum())


class BiDense(Cell):
    """y = x1^T W x2 + b with W [out, in1, in2]."""

    def __init__(self, in1_channels, in2_channels, out_channels, weight_init=None, bias_init=None, has_bias=True,
                 dtype=mstype.float32):
        super().__init__()
        k = 1 / math.sqrt(in1_channels)
        self.weight = Parameter(initializer(weight_init or Uniform(k), (out_channels, in1_channels, in2_channels), dtype),
                                name="weight")
        self.bias = Parameter(initializer(bias_init or Uniform(k), (out_channels,), dtype), name="bias") if has_bias else None

    def construct(self, x1, x2):
        return _wrap_out(F.bilinear(x1, x2, self.weight, self.bias))


Bilinear = BiDense
__all__ += ["RReLU", "Dropout1d", "Dropout2d", "Dropout3d", "ResizeBilinear", "FractionalMaxPool2d", "ClipByNorm",
            "L1Regularizer", "BiDense", "Bilinear"]


# ------------------------------------------------------------------------------------------------ math / image / wrappers
_fn_cell("ReduceLogSumExp", lambda x, axis, keep_dims: torch.logsumexp(x, axis, keep_dims), ("axis", "keep_dims"), (None, False))
_fn_cell("LGamma", torch.lgamma)
_fn_cell("DiGamma", torch.digamma)
_fn_cell("IGamma", lambda a, x: torch.special.gammainc(a, x))
_fn_cell("LBeta", lambda x, y: torch.lgamma(x) + torch.lgamma(y) - torch.lgamma(x + y))
_fn_cell("MatDet", torch.linalg.det)
_fn_cell("MatInverse", torch.linalg.inv)
_fn_cell("MatrixDiag", torch.diag_embed)
_fn_cell("MatrixDiagPart", lambda x: torch.diagonal(x, dim1=-2, dim2=-1))
_fn_cell("MatrixSetDiag", lambda x, d: x - torch.diag_embed(torch.diagonal(x, dim1=-2, dim2=-1)) + torch.diag_embed(d))
def _moments(x, axis, keep_dims):
    t = x.float().as_subclass(torch.Tensor)
    dims = tuple(range(t.dim())) if axis is None else axis
    return torch.mean(t, dims, bool(keep_dims)), torch.var(t, dims, unbiased=False, keepdim=bool(keep_dims))


_fn_cell("Moments", _moments, ("axis", "keep_dims"), (None, None))


class MatMul(Cell):
    def __init__(self, transpose_x1=False, transpose_x2=False):
        super().__init__()
        self.t1, self.t2 = transpose_x1, transpose_x2

    def construct(self, x1, x2):
        a = x1.transpose(-1, -2) if self.t1 else x1
        b = x2.transpose(-1, -2) if self.t2 else x2
        return _wrap_out(torch.matmul(a, b))


class Range(Cell):
    def __init__(self, start, limit=None, delta=1):
        super().__init__()
        if limit is None:
            start, limit = 0, start
        self.args = (start, limit, delta)

    def construct(self):
        return _wrap_out(torch.arange(*self.args))


class CentralCrop(Cell):
    def __init__(self, central_fraction):
        super().__init__()
        if not 0 < central_fraction <= 1:
            raise ValueError("For 'CentralCrop', 'central_fraction' must be in (0, 1], got %r" % (central_fraction,))
        self.f = central_fraction

    def construct(self, image):
        h, w = image.shape[-2:]
        ch, cw = int(h * self.f), int(w * self.f)
        t, l = (h - ch) // 2, (w - cw) // 2
        return _wrap_out(image[..., t:t + ch, l:l + cw])


class ImageGradients(Cell):
    def construct(self, images):
        dy = torch.zeros_like(images)
        dx = torch.zeros_like(images)
        dy[..., :-1, :] = images[..., 1:, :] - images[..., :-1, :]
        dx[..., :, :-1] = images[..., :, 1:] - images[..., :, :-1]
        return _wrap_out(dy), _wrap_out(dx)


class PSNR(Cell):
    def __init__(self, max_val=1.0):
        super().__init__()
        self.max_val = float(max_val)

    def construct(self, img1, img2):
        mse = ((img1.float() - img2.float()) ** 2).mean((-3, -2, -1))
        return _wrap_out(10 * torch.log10(self.max_val ** 2 / mse))


def _gauss_window(size, sigma, channels, device):
    x = torch.arange(size, dtype=torch.float32, device=device) - (size - 1) / 2
    g = torch.exp(-x * x / (2 * sigma * sigma))
    g = g / g.sum()
    return (g[:, None] * g[None]).expand(channels, 1, size, size).contiguous()


def _ssim_terms(a, b, max_val, size, sigma, k1, k2):
    c = a.shape[1]
    w = _gauss_window(size, sigma, c, a.device)
    mu_a, mu_b = F.conv2d(a, w, groups=c), F.conv2d(b, w, groups=c)
    va = F.conv2d(a * a, w, groups=c) - mu_a ** 2
    vb = F.conv2d(b * b, w, groups=c) - mu_b ** 2
    cov = F.conv2d(a * b, w, groups=c) - mu_a * mu_b
    c1, c2 = (k1 * max_val) ** 2, (k2 * max_val) ** 2
    cs = (2 * cov + c2) / (va + vb + c2)
    return ((2 * mu_a * mu_b + c1) / (mu_a ** 2 + mu_b ** 2 + c1)) * cs, cs


class SSIM(Cell):
    def __init__(self, max_val=1.0, filter_size=11, filter_sigma=1.5, k1=0.01, k2=0.03):
        super().__init__()
        self.args = (float(max_val), int(filter_size), float(filter_sigma), k1, k2)

    def construct(self, img1, img2):
        ssim, _ = _ssim_terms(img1.float(), img2.float(), *self.args)
        return _wrap_out(ssim.mean((-3, -2, -1)))


class MSSSIM(Cell):
    def __init__(self, max_val=1.0, power_factors=(0.0448, 0.2856, 0.3001, 0.2363, 0.1333), filter_size=11,
                 filter_sigma=1.5, k1=0.01, k2=0.03):
        super().__init__()
        self.weights = tuple(power_factors)
        self.args = (float(max_val), int(filter_size), float(filter_sigma), k1, k2)

    def construct(self, img1, img2):
        a, b = img1.float(), img2.float()
        out = 1.0
        for i, w in enumerate(self.weights):
            ssim, cs = _ssim_terms(a, b, *self.args)
            last = i == len(self.weights) - 1
            term = (ssim if last else cs).mean((-3, -2, -1)).clamp_min(0)
            out = out * term ** w
            if not last:
                a, b = F.avg_pool2d(a, 2), F.avg_pool2d(b, 2)
        return _wrap_out(out)


class TimeDistributed(Cell):
    """Applies ``layer`` to every slice along ``time_axis`` (folded into the batch axis for the call)."""

    def __init__(self, layer, time_axis, reshape_with_axis=None):
        super().__init__()
        self.layer, self.time_axis, self.reshape_with_axis = layer, time_axis, reshape_with_axis

    def construct(self, x):
        t = self.time_axis % x.dim()
        moved = x.movedim(t, 1) if t != 1 else x
        b, steps = moved.shape[0], moved.shape[1]
        y = self.layer(_wrap_out(moved.reshape((b * steps,) + tuple(moved.shape[2:]))))
        y = y.reshape((b, steps) + tuple(y.shape[1:]))
        return _wrap_out(y.movedim(1, t) if t != 1 else y)


class ParameterUpdate(Cell):
    """Cell whose call assigns a new value to ``param`` (e.g. to change a learning-rate parameter from outside)."""

    def __init__(self, param):
        super().__init__(auto_prefix=False)
        if not isinstance(param, Parameter):
            raise TypeError("For 'ParameterUpdate', 'param' must be a Parameter, got %s" % type(param).__name__)
        self._param = param

    def construct(self, x):
        with torch.no_grad():
            self._param.copy_(torch.as_tensor(x).to(self._param.dtype).reshape(self._param.shape))
        return x


class Jvp(Cell):
    def __init__(self, fn):
        super().__init__(auto_prefix=False)
        self.fn = fn

    def construct(self, *args):
        from ..ops.composite import jvp
        n = len(args) // 2
        inputs, v = args[:n], args[n:]
        return jvp(self.fn, inputs if n > 1 else inputs[0], v if n > 1 else v[0])


class Vjp(Cell):
    def __init__(self, fn):
        super().__init__(auto_prefix=False)
        self.fn = fn

    def construct(self, *args):
        from ..ops.composite import vjp
        inputs, v = args[:-1], args[-1]
        out, fn = vjp(self.fn, *inputs)
        return out, fn(v)


class VirtualDatasetCellTriple(Cell):
    def __init__(self, backbone):
        super().__init__(auto_prefix=False)
        self._backbone = backbone

    def construct(self, a, b, c):
        return self._backbone(a, b, c)


class SparseToDense(Cell):
    def construct(self, coo_tensor):
        return coo_tensor.to_dense()


class SparseTensorDenseMatmul(Cell):
    def __init__(self, adjoint_st=False, adjoint_dt=False):
        super().__init__()
        self.adj_s, self.adj_d = adjoint_st, adjoint_dt

    def construct(self, indices, values, sparse_shape, dense):
        s = torch.sparse_coo_tensor(indices.t().long(), values, tuple(int(v) for v in sparse_shape)).to_dense()
        s = s.t() if self.adj_s else s
        d = dense.t() if self.adj_d else dense
        return _wrap_out(s @ d)


__all__ += ["MatMul", "Range", "CentralCrop", "ImageGradients", "PSNR", "SSIM", "MSSSIM", "TimeDistributed",
            "ParameterUpdate", "Jvp", "Vjp", "VirtualDatasetCellTriple", "SparseToDense", "SparseTensorDenseMatmul"]


# ------------------------------------------------------------------------------------------------ combined / THOR layers
_fn_cell("MaxUnpool1d", lambda x, idx, k, s, p: F.max_unpool1d(x, idx.long(), k, s, p),
         ("kernel_size", "stride", "padding"), (1, None, 0))
_fn_cell("MaxUnpool3d", lambda x, idx, k, s, p: F.max_unpool3d(x, idx.long(), k, s, p),
         ("kernel_size", "stride", "padding"), (1, None, 0))


class FractionalMaxPool3d(Cell):
    def __init__(self, kernel_size, output_size=None, output_ratio=None, return_indices=False, _random_samples=None):
        super().__init__()
        self.args = (kernel_size, output_size, output_ratio, return_indices, _random_samples)

    def construct(self, x):
        k, o, r, ri, rs = self.args
        return _wrap_out(F.fractional_max_pool3d(x, k, o, r, ri, rs))


class DropoutExt(Dropout):
    """``Dropout`` with the probability of zeroing as its only argument."""

    def __init__(self, p=0.5):
        super().__init__(p=p)


class Conv2dBnAct(Cell):
    """Conv2d, then optionally BatchNorm2d, then optionally an activation (``'relu'``, ``'leakyrelu'`` with
    ``alpha``, any name ``get_activation`` knows, or a Cell).  Parity: nn/layer/combined.py (Conv2dBnAct)."""

    def __init__(self, in_channels, out_channels, kernel_size, stride=1, pad_mode="same", padding=0, dilation=1,
                 group=1, has_bias=False, weight_init="normal", bias_init="zeros", has_bn=False, momentum=0.997,
                 eps=1e-5, activation=None, alpha=0.2, after_fake=True, dtype=mstype.float32):
        super().__init__()
        from .layer import BatchNorm2d, Conv2d, LeakyReLU, get_activation
        self.conv = Conv2d(in_channels, out_channels, kernel_size, stride, pad_mode, padding, dilation, group,
                           has_bias, weight_init, bias_init, dtype=dtype)
        self.has_bn = has_bn
        if has_bn:
            self.batchnorm = BatchNorm2d(out_channels, eps, momentum)
        if activation == "leakyrelu":
            self.activation = LeakyReLU(alpha)
        else:
            self.activation = get_activation(activation) if isinstance(activation, str) else activation
        self.has_act = self.activation is not None

    def construct(self, x):
        x = self.conv(x)
        if self.has_bn:
            x = self.batchnorm(x)
        return self.activation(x) if self.has_act else x


class DenseBnAct(Cell):
    """Dense, then optionally BatchNorm1d, then optionally an activation.  Parity: nn/layer/combined.py."""

    def __init__(self, in_channels, out_channels, weight_init="normal", bias_init="zeros", has_bias=True,
                 has_bn=False, momentum=0.9, eps=1e-5, activation=None, alpha=0.2, after_fake=True,
                 dtype=mstype.float32):
        super().__init__()
        from .layer import BatchNorm1d, LeakyReLU, get_activation
        self.dense = Dense(in_channels, out_channels, weight_init, bias_init, has_bias, dtype=dtype)
        self.has_bn = has_bn
        if has_bn:
            self.batchnorm = BatchNorm1d(out_channels, eps, momentum)
        if activation == "leakyrelu":
            self.activation = LeakyReLU(alpha)
        else:
            self.activation = get_activation(activation) if isinstance(activation, str) else activation
        self.has_act = self.activation is not None

    def construct(self, x):
        x = self.dense(x)
        if self.has_bn:
            x = self.batchnorm(x)
        return self.activation(x) if self.has_act else x


class DenseThor(Dense):
    """``Dense`` as the THOR optimizer's layer type: carries the Kronecker factors ``matrix_a`` (input second
    moment) and ``matrix_g`` (output-gradient second moment) as non-trainable parameters; ``nn.THOR`` fills them
    from hooks on any Dense layer, this class only provides the named state the reference's checkpoints hold.
    Parity: nn/layer/thor_layer.py (DenseThor)."""

    def __init__(self, in_channels, out_channels, weight_init="normal", bias_init="zeros", has_bias=True,
                 activation=None):
        super().__init__(in_channels, out_channels, weight_init, bias_init, has_bias, activation)
        self.thor = True
        self.matrix_a = Parameter(torch.eye(in_channels), name="matrix_a", requires_grad=False)
        self.matrix_g = Parameter(torch.eye(out_channels), name="matrix_g", requires_grad=False)


def _thor_conv():
    from .layer import Conv2d

    class Conv2dThor(Conv2d):
        """``Conv2d`` with the THOR factor state (``matrix_a`` over in_channels * kh * kw, ``matrix_g`` over
        out_channels).  Parity: nn/layer/thor_layer.py (Conv2dThor)."""

        def __init__(self, in_channels, out_channels, kernel_size, stride=1, pad_mode="same", padding=0, dilation=1,
                     group=1, has_bias=False, weight_init="normal", bias_init="zeros"):
            super().__init__(in_channels, out_channels, kernel_size, stride, pad_mode, padding, dilation, group,
                             has_bias, weight_init, bias_init)
            self.thor = True
            a_dim = in_channels * self.kernel_size[0] * self.kernel_size[1]
            self.matrix_a = Parameter(torch.eye(a_dim), name="matrix_a", requires_grad=False)
            self.matrix_g = Parameter(torch.eye(out_channels), name="matrix_g", requires_grad=False)
    return Conv2dThor


def _thor_embeddings():
    from .layer import Embedding, EmbeddingLookup

    class EmbeddingThor(Embedding):
        """``Embedding`` with the THOR factor state: ``matrix_a`` is diagonal (token frequencies, [vocab_size]),
        ``matrix_g`` is [embedding_size, embedding_size].  Parity: nn/layer/thor_layer.py (EmbeddingThor)."""

        def __init__(self, vocab_size, embedding_size, use_one_hot=False, embedding_table="normal",
                     dtype=mstype.float32, padding_idx=None):
            super().__init__(vocab_size, embedding_size, use_one_hot, embedding_table, dtype, padding_idx)
            self.thor = True
            self.matrix_a = Parameter(torch.ones(vocab_size), name="matrix_a", requires_grad=False)
            self.matrix_g = Parameter(torch.eye(embedding_size), name="matrix_g", requires_grad=False)

    class EmbeddingLookupThor(EmbeddingLookup):
        """``EmbeddingLookup`` with the THOR factor state.  Parity: nn/layer/thor_layer.py (EmbeddingLookupThor)."""

        def __init__(self, vocab_size, embedding_size, param_init="normal", target="CPU", slice_mode="batch_slice",
                     manual_shapes=None, max_norm=None, sparse=True, vocab_cache_size=0):
            super().__init__(vocab_size, embedding_size, param_init, target, slice_mode, manual_shapes, max_norm,
                             sparse, vocab_cache_size)
            self.thor = True
            self.matrix_a = Parameter(torch.ones(vocab_size), name="matrix_a", requires_grad=False)
            self.matrix_g = Parameter(torch.eye(embedding_size), name="matrix_g", requires_grad=False)
    return EmbeddingThor, EmbeddingLookupThor


Conv2dThor = _thor_conv()
EmbeddingThor, EmbeddingLookupThor = _thor_embeddings()
__all__ += ["FractionalMaxPool3d", "DropoutExt", "Conv2dBnAct", "DenseBnAct", "DenseThor", "Conv2dThor",
            "EmbeddingThor", "EmbeddingLookupThor"]


class TensorArray(Cell):
    """A growable (``dynamic_size``) or fixed-size list of tensors of one dtype and element shape:
    ``write(index, value)``, ``read(index)``, ``size()``, ``stack()``, ``clear()``, ``close()``.
    Parity: nn/reinforcement/tensor_array.py."""

    def __init__(self, dtype, element_shape, dynamic_size=True, size=0, name="TA"):
        super().__init__()
        if not isinstance(element_shape, (tuple, list)):
            raise TypeError("For 'TensorArray', 'element_shape' must be a tuple or a list")
        if isinstance(size, bool) or not isinstance(size, int) or size < 0:
            raise ValueError("For 'TensorArray', 'size' must be a non-negative int")
        self.dtype, self.element_shape = dtype, tuple(element_shape)
        self.dynamic_size, self.max_size, self.array_name = bool(dynamic_size), size, name
        self._items = [None] * (0 if dynamic_size else size)
        self._closed = False

    def _check(self):
        if self._closed:
            raise RuntimeError("For 'TensorArray', the array %r has been closed" % self.array_name)

    def write(self, index, value):
        self._check()
        index = int(index)
        value = torch.as_tensor(value)
        if value.dtype != self.dtype or tuple(value.shape) != self.element_shape:
            raise TypeError("For 'TensorArray.write', the value must be %s of shape %s, but got %s of shape %s"
                            % (self.dtype, self.element_shape, value.dtype, tuple(value.shape)))
        if index < 0:
            raise ValueError("For 'TensorArray.write', 'index' must not be negative")
        if index >= len(self._items):
            if not self.dynamic_size:
                raise ValueError("For 'TensorArray.write', index %d is out of the fixed size %d"
                                 % (index, len(self._items)))
            self._items.extend([None] * (index + 1 - len(self._items)))
        self._items[index] = value.clone()
        return True

    def read(self, index):
        self._check()
        index = int(index)
        if index < 0 or index >= len(self._items):
            raise ValueError("For 'TensorArray.read', index %d is out of range (size %d)" % (index, len(self._items)))
        item = self._items[index]
        return torch.zeros(self.element_shape, dtype=self.dtype) if item is None else item

    def size(self):
        self._check()
        return len(self._items)

    def stack(self):
        self._check()
        if not self._items:
            return torch.zeros((0,) + self.element_shape, dtype=self.dtype)
        return torch.stack([self.read(k) for k in range(len(self._items))])

    def clear(self):
        self._check()
        self._items = [None] * (0 if self.dynamic_size else self.max_size)
        return True

    def close(self):
        self._items, self._closed = [], True
        return True


class Linear(Dense):
    """``Dense`` under the argument names of the extend namespace: ``Linear(in_features, out_features, bias=True)``.
    Parity: nn/extend/basic.py."""

    def __init__(self, in_features, out_features, bias=True, weight_init=None, bias_init=None, dtype=None):
        kwargs = {} if dtype is None else {"dtype": dtype}
        super().__init__(in_features, out_features, weight_init if weight_init is not None else "normal",
                         bias_init if bias_init is not None else "zeros", has_bias=bias, **kwargs)
        self.in_features, self.out_features = in_features, out_features


__all__ += ["TensorArray", "Linear"]
