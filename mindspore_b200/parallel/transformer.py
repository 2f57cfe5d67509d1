"""GPT-style model-parallel transformer blocks (the reference's ``parallel._transformer`` / ``nn.transformer``).

``TransformerOpParallelConfig`` describes the device mesh ``pipeline_stage x data_parallel x model_parallel`` (rank
order: model-parallel ranks are adjacent, then data-parallel, then pipeline stages) and creates the communication
groups.  The layers are written against those groups with explicit, differentiable collectives and sequence
parallelism between tensor-parallel regions (``parallel.tp``); activations are token-major ``[batch*seq, hidden]``.

Parity: python/mindspore/parallel/_transformer/op_parallel_config.py:44-200, transformer.py:60
(EmbeddingOpParallelConfig), :118 (TransformerRecomputeConfig), :191 (TransformerOpParallelConfig), :349
(FeedForward), :597 (AttentionMask), :671 (VocabEmbedding), :756 (MultiHeadAttention), :1365
(TransformerEncoderLayer), :1777 (TransformerDecoderLayer), :2276 (TransformerEncoder), :2532 (TransformerDecoder),
:2780 (Transformer); layers.py:261 (_LayerNorm), :347 (_Linear), :545 (FixedSparseAttention); loss.py:157
(CrossEntropyLoss)."""
from __future__ import annotations

import math

import torch

from .. import context
from ..common.initializer import Normal, initializer
from ..common.parameter import Parameter
from ..communication import management as M
from ..nn.cell import Cell
from ..nn.layer import CellList
from ..ops import fused
from . import tp as TP
from .moe import MoE, MoEConfig, Router, TopkRouter, default_moe_config


class TransformerRecomputeConfig:
    def __init__(self, recompute=False, parallel_optimizer_comm_recompute=False, mp_comm_recompute=True,
                 recompute_slice_activation=False):
        for n, v in (("recompute", recompute), ("parallel_optimizer_comm_recompute", parallel_optimizer_comm_recompute),
                     ("mp_comm_recompute", mp_comm_recompute), ("recompute_slice_activation", recompute_slice_activation)):
            if not isinstance(v, bool):
                raise TypeError("'%s' must be bool, but got %s" % (n, type(v).__name__))
        self.recompute, self.mp_comm_recompute = recompute, mp_comm_recompute
        self.parallel_optimizer_comm_recompute = parallel_optimizer_comm_recompute
        self.recompute_slice_activation = recompute_slice_activation


class EmbeddingOpParallelConfig:
    def __init__(self, data_parallel=1, model_parallel=1, vocab_emb_dp=True):
        self.data_parallel, self.model_parallel, self.vocab_emb_dp = data_parallel, model_parallel, vocab_emb_dp


class TransformerOpParallelConfig:
    def __init__(self, data_parallel=1, model_parallel=1, expert_parallel=1, pipeline_stage=1, micro_batch_num=1,
                 recompute=None, optimizer_shard=False, gradient_aggregation_group=4, vocab_emb_dp=True,
                 sequence_parallel=True):
        for n, v in (("data_parallel", data_parallel), ("model_parallel", model_parallel),
                     ("expert_parallel", expert_parallel), ("pipeline_stage", pipeline_stage),
                     ("micro_batch_num", micro_batch_num), ("gradient_aggregation_group", gradient_aggregation_group)):
            if not isinstance(v, int) or isinstance(v, bool) or v <= 0:
                raise TypeError("'%s' must be a positive int, but got %r" % (n, v))
        if isinstance(recompute, bool):
            recompute = TransformerRecomputeConfig(recompute=recompute)
        self.recompute = recompute or TransformerRecomputeConfig()
        self.data_parallel, self.model_parallel, self.expert_parallel = data_parallel, model_parallel, expert_parallel
        self.pipeline_stage, self.micro_batch_num = pipeline_stage, micro_batch_num
        self.optimizer_shard, self.gradient_aggregation_group = optimizer_shard, gradient_aggregation_group
        self.vocab_emb_dp, self.sequence_parallel = vocab_emb_dp, sequence_parallel
        self._groups = None

    @property
    def embedding_dp_mp_config(self):
        return EmbeddingOpParallelConfig(self.data_parallel, self.model_parallel, self.vocab_emb_dp)

    @property
    def dp_mp_config(self):
        return self

    def groups(self):
        """Creates (once; collective over the world) the model-, data- and expert-parallel groups of this rank.
        Returns a dict with ``tp`` (TPGroup), ``dp`` / ``ep`` (group names or None), ``stage``."""
        if self._groups is not None:
            return self._groups
        dp, mp, pp = self.data_parallel, self.model_parallel, self.pipeline_stage
        if not M.GlobalComm.INITED or dp * mp * pp == 1:
            self._groups = {"tp": TP.TPGroup(name=None, size=1, rank=0), "dp": None, "ep": None, "stage": 0,
                            "dp_size": 1}
            return self._groups
        world, rank = M.get_group_size(), M.get_rank()
        if dp * mp * pp != world:
            raise ValueError("data_parallel * model_parallel * pipeline_stage = %d does not match the %d devices"
                             % (dp * mp * pp, world))
        if dp % self.expert_parallel:
            raise ValueError("data_parallel (%d) must be a multiple of expert_parallel (%d)"
                             % (dp, self.expert_parallel))
        my = {"stage": rank // (dp * mp), "dp_size": dp}
        for s in range(pp):                                # every rank creates every group, in the same order
            base = s * dp * mp
            for d in range(dp):
                ranks = [base + d * mp + m for m in range(mp)]
                name = M.group_for_ranks(ranks) if mp > 1 else None
                if rank in ranks:
                    my["tp"] = TP.TPGroup(name=name, size=mp, rank=ranks.index(rank)) if mp > 1 else \
                        TP.TPGroup(name=None, size=1, rank=0)
            for m in range(mp):
                ranks = [base + d * mp + m for d in range(dp)]
                name = M.group_for_ranks(ranks) if dp > 1 else None
                if rank in ranks:
                    my["dp"] = name
                ep = self.expert_parallel
                for g0 in range(0, dp, ep):
                    sub = ranks[g0:g0 + ep]
                    ename = M.group_for_ranks(sub) if ep > 1 else None
                    if rank in sub:
                        my["ep"] = ename
        self._groups = my
        return my


default_transformer_config = TransformerOpParallelConfig()


def _mat(shape, std, dtype, name, tp_sharded):
    p = Parameter(initializer(Normal(std), shape, dtype), name=name)
    p.tp_sharded = tp_sharded
    return p


def _vec(n, value, dtype, name, tp, sp, sharded=False):
    p = Parameter(torch.full((n,), value, dtype=dtype), name=name)
    p.tp_sharded = sharded
    # replicated over the model-parallel group but fed by token-sharded activations: gradients are partial sums
    p.tp_grad_reduce = (not sharded) and tp.active and sp
    return p


class _LayerNorm(Cell):
    def __init__(self, normalized_shape, eps=1e-5, param_init_type=torch.float32, tp=None, sequence_parallel=True):
        super().__init__()
        n = normalized_shape[-1] if isinstance(normalized_shape, (tuple, list)) else int(normalized_shape)
        tp = tp or TP.TPGroup(name=None, size=1, rank=0)
        self.gamma = _vec(n, 1.0, param_init_type, "gamma", tp, sequence_parallel)
        self.beta = _vec(n, 0.0, param_init_type, "beta", tp, sequence_parallel)
        self.eps = eps

    def construct(self, x):
        return fused.layer_norm(x, self.gamma, self.beta, self.eps)

    def shard(self, strategy):
        return self


class _Linear(Cell):
    """Dense with optional expert dimension (``expert_num`` > 1 makes it a batched matmul over experts)."""

    def __init__(self, in_channels, out_channels, has_bias=True, activation=None, expert_num=1,
                 param_init_type=torch.float32, std=0.02):
        super().__init__()
        shape = (out_channels, in_channels) if expert_num == 1 else (expert_num, in_channels, out_channels)
        self.expert_num = expert_num
        self.weight = _mat(shape, std, param_init_type, "weight", False)
        self.bias = Parameter(torch.zeros((out_channels,) if expert_num == 1 else (expert_num, 1, out_channels),
                                          dtype=param_init_type), name="bias") if has_bias else None
        self.activation = activation

    def construct(self, x):
        if self.expert_num == 1:
            y = fused.linear(x.reshape(-1, x.shape[-1]), self.weight, self.bias).reshape(*x.shape[:-1], -1)
        else:
            y = fused.matmul(x, self.weight)
            if self.bias is not None:
                y = y + self.bias
        if self.activation == "gelu":
            y = torch.nn.functional.gelu(y, approximate="tanh")
        elif self.activation == "relu":
            y = torch.relu(y)
        return y


class VocabEmbedding(Cell):
    """Token embedding with the table split over the model-parallel group along the vocabulary
    (``vocab_emb_dp=False``) or replicated (``True``).  Returns (embeddings [T(/mp), H], table)."""

    def __init__(self, vocab_size, embedding_size, parallel_config=None, param_init="normal",
                 param_init_type=torch.float32, tp=None, sequence_parallel=True):
        super().__init__()
        self.tp = tp or TP.TPGroup(name=None, size=1, rank=0)
        self.sp = sequence_parallel
        self.split_vocab = self.tp.active and not (parallel_config.vocab_emb_dp if parallel_config else False)
        rows = vocab_size // self.tp.size if self.split_vocab else vocab_size
        if self.split_vocab and vocab_size % self.tp.size:
            raise ValueError("vocab_size %d must be divisible by model_parallel %d" % (vocab_size, self.tp.size))
        self.vocab_size, self.embedding_size = vocab_size, embedding_size
        self.embedding_table = _mat((rows, embedding_size), 0.02, param_init_type, "embedding_table", self.split_vocab)

    def construct(self, input_ids):
        ids = input_ids.reshape(-1)
        if self.split_vocab:
            out = TP.vocab_parallel_embedding(self.embedding_table, ids, self.tp, self.sp)
        else:
            out = fused.embedding(self.embedding_table, ids)
            if self.tp.active and self.sp:
                n = out.shape[0] // self.tp.size
                out = out[self.tp.rank * n:(self.tp.rank + 1) * n]
        return out, self.embedding_table


class AttentionMask(Cell):
    """Lower-triangular mask from the input mask [B, S] -> [B, S, S] (kept for API parity; the attention kernel
    applies causality itself and never materialises this tensor)."""

    def __init__(self, seq_length, parallel_config=None):
        super().__init__()
        self.seq_length = seq_length

    def construct(self, input_mask):
        m = input_mask.float()
        tri = torch.tril(torch.ones(self.seq_length, self.seq_length, device=m.device))
        return m[:, :, None] * m[:, None, :] * tri[None]


class FeedForward(Cell):
    """Linear -> activation -> Linear, column- then row-parallel over the model-parallel group; with
    ``expert_num`` > 1 it is the expert FFN of ``MoE``."""

    def __init__(self, hidden_size, ffn_hidden_size, dropout_rate=0.0, hidden_act="gelu", expert_num=1,
                 expert_group_size=None, param_init_type=torch.float32, parallel_config=None, tp=None,
                 sequence_parallel=True, num_layers=1):
        super().__init__()
        self.tp = tp or TP.TPGroup(name=None, size=1, rank=0)
        self.sp = sequence_parallel
        if ffn_hidden_size % self.tp.size:
            raise ValueError("ffn_hidden_size %d must be divisible by model_parallel %d"
                             % (ffn_hidden_size, self.tp.size))
        f = ffn_hidden_size // self.tp.size
        self.act = hidden_act
        self.mapping_weight = _mat((f, hidden_size), 0.02, param_init_type, "mapping.weight", self.tp.active)
        self.mapping_bias = _vec(f, 0.0, param_init_type, "mapping.bias", self.tp, sequence_parallel, self.tp.active)
        self.projection_weight = _mat((hidden_size, f), 0.02 / math.sqrt(2 * num_layers), param_init_type,
                                      "projection.weight", self.tp.active)
        self.projection_bias = _vec(hidden_size, 0.0, param_init_type, "projection.bias", self.tp, sequence_parallel)
        self.dropout_rate = dropout_rate

    def construct(self, x):
        h = TP.column_parallel_linear(x, self.mapping_weight, self.tp, sequence_parallel=self.sp)
        if self.act == "gelu":
            h = fused.gelu_tanh(h, self.mapping_bias)
        else:
            h = h + self.mapping_bias
            h = torch.relu(h) if self.act == "relu" else torch.nn.functional.silu(h)
        y = TP.row_parallel_linear(h, self.projection_weight, self.tp, self.projection_bias, sequence_parallel=self.sp)
        if self.dropout_rate > 0 and self.training:
            y = torch.nn.functional.dropout(y, self.dropout_rate)
        return y


class MultiHeadAttention(Cell):
    """Causal self-attention: fused QKV column-parallel Dense, FlashAttention kernel, row-parallel output Dense.
    ``construct(x, batch, seq)`` with ``x`` [T(/mp), H]."""

    def __init__(self, batch_size, src_seq_length, tgt_seq_length, hidden_size, num_heads, hidden_dropout_rate=0.0,
                 attention_dropout_rate=0.0, compute_dtype=torch.bfloat16, softmax_compute_type=torch.float32,
                 param_init_type=torch.float32, use_past=False, parallel_config=None, tp=None, sequence_parallel=True,
                 num_layers=1, causal=True):
        super().__init__()
        self.tp = tp or TP.TPGroup(name=None, size=1, rank=0)
        self.sp = sequence_parallel
        self.causal = causal
        if hidden_size % num_heads:
            raise ValueError("hidden_size %d must be divisible by num_heads %d" % (hidden_size, num_heads))
        if num_heads % self.tp.size:
            raise ValueError("num_heads %d must be divisible by model_parallel %d" % (num_heads, self.tp.size))
        self.heads = num_heads // self.tp.size
        self.d = hidden_size // num_heads
        hd = self.heads * self.d
        self.wqkv = _mat((3 * hd, hidden_size), 0.02, param_init_type, "qkv.weight", self.tp.active)
        self.bqkv = _vec(3 * hd, 0.0, param_init_type, "qkv.bias", self.tp, sequence_parallel, self.tp.active)
        self.wo = _mat((hidden_size, hd), 0.02 / math.sqrt(2 * num_layers), param_init_type, "projection.weight",
                       self.tp.active)
        self.bo = _vec(hidden_size, 0.0, param_init_type, "projection.bias", self.tp, sequence_parallel)
        self.hidden_dropout_rate = hidden_dropout_rate

    def construct(self, x, batch, seq):
        qkv = TP.column_parallel_linear(x, self.wqkv, self.tp, self.bqkv, sequence_parallel=self.sp)
        hd, d = self.heads * self.d, self.d
        q, k, v = (qkv[:, i * hd:(i + 1) * hd].reshape(batch, seq, self.heads, d) for i in range(3))
        if d < 128 and q.is_cuda and q.dtype == torch.bfloat16 and seq % 128 == 0:
            # the attention kernel is built for head dim 128: zero columns leave QK^T and PV unchanged
            pad = lambda t: torch.nn.functional.pad(t, (0, 128 - d))
            o = fused.flash_attention(pad(q), pad(k), pad(v), causal=self.causal, scale=1.0 / math.sqrt(d))[..., :d]
        else:
            o = fused.flash_attention(q, k, v, causal=self.causal)
        y = TP.row_parallel_linear(o.reshape(batch * seq, hd), self.wo, self.tp, self.bo, sequence_parallel=self.sp)
        if self.hidden_dropout_rate > 0 and self.training:
            y = torch.nn.functional.dropout(y, self.hidden_dropout_rate)
        return y


class TransformerEncoderLayer(Cell):
    """Pre-LayerNorm decoder-only block: x + Attn(LN(x)); x + FFN(LN(x)).  With ``moe_config.expert_num > 1`` the
    FFN is a mixture of experts and ``construct`` returns (x, aux_loss)."""

    def __init__(self, batch_size, hidden_size, ffn_hidden_size, num_heads, seq_length, attention_dropout_rate=0.0,
                 hidden_dropout_rate=0.0, post_layernorm_residual=False, layernorm_compute_type=torch.float32,
                 softmax_compute_type=torch.float32, param_init_type=torch.float32, hidden_act="gelu", use_past=False,
                 moe_config=default_moe_config, parallel_config=default_transformer_config, num_layers=1,
                 causal=True):
        super().__init__()
        g = parallel_config.groups()
        tp, sp = g["tp"], parallel_config.sequence_parallel
        self.use_moe = moe_config.expert_num > 1
        self.layernorm1 = _LayerNorm((hidden_size,), param_init_type=param_init_type, tp=tp, sequence_parallel=sp)
        self.layernorm2 = _LayerNorm((hidden_size,), param_init_type=param_init_type, tp=tp, sequence_parallel=sp)
        self.attention = MultiHeadAttention(batch_size, seq_length, seq_length, hidden_size, num_heads,
                                            hidden_dropout_rate, attention_dropout_rate,
                                            param_init_type=param_init_type, tp=tp, sequence_parallel=sp,
                                            num_layers=num_layers, causal=causal)
        if self.use_moe:
            self.output = MoE(hidden_size, ffn_hidden_size, hidden_dropout_rate, hidden_act, param_init_type,
                              moe_config, parallel_config, expert_parallel_group=g["ep"])
            for p in self.output.get_parameters():
                # not split over the model-parallel group, but every one of its ranks routes different tokens
                p.tp_sharded = False
                p.tp_grad_reduce = tp.active and sp
        else:
            self.output = FeedForward(hidden_size, ffn_hidden_size, hidden_dropout_rate, hidden_act,
                                      param_init_type=param_init_type, tp=tp, sequence_parallel=sp,
                                      num_layers=num_layers)
        if parallel_config.recompute.recompute:
            self.recompute()

    def construct(self, x, batch, seq):
        x = x + self.attention(self.layernorm1(x), batch, seq)
        h = self.layernorm2(x)
        if self.use_moe:
            y, aux = self.output(h)
            return x + y, aux
        return x + self.output(h)


class TransformerEncoder(Cell):
    def __init__(self, batch_size, num_layers, hidden_size, ffn_hidden_size, seq_length, num_heads,
                 attention_dropout_rate=0.0, hidden_dropout_rate=0.0, hidden_act="gelu",
                 post_layernorm_residual=False, layernorm_compute_type=torch.float32,
                 softmax_compute_type=torch.float32, param_init_type=torch.float32, lambda_func=None, offset=0,
                 use_past=False, moe_config=default_moe_config, parallel_config=default_transformer_config,
                 causal=True):
        super().__init__()
        self.use_moe = moe_config.expert_num > 1
        self.blocks = CellList([
            TransformerEncoderLayer(batch_size, hidden_size, ffn_hidden_size, num_heads, seq_length,
                                    attention_dropout_rate, hidden_dropout_rate, post_layernorm_residual,
                                    layernorm_compute_type, softmax_compute_type, param_init_type, hidden_act,
                                    use_past, moe_config, parallel_config, num_layers, causal)
            for _ in range(num_layers)])
        _assign_stages(self.blocks, num_layers, offset, parallel_config, lambda_func)

    def construct(self, x, batch, seq):
        aux_total = None
        for b in self.blocks:
            if self.use_moe:
                x, aux = b(x, batch, seq)
                aux_total = aux if aux_total is None else aux_total + aux
            else:
                x = b(x, batch, seq)
        return (x, aux_total) if self.use_moe else x


class CrossAttention(Cell):
    """Attention of decoder tokens over the encoder output: column-parallel query and fused key / value
    projections, full (non-causal) attention, row-parallel output projection.  ``construct(x, memory, batch,
    tgt_seq, src_seq)`` with ``x`` [batch * tgt_seq (/mp), H] and ``memory`` [batch * src_seq (/mp), H]
    (the second attention of the reference's TransformerDecoderLayer, transformer.py:1777)."""

    def __init__(self, hidden_size, num_heads, hidden_dropout_rate=0.0, param_init_type=torch.float32, tp=None,
                 sequence_parallel=True, num_layers=1):
        super().__init__()
        self.tp = tp or TP.TPGroup(name=None, size=1, rank=0)
        self.sp = sequence_parallel
        if hidden_size % num_heads or num_heads % self.tp.size:
            raise ValueError("hidden_size %d / num_heads %d / model_parallel %d do not divide"
                             % (hidden_size, num_heads, self.tp.size))
        self.heads = num_heads // self.tp.size
        self.d = hidden_size // num_heads
        hd = self.heads * self.d
        self.wq = _mat((hd, hidden_size), 0.02, param_init_type, "q.weight", self.tp.active)
        self.bq = _vec(hd, 0.0, param_init_type, "q.bias", self.tp, sequence_parallel, self.tp.active)
        self.wkv = _mat((2 * hd, hidden_size), 0.02, param_init_type, "kv.weight", self.tp.active)
        self.bkv = _vec(2 * hd, 0.0, param_init_type, "kv.bias", self.tp, sequence_parallel, self.tp.active)
        self.wo = _mat((hidden_size, hd), 0.02 / math.sqrt(2 * num_layers), param_init_type, "projection.weight",
                       self.tp.active)
        self.bo = _vec(hidden_size, 0.0, param_init_type, "projection.bias", self.tp, sequence_parallel)
        self.hidden_dropout_rate = hidden_dropout_rate

    def construct(self, x, memory, batch, tgt_seq, src_seq):
        hd, d = self.heads * self.d, self.d
        q = TP.column_parallel_linear(x, self.wq, self.tp, self.bq, sequence_parallel=self.sp)
        kv = TP.column_parallel_linear(memory, self.wkv, self.tp, self.bkv, sequence_parallel=self.sp)
        q = q.reshape(batch, tgt_seq, self.heads, d)
        k = kv[:, :hd].reshape(batch, src_seq, self.heads, d)
        v = kv[:, hd:].reshape(batch, src_seq, self.heads, d)
        o = fused.flash_attention(q, k, v, causal=False)
        y = TP.row_parallel_linear(o.reshape(batch * tgt_seq, hd), self.wo, self.tp, self.bo,
                                   sequence_parallel=self.sp)
        if self.hidden_dropout_rate > 0 and self.training:
            y = torch.nn.functional.dropout(y, self.hidden_dropout_rate)
        return y


class TransformerDecoderLayer(Cell):
    """Pre-LayerNorm decoder block: causal self-attention, attention over the encoder output, feed-forward (or MoE),
    each behind a residual connection.  ``construct(x, memory, batch, tgt_seq, src_seq)``; with
    ``moe_config.expert_num > 1`` it returns (x, aux_loss).  Parity: transformer.py:1777."""

    def __init__(self, hidden_size, ffn_hidden_size, num_heads, batch_size, src_seq_length, tgt_seq_length,
                 attention_dropout_rate=0.0, hidden_dropout_rate=0.0, post_layernorm_residual=False, use_past=False,
                 layernorm_compute_type=torch.float32, softmax_compute_type=torch.float32,
                 param_init_type=torch.float32, hidden_act="gelu", moe_config=default_moe_config,
                 parallel_config=default_transformer_config, num_layers=1):
        super().__init__()
        g = parallel_config.groups()
        tp, sp = g["tp"], parallel_config.sequence_parallel
        self.use_moe = moe_config.expert_num > 1
        ln = lambda: _LayerNorm((hidden_size,), param_init_type=param_init_type, tp=tp, sequence_parallel=sp)
        self.layernorm1, self.layernorm2, self.cross_attention_layernorm = ln(), ln(), ln()
        self.attention = MultiHeadAttention(batch_size, tgt_seq_length, tgt_seq_length, hidden_size, num_heads,
                                            hidden_dropout_rate, attention_dropout_rate,
                                            param_init_type=param_init_type, tp=tp, sequence_parallel=sp,
                                            num_layers=num_layers, causal=True)
        self.cross_attention = CrossAttention(hidden_size, num_heads, hidden_dropout_rate, param_init_type, tp, sp,
                                              num_layers)
        if self.use_moe:
            self.output = MoE(hidden_size, ffn_hidden_size, hidden_dropout_rate, hidden_act, param_init_type,
                              moe_config, parallel_config, expert_parallel_group=g["ep"])
            for p in self.output.get_parameters():
                p.tp_sharded = False
                p.tp_grad_reduce = tp.active and sp
        else:
            self.output = FeedForward(hidden_size, ffn_hidden_size, hidden_dropout_rate, hidden_act,
                                      param_init_type=param_init_type, tp=tp, sequence_parallel=sp,
                                      num_layers=num_layers)
        if parallel_config.recompute.recompute:
            self.recompute()

    def construct(self, x, memory, batch, tgt_seq, src_seq):
        x = x + self.attention(self.layernorm1(x), batch, tgt_seq)
        x = x + self.cross_attention(self.cross_attention_layernorm(x), memory, batch, tgt_seq, src_seq)
        h = self.layernorm2(x)
        if self.use_moe:
            y, aux = self.output(h)
            return x + y, aux
        return x + self.output(h)


def _assign_stages(blocks, num_layers, offset, parallel_config, lambda_func):
    stages = parallel_config.pipeline_stage
    if stages > 1:
        per = (num_layers + stages - 1) // stages
        for i, b in enumerate(blocks):
            b.pipeline_stage = min((i + offset) // per, stages - 1)
    if lambda_func is not None:
        for i, b in enumerate(blocks):
            lambda_func(b, i, offset, parallel_config, num_layers)


class TransformerDecoder(Cell):
    """``num_layers`` decoder blocks.  Parity: transformer.py:2532."""

    def __init__(self, num_layers, batch_size, hidden_size, ffn_hidden_size, src_seq_length, tgt_seq_length,
                 num_heads, attention_dropout_rate=0.0, hidden_dropout_rate=0.0, post_layernorm_residual=False,
                 layernorm_compute_type=torch.float32, softmax_compute_type=torch.float32,
                 param_init_type=torch.float32, hidden_act="gelu", lambda_func=None, use_past=False, offset=0,
                 moe_config=default_moe_config, parallel_config=default_transformer_config):
        super().__init__()
        self.use_moe = moe_config.expert_num > 1
        self.blocks = CellList([
            TransformerDecoderLayer(hidden_size, ffn_hidden_size, num_heads, batch_size, src_seq_length,
                                    tgt_seq_length, attention_dropout_rate, hidden_dropout_rate,
                                    post_layernorm_residual, use_past, layernorm_compute_type, softmax_compute_type,
                                    param_init_type, hidden_act, moe_config, parallel_config, num_layers)
            for _ in range(num_layers)])
        _assign_stages(self.blocks, num_layers, offset, parallel_config, lambda_func)

    def construct(self, x, memory, batch, tgt_seq, src_seq):
        aux_total = None
        for b in self.blocks:
            if self.use_moe:
                x, aux = b(x, memory, batch, tgt_seq, src_seq)
                aux_total = aux if aux_total is None else aux_total + aux
            else:
                x = b(x, memory, batch, tgt_seq, src_seq)
        return (x, aux_total) if self.use_moe else x


class Transformer(Cell):
    """Encoder (bidirectional) + decoder (causal, attending over the encoder output).  ``construct(encoder_inputs
    [batch * src_seq (/mp), H], decoder_inputs [batch * tgt_seq (/mp), H] or None, batch)`` returns
    ``(decoder_output or encoder_output, encoder_output)`` plus the summed MoE auxiliary loss when experts are
    configured.  With ``decoder_layers=0`` it is the encoder alone.  Parity: transformer.py:2780."""

    def __init__(self, hidden_size, batch_size, ffn_hidden_size, src_seq_length, tgt_seq_length, encoder_layers=3,
                 decoder_layers=3, num_heads=2, attention_dropout_rate=0.0, hidden_dropout_rate=0.0, hidden_act="gelu",
                 post_layernorm_residual=False, layernorm_compute_type=torch.float32,
                 softmax_compute_type=torch.float32, param_init_type=torch.float32, lambda_func=None, use_past=False,
                 moe_config=default_moe_config, parallel_config=default_transformer_config):
        super().__init__()
        if encoder_layers <= 0:
            raise ValueError("Transformer needs at least one encoder layer, got encoder_layers=%d" % encoder_layers)
        self.src_seq, self.tgt_seq = src_seq_length, tgt_seq_length
        self.use_moe = moe_config.expert_num > 1
        self.encoder = TransformerEncoder(batch_size, encoder_layers, hidden_size, ffn_hidden_size, src_seq_length,
                                          num_heads, attention_dropout_rate, hidden_dropout_rate, hidden_act,
                                          post_layernorm_residual, layernorm_compute_type, softmax_compute_type,
                                          param_init_type, lambda_func, 0, use_past, moe_config, parallel_config,
                                          causal=False)
        self.decoder = TransformerDecoder(decoder_layers, batch_size, hidden_size, ffn_hidden_size, src_seq_length,
                                          tgt_seq_length, num_heads, attention_dropout_rate, hidden_dropout_rate,
                                          post_layernorm_residual, layernorm_compute_type, softmax_compute_type,
                                          param_init_type, hidden_act, lambda_func, use_past, encoder_layers,
                                          moe_config, parallel_config) if decoder_layers > 0 else None

    def construct(self, encoder_inputs, decoder_inputs=None, batch=None):
        if batch is None:
            batch = encoder_inputs.shape[0] // self.src_seq
        memory = self.encoder(encoder_inputs, batch, self.src_seq)
        aux = None
        if self.use_moe:
            memory, aux = memory
        if self.decoder is None or decoder_inputs is None:
            return (memory, memory, aux) if self.use_moe else (memory, memory)
        out = self.decoder(decoder_inputs, memory, batch, self.tgt_seq, self.src_seq)
        if self.use_moe:
            out, aux2 = out
            return out, memory, aux + aux2
        return out, memory


class FixedSparseAttention(Cell):
    """The "fixed" pattern of Sparse Transformers (Child et al. 2019) on [batch, seq, hidden] inputs: a query attends
    causally inside its own block of ``block_size`` tokens, and to the summary columns of every earlier block - the
    last ``block_size / num_different_global_patterns`` tokens of a block for head pattern 0, the slice before it
    for pattern 1, and so on, heads cycling through the patterns.  ``attention_mask`` [batch, seq, seq] (1 = may
    attend) is applied on top.  The sparse pattern is evaluated as a mask of a dense attention (the reference
    computes it with a block-sparse kernel pair that exists for one Ascend layout only, layers.py:545): same result
    for the pattern above, not the same cost."""

    def __init__(self, batch_size, num_heads, size_per_head, block_size, seq_length=1024,
                 num_different_global_patterns=4, parallel_config=None):
        super().__init__()
        if seq_length % block_size or block_size % num_different_global_patterns:
            raise ValueError("For 'FixedSparseAttention', seq_length %d must be a multiple of block_size %d and "
                             "block_size a multiple of num_different_global_patterns %d"
                             % (seq_length, block_size, num_different_global_patterns))
        self.batch_size, self.num_heads, self.size_per_head = batch_size, num_heads, size_per_head
        self.block_size, self.seq_length, self.patterns = block_size, seq_length, num_different_global_patterns
        pos = torch.arange(seq_length)
        blk, inb = pos // block_size, pos % block_size
        local = (blk[:, None] == blk[None, :]) & (pos[None, :] <= pos[:, None])
        width = block_size // num_different_global_patterns
        masks = []
        for pat in range(num_different_global_patterns):
            lo = block_size - (pat + 1) * width
            summary = (inb >= lo) & (inb < lo + width)
            masks.append(local | ((blk[None, :] < blk[:, None]) & summary[None, :]))
        self.pattern_masks = torch.stack(masks)                                  # [patterns, S, S] bool

    def layout(self):
        """[num_heads, seq, seq] bool: which keys each query of each head may look at."""
        return self.pattern_masks[torch.arange(self.num_heads) % self.patterns]

    def construct(self, q, k, v, attention_mask=None):
        B, S, _ = q.shape
        H, D = self.num_heads, self.size_per_head
        split = lambda t: t.reshape(B, S, H, D).permute(0, 2, 1, 3)
        allowed = self.layout().to(q.device)[None]
        if attention_mask is not None:
            allowed = allowed & (attention_mask.reshape(B, 1, S, S) > 0)
        out = torch.nn.functional.scaled_dot_product_attention(split(q), split(k), split(v), attn_mask=allowed,
                                                               scale=1.0 / math.sqrt(D))
        return out.permute(0, 2, 1, 3).reshape(B, S, H * D)


class CrossEntropyLoss(Cell):
    """Mean cross entropy over tokens with logits split over the model-parallel group along the vocabulary."""

    def __init__(self, parallel_config=default_transformer_config, tp=None):
        super().__init__()
        self.tp = tp or parallel_config.groups()["tp"]

    def construct(self, logits, label, input_mask=None):
        labels = label.reshape(-1)
        if input_mask is not None:
            labels = torch.where(input_mask.reshape(-1) > 0, labels, torch.full_like(labels, -100))
        return TP.vocab_parallel_cross_entropy(logits, labels, self.tp)
