"""Llama-2 style decoder (RMSNorm, RoPE, SwiGLU, optional grouped kv heads), written with primitives and shard
strategies only.

Every operator of a block is an ``ops`` primitive; model parallelism is nothing but the strategies set on them
(``cfg.model_parallel = mp``, reference notation):

  wqkv / w_gate_up / lm_head : MatMul(transpose_b).shard(((1, 1), (mp, 1)))                  column parallel
  wo / w_down                : MatMul(transpose_b).shard(((1, mp), (1, mp)), out_strategy=((mp, 1),))
                                                                                row parallel -> ReduceScatter
  (Add)RmsNorm, residual     : shard(((mp, 1), ..., (1,)))         token (sequence) parallel, gamma mirrored
  RotaryFlashAttention       : shard(((1, mp), (1, 1), (1, 1)))    heads over mp
  SwiGLU                     : shard(((1, mp),))
  embedding                  : Gather.shard(((mp, 1), (1,)), out_strategy=((mp, 1),))   vocabulary parallel
  loss                       : SparseSoftmaxCrossEntropyWithLogits.shard(((1, mp), (1,)))  vocabulary parallel

Under ``semi_auto_parallel`` the dispatcher (``parallel/spmd.py``) derives layouts from these strategies, slices
the parameters, inserts the redistribution (the AllGather in front of a column-parallel MatMul) and the forward
communication (the ReduceScatter behind a row-parallel one) - and runs each (collective, MatMul) pair as one fused
NVLink kernel.  With ``sequence_parallel=False`` the row-parallel MatMuls all-reduce and the norms run replicated.
In stand-alone mode the same code runs the kernels directly.  ``models/llama_tp.py`` is the hand-placed
tensor-parallel formulation of the same network, kept as the baseline the strategy-driven one is tested against.

Parity: the reference's Llama system test model (tests/st/networks/llama/parallel_llama.py:66-112, mindformers
Llama) and parallel/_transformer/transformer.py building blocks.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch

from .. import nn, ops
from ..common import dtype as mstype
from ..common.initializer import Normal, initializer
from ..common.parameter import Parameter
from ..ops import fused
from ..parallel import spmd


@dataclass
class LlamaConfig:
    vocab_size: int = 32000
    hidden_size: int = 4096
    num_layers: int = 32
    num_heads: int = 32
    num_kv_heads: int = 32
    ffn_hidden_size: int = 11008
    seq_length: int = 4096
    rms_norm_eps: float = 1e-5
    rope_theta: float = 10000.0
    dtype: torch.dtype = mstype.bfloat16
    model_parallel: int = 1
    sequence_parallel: bool = True
    recompute: bool = False
    init_std: float = 0.02

    @property
    def head_dim(self):
        return self.hidden_size // self.num_heads

    def num_parameters(self):
        h, f, v = self.hidden_size, self.ffn_hidden_size, self.vocab_size
        kv = self.num_kv_heads * self.head_dim
        per_layer = h * (h + 2 * kv) + h * h + 3 * h * f + 2 * h
        return self.num_layers * per_layer + 2 * v * h + h

    def flops_per_token(self, seq=None):
        """Forward+backward model FLOPs per token (6*N for the GEMMs plus causal attention)."""
        seq = seq or self.seq_length
        h, f = self.hidden_size, self.ffn_hidden_size
        kv = self.num_kv_heads * self.head_dim
        gemm = self.num_layers * (h * (h + 2 * kv) + h * h + 3 * h * f) + self.vocab_size * h
        attn = self.num_layers * 2 * seq * h / 2          # QK^T and PV, causal half
        return 6 * gemm + 6 * attn


LLAMA2_7B = LlamaConfig()


def _mp(cfg):
    """Model-parallel width the strategies use: ``cfg.model_parallel`` when the dispatcher is active, else 1."""
    return cfg.model_parallel if (cfg.model_parallel > 1 and spmd.active()) else 1


def _pipeline_stages():
    from .. import context
    return int(context.get_auto_parallel_context("pipeline_stages")) if spmd.active() else 1


def _sharded(prim, *strategy, out=None):
    """``prim.shard`` when there is something to shard (keeps stand-alone runs free of strategy warnings)."""
    if any(s != 1 for st in strategy for s in st):
        prim.shard(tuple(strategy), out)
    return prim


def _weight(shape, std, dtype, name, prim):
    """Full-shape parameter, sliced at once to what input 1 of ``prim`` (a MatMul) needs."""
    p = Parameter(initializer(Normal(std), shape, dtype), name=name)
    return spmd.shard_parameter(p, prim, 1)


class LlamaAttention(nn.Cell):
    def __init__(self, cfg: LlamaConfig):
        super().__init__()
        mp = _mp(cfg)
        if cfg.num_heads % cfg.model_parallel or cfg.num_kv_heads % cfg.model_parallel:
            raise ValueError("heads (%d, kv %d) must be divisible by model_parallel %d"
                             % (cfg.num_heads, cfg.num_kv_heads, cfg.model_parallel))
        sp = cfg.sequence_parallel
        d = cfg.head_dim
        self.qkv_proj = _sharded(ops.MatMul(transpose_b=True), (1, 1), (mp, 1))
        self.attention = _sharded(ops.RotaryFlashAttention(cfg.num_heads, cfg.num_kv_heads, d,
                                                           groups=cfg.model_parallel, causal=True),
                                  (1, mp), (1, 1), (1, 1))
        self.out_proj = _sharded(ops.MatMul(transpose_b=True), (1, mp), (1, mp),
                                 out=((mp, 1),) if (sp and mp > 1) else None)
        qkv_out = (cfg.num_heads + 2 * cfg.num_kv_heads) * d
        self.wqkv = _weight((qkv_out, cfg.hidden_size), cfg.init_std, cfg.dtype, "wqkv", self.qkv_proj)
        self.wo = _weight((cfg.hidden_size, cfg.num_heads * d), cfg.init_std / math.sqrt(2 * cfg.num_layers),
                          cfg.dtype, "wo", self.out_proj)

    def construct(self, x, cos, sin):
        """x: [tokens(/mp), hidden] -> [tokens(/mp), hidden]"""
        qkv = self.qkv_proj(x, self.wqkv)                 # [T, (h + 2 hk) d], heads split over mp
        o = self.attention(qkv, cos, sin)                 # [T, h d]
        return self.out_proj(o, self.wo)


class LlamaMLP(nn.Cell):
    def __init__(self, cfg: LlamaConfig):
        super().__init__()
        if cfg.ffn_hidden_size % cfg.model_parallel:
            raise ValueError("ffn_hidden_size must be divisible by model_parallel")
        mp = _mp(cfg)
        sp = cfg.sequence_parallel
        self.gate_up_proj = _sharded(ops.MatMul(transpose_b=True), (1, 1), (mp, 1))
        self.act = _sharded(ops.SwiGLU(groups=cfg.model_parallel), (1, mp))
        self.down_proj = _sharded(ops.MatMul(transpose_b=True), (1, mp), (1, mp),
                                  out=((mp, 1),) if (sp and mp > 1) else None)
        f = cfg.ffn_hidden_size
        self.w_gate_up = _weight((2 * f, cfg.hidden_size), cfg.init_std, cfg.dtype, "w_gate_up", self.gate_up_proj)
        self.w_down = _weight((cfg.hidden_size, f), cfg.init_std / math.sqrt(2 * cfg.num_layers), cfg.dtype,
                              "w_down", self.down_proj)

    def construct(self, x):
        return self.down_proj(self.act(self.gate_up_proj(x, self.w_gate_up)), self.w_down)


def _norm_prims(cfg):
    mp = _mp(cfg) if cfg.sequence_parallel else 1
    return (_sharded(ops.RmsNorm(cfg.rms_norm_eps), (mp, 1), (1,)),
            _sharded(ops.AddRmsNorm(cfg.rms_norm_eps), (mp, 1), (mp, 1), (1,)))


class LlamaDecoderLayer(nn.Cell):
    def __init__(self, cfg: LlamaConfig):
        super().__init__()
        self.cfg = cfg
        self.attention_norm = Parameter(torch.ones(cfg.hidden_size, dtype=cfg.dtype), name="attention_norm")
        self.ffn_norm = Parameter(torch.ones(cfg.hidden_size, dtype=cfg.dtype), name="ffn_norm")
        self.norm, self.add_norm = _norm_prims(cfg)
        self.attention = LlamaAttention(cfg)
        self.feed_forward = LlamaMLP(cfg)
        self.pipeline_outputs = 2          # (residual stream, pending delta): what a later pipeline stage skips over

    def construct(self, x, delta, cos, sin):
        """The residual stream is carried as (x, delta): the add is part of the next norm kernel."""
        if delta is None:
            h = self.norm(x, self.attention_norm)[0]
        else:
            h, x = self.add_norm(x, delta, self.attention_norm)
        a = self.attention(h, cos, sin)
        h, x = self.add_norm(x, a, self.ffn_norm)
        return x, self.feed_forward(h)


class LlamaModel(nn.Cell):
    def __init__(self, cfg: LlamaConfig):
        super().__init__()
        self.cfg = cfg
        if cfg.vocab_size % cfg.model_parallel:
            raise ValueError("vocab_size must be divisible by model_parallel")
        mp = _mp(cfg)
        sp = cfg.sequence_parallel and mp > 1
        self.embedding = _sharded(ops.Gather(), (mp, 1), (1,), out=((mp, 1),) if sp else None)
        self.tok_embeddings = Parameter(initializer(Normal(cfg.init_std), (cfg.vocab_size, cfg.hidden_size),
                                                    cfg.dtype), name="tok_embeddings")
        spmd.shard_parameter(self.tok_embeddings, self.embedding, 0,
                             shapes=[(cfg.vocab_size, cfg.hidden_size), (cfg.model_parallel * 128,)], axis=0)
        self.layers = nn.CellList([LlamaDecoderLayer(cfg) for _ in range(cfg.num_layers)])
        self.norm_out = Parameter(torch.ones(cfg.hidden_size, dtype=cfg.dtype), name="norm_out")
        self.norm, self.add_norm = _norm_prims(cfg)
        self._rope = {}
        if cfg.recompute:
            for layer in self.layers:
                layer.recompute()
        # pipeline parallelism: consecutive blocks of layers per stage.  The embedding runs in front of the first
        # tagged cell (so on the first stage it feeds layer 0; later stages skip to their first own layer and take
        # the residual stream from the previous stage); the final norm, the LM head and the loss follow the last
        # tagged cell, i.e. they run on the last stage only.
        stages = _pipeline_stages()
        if stages > 1:
            if cfg.num_layers % stages:
                raise ValueError("num_layers %d must be divisible by pipeline_stages %d" % (cfg.num_layers, stages))
            per = cfg.num_layers // stages
            for i, layer in enumerate(self.layers):
                layer.pipeline_stage = i // per

    def rope(self, seq, device):
        key = (seq, str(device))
        if key not in self._rope:
            self._rope[key] = fused.rope_tables(seq, self.cfg.head_dim, self.cfg.rope_theta, device)
        return self._rope[key]

    def construct(self, tokens):
        """tokens [B, S] int -> hidden states [B*S(/mp), hidden]"""
        batch, seq = tokens.shape
        cos, sin = self.rope(seq, tokens.device)
        x = self.embedding(self.tok_embeddings, tokens.reshape(-1), 0)
        delta = None
        for layer in self.layers:
            x, delta = layer(x, delta, cos, sin)
        if delta is None:
            return self.norm(x, self.norm_out)[0]
        return self.add_norm(x, delta, self.norm_out)[0]


class LlamaForCausalLM(nn.Cell):
    """tokens [B, S+1] (or (inputs, labels)) -> mean next-token cross entropy."""

    def __init__(self, cfg: LlamaConfig):
        super().__init__()
        self.cfg = cfg
        mp = _mp(cfg)
        self.model = LlamaModel(cfg)
        self.head_proj = _sharded(ops.MatMul(transpose_b=True), (1, 1), (mp, 1))
        self.loss = _sharded(ops.SparseSoftmaxCrossEntropyWithLogits(), (1, mp), (1,))
        self.lm_head = _weight((cfg.vocab_size, cfg.hidden_size), cfg.init_std, cfg.dtype, "lm_head", self.head_proj)

    def logits(self, tokens):
        return self.head_proj(self.model(tokens), self.lm_head)

    def construct(self, tokens, labels=None):
        if labels is None:
            tokens, labels = tokens[:, :-1], tokens[:, 1:]
        return self.loss(self.logits(tokens), labels.reshape(-1))


def pack_full_weights(full, cfg: LlamaConfig, groups: int):
    """Re-orders the fused matrices of a {name: full tensor} dict from the plain layout (all q heads, then k, then
    v; all gate rows, then up) to the one packed in ``groups`` blocks that ``RotaryFlashAttention`` /
    ``SwiGLU(groups=...)`` read: block i = [q_i, k_i, v_i] (resp. [gate_i, up_i]) of the i-th 1/groups of the heads
    (resp. FFN rows).  With groups = 1 nothing moves."""
    d = cfg.head_dim
    hq, hk = cfg.num_heads * d, cfg.num_kv_heads * d
    f = cfg.ffn_hidden_size
    out = {}
    for name, w in full.items():
        if name.endswith("wqkv"):
            q, k, v = w[:hq], w[hq:hq + hk], w[hq + hk:]
            out[name] = torch.cat([t for i in range(groups) for t in (torch.chunk(q, groups, 0)[i],
                                                                       torch.chunk(k, groups, 0)[i],
                                                                       torch.chunk(v, groups, 0)[i])], 0)
        elif name.endswith("w_gate_up"):
            g, u = w[:f], w[f:]
            out[name] = torch.cat([t for i in range(groups) for t in (torch.chunk(g, groups, 0)[i],
                                                                       torch.chunk(u, groups, 0)[i])], 0)
        else:
            out[name] = w
    return {k: v.contiguous() for k, v in out.items()}
