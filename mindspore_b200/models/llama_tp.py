"""Llama-2 style decoder with hand-placed tensor + sequence parallelism (the baseline formulation).

``models/llama.py`` expresses the same network with primitives and shard strategies and lets the dispatcher insert
the communication; this file places every collective by hand (``parallel.tp``) and is what that one is tested
against.  The network is written against the framework's own cells and fused ops; with ``parallel_config.model_parallel =
mp`` every Dense becomes column- or row-parallel (weights are created already sharded, so a 7B model never
materialises in full on one GPU), activations between the parallel regions are token-sharded, the embedding and
the LM head are vocabulary-parallel and the loss is the vocab-parallel cross entropy.

Shard strategies equivalent to what this model does, in the reference's notation (mp = model_parallel):
  wqkv / w_gate_up : MatMul.shard(((1, 1), (mp, 1)))                      column parallel
  wo / w_down      : MatMul.shard(((1, mp), (1, mp)), out_strategy=((mp, 1),))   row parallel + ReduceScatter
  RMSNorm, residual: shard(((mp, 1),)) on the token dim                    sequence parallel
  FlashAttention   : shard over heads (mp)
Parity: the reference's Llama system test model (tests/st/networks/llama/parallel_llama.py:66-112, mindformers
Llama) and parallel/_transformer/transformer.py building blocks.
"""
from __future__ import annotations

import math

import torch

from .. import nn
from ..common import dtype as mstype
from ..common.initializer import Normal, initializer
from ..common.parameter import Parameter
from ..ops import fused
from ..ops.primitive import _wrap_out
from ..parallel import tp as TP


from .llama import LLAMA2_7B, LlamaConfig  # noqa: E402,F401  (one config class for both formulations)


def _param(shape, std, dtype, name):
    p = Parameter(initializer(Normal(std), shape, dtype), name=name)
    p.tp_sharded = True          # every matrix of this model is sharded over the model-parallel group
    return p


def _norm_weight(cfg, tp, name):
    p = Parameter(torch.ones(cfg.hidden_size, dtype=cfg.dtype), name=name)
    # replicated over the model-parallel group but fed by token-sharded activations: gradients are partial sums
    p.tp_grad_reduce = tp.active and cfg.sequence_parallel
    return p


class LlamaAttention(nn.Cell):
    def __init__(self, cfg: LlamaConfig, tp: TP.TPGroup):
        super().__init__()
        mp = tp.size
        if cfg.num_heads % mp or cfg.num_kv_heads % mp:
            raise ValueError("heads (%d, kv %d) must be divisible by model_parallel %d"
                             % (cfg.num_heads, cfg.num_kv_heads, mp))
        self.cfg, self.tp = cfg, tp
        self.heads, self.kv_heads, self.d = cfg.num_heads // mp, cfg.num_kv_heads // mp, cfg.head_dim
        qkv_out = (self.heads + 2 * self.kv_heads) * self.d
        self.wqkv = _param((qkv_out, cfg.hidden_size), cfg.init_std, cfg.dtype, "wqkv")
        self.wo = _param((cfg.hidden_size, self.heads * self.d), cfg.init_std / math.sqrt(2 * cfg.num_layers),
                         cfg.dtype, "wo")

    def construct(self, x, cos, sin, batch, seq):
        """x: [tokens(/mp), hidden] -> [tokens(/mp), hidden]"""
        sp = self.cfg.sequence_parallel
        qkv = TP.column_parallel_linear(x, self.wqkv, self.tp, sequence_parallel=sp)      # [T, (h+2hk)*d]
        hd = self.heads * self.d
        o = fused.qkv_rope_attention(qkv, cos, sin, batch, seq, self.heads, self.kv_heads, self.d, causal=True)
        return TP.row_parallel_linear(o.reshape(batch * seq, hd), self.wo, self.tp, sequence_parallel=sp)


class LlamaMLP(nn.Cell):
    def __init__(self, cfg: LlamaConfig, tp: TP.TPGroup):
        super().__init__()
        if cfg.ffn_hidden_size % tp.size:
            raise ValueError("ffn_hidden_size must be divisible by model_parallel")
        self.cfg, self.tp = cfg, tp
        f = cfg.ffn_hidden_size // tp.size
        self.w_gate_up = _param((2 * f, cfg.hidden_size), cfg.init_std, cfg.dtype, "w_gate_up")
        self.w_down = _param((cfg.hidden_size, f), cfg.init_std / math.sqrt(2 * cfg.num_layers), cfg.dtype, "w_down")

    def construct(self, x):
        sp = self.cfg.sequence_parallel
        gu = TP.column_parallel_linear(x, self.w_gate_up, self.tp, sequence_parallel=sp)
        return TP.row_parallel_linear(fused.swiglu(gu), self.w_down, self.tp, sequence_parallel=sp)


class LlamaDecoderLayer(nn.Cell):
    def __init__(self, cfg: LlamaConfig, tp: TP.TPGroup):
        super().__init__()
        self.cfg = cfg
        self.attention_norm = _norm_weight(cfg, tp, "attention_norm")
        self.ffn_norm = _norm_weight(cfg, tp, "ffn_norm")
        self.attention = LlamaAttention(cfg, tp)
        self.feed_forward = LlamaMLP(cfg, tp)

    def construct(self, x, delta, cos, sin, batch, seq):
        """Residual stream is carried as (x, delta): the add is fused into the next RMSNorm kernel."""
        eps = self.cfg.rms_norm_eps
        h, x = fused.rms_norm(x, self.attention_norm, eps, delta)
        a = self.attention(h, cos, sin, batch, seq)
        h, x = fused.rms_norm(x, self.ffn_norm, eps, a)
        return x, self.feed_forward(h)


class LlamaModel(nn.Cell):
    def __init__(self, cfg: LlamaConfig, tp: TP.TPGroup = None):
        super().__init__()
        self.cfg = cfg
        self.tp = tp or TP.TPGroup(size=1, rank=0, name=None)
        if cfg.model_parallel != self.tp.size:
            raise ValueError("config.model_parallel (%d) does not match the model-parallel group size (%d)"
                             % (cfg.model_parallel, self.tp.size))
        if cfg.vocab_size % self.tp.size:
            raise ValueError("vocab_size must be divisible by model_parallel")
        self.tok_embeddings = _param((cfg.vocab_size // self.tp.size, cfg.hidden_size), cfg.init_std, cfg.dtype,
                                     "tok_embeddings")
        self.layers = nn.CellList([LlamaDecoderLayer(cfg, self.tp) for _ in range(cfg.num_layers)])
        self.norm_out = _norm_weight(cfg, self.tp, "norm_out")
        self._rope = {}
        if cfg.recompute:
            for layer in self.layers:
                layer.recompute()

    def rope(self, seq, device):
        key = (seq, str(device))
        if key not in self._rope:
            self._rope[key] = fused.rope_tables(seq, self.cfg.head_dim, self.cfg.rope_theta, device)
        return self._rope[key]

    def construct(self, tokens):
        """tokens [B, S] int -> hidden states [B*S(/mp), hidden]"""
        batch, seq = tokens.shape
        cos, sin = self.rope(seq, tokens.device)
        ids = tokens.reshape(-1)
        x = TP.vocab_parallel_embedding(self.tok_embeddings, ids, self.tp, self.cfg.sequence_parallel)
        delta = None
        for layer in self.layers:
            x, delta = layer(x, delta, cos, sin, batch, seq)
        h, _ = fused.rms_norm(x, self.norm_out, self.cfg.rms_norm_eps, delta)
        return h


class LlamaForCausalLM(nn.Cell):
    """tokens [B, S+1] (or (inputs, labels)) -> mean next-token cross entropy."""

    def __init__(self, cfg: LlamaConfig, tp: TP.TPGroup = None):
        super().__init__()
        self.cfg = cfg
        self.model = LlamaModel(cfg, tp)
        self.tp = self.model.tp
        self.lm_head = _param((cfg.vocab_size // self.tp.size, cfg.hidden_size), cfg.init_std, cfg.dtype, "lm_head")

    def logits(self, tokens):
        h = self.model(tokens)
        return TP.column_parallel_linear(h, self.lm_head, self.tp, sequence_parallel=self.cfg.sequence_parallel)

    def construct(self, tokens, labels=None):
        if labels is None:
            tokens, labels = tokens[:, :-1], tokens[:, 1:]
        logits = self.logits(tokens)
        loss = TP.vocab_parallel_cross_entropy(logits, labels.reshape(-1), self.tp)
        return _wrap_out(loss)


def shard_full_weights(full, cfg: LlamaConfig, mp: int, rank: int):
    """Slices a dict {name: full tensor} of the mp=1 model into the shard held by ``rank`` of an mp-way model:
    q/k/v heads and gate/up columns are split per rank inside the fused matrices, wo / w_down by input columns,
    embedding and LM head by vocabulary rows; norm weights are replicated."""
    d = cfg.head_dim
    hq, hk = cfg.num_heads * d, cfg.num_kv_heads * d
    f = cfg.ffn_hidden_size
    out = {}
    for name, w in full.items():
        if name.endswith("wqkv"):
            q, k, v = w[:hq], w[hq:hq + hk], w[hq + hk:]
            out[name] = torch.cat([torch.chunk(q, mp, 0)[rank], torch.chunk(k, mp, 0)[rank],
                                   torch.chunk(v, mp, 0)[rank]], 0)
        elif name.endswith("w_gate_up"):
            g, u = w[:f], w[f:]
            out[name] = torch.cat([torch.chunk(g, mp, 0)[rank], torch.chunk(u, mp, 0)[rank]], 0)
        elif name.endswith("wo") or name.endswith("w_down"):
            out[name] = torch.chunk(w, mp, 1)[rank]
        elif name.endswith("tok_embeddings") or name.endswith("lm_head"):
            out[name] = torch.chunk(w, mp, 0)[rank]
        else:
            out[name] = w
    return {k: v.contiguous() for k, v in out.items()}
