"""GPT-style decoder (learned positions, pre-LayerNorm, GELU FFN, tied output embedding), optionally with
mixture-of-experts FFNs.  Built from ``parallel.transformer`` blocks, so one definition runs stand-alone, tensor +
sequence parallel, data parallel, pipeline parallel and expert parallel, chosen by ``TransformerOpParallelConfig``.

The 2.6B configuration (32 layers, hidden 2560, 32 heads, FFN 10240, vocab 40000, sequence 1024) matches the
GPT/PanGu-alpha 2.6B networks the reference trains with ``parallel._transformer``
(python/mindspore/parallel/_transformer/transformer.py:2276 TransformerEncoder, :671 VocabEmbedding)."""
from __future__ import annotations

import torch

from ..common.initializer import Normal, initializer
from ..common.parameter import Parameter
from ..nn.cell import Cell
from ..ops import fused
from ..ops.primitive import _wrap_out
from ..parallel import tp as TP
from ..parallel.moe import MoEConfig, default_moe_config
from ..parallel.transformer import (CrossEntropyLoss, TransformerEncoder, TransformerOpParallelConfig, VocabEmbedding,
                                    _LayerNorm)


class GPTConfig:
    def __init__(self, batch_size=1, seq_length=1024, vocab_size=40000, hidden_size=2560, num_layers=32,
                 num_heads=32, ffn_hidden_size=None, hidden_act="gelu", dtype=torch.bfloat16, dropout_rate=0.0,
                 moe_config=default_moe_config, parallel_config=None):
        self.batch_size, self.seq_length, self.vocab_size = batch_size, seq_length, vocab_size
        self.hidden_size, self.num_layers, self.num_heads = hidden_size, num_layers, num_heads
        self.ffn_hidden_size = ffn_hidden_size or 4 * hidden_size
        self.hidden_act, self.dtype, self.dropout_rate = hidden_act, dtype, dropout_rate
        self.moe_config = moe_config
        self.parallel_config = parallel_config or TransformerOpParallelConfig(vocab_emb_dp=False)

    def flops_per_token(self, seq=None):
        seq = seq or self.seq_length
        h, f = self.hidden_size, self.ffn_hidden_size
        k = self.moe_config.num_experts_chosen if self.moe_config.expert_num > 1 else 1
        mats = 3 if self.hidden_act == "swiglu" else 2
        gemm = self.num_layers * (4 * h * h + k * mats * h * f) + self.vocab_size * h
        return 6 * gemm + 6 * self.num_layers * 2 * seq * h / 2


GPT_2_6B = dict(seq_length=1024, vocab_size=40000, hidden_size=2560, num_layers=32, num_heads=32,
                ffn_hidden_size=10240)


class GPTModel(Cell):
    def __init__(self, cfg: GPTConfig):
        super().__init__()
        self.cfg = cfg
        pc = cfg.parallel_config
        g = pc.groups()
        self.tp, self.sp = g["tp"], pc.sequence_parallel
        self.word_embedding = VocabEmbedding(cfg.vocab_size, cfg.hidden_size, pc, param_init_type=cfg.dtype,
                                             tp=self.tp, sequence_parallel=self.sp)
        self.position_embedding = Parameter(initializer(Normal(0.02), (cfg.seq_length, cfg.hidden_size), cfg.dtype),
                                            name="position_embedding")
        self.position_embedding.tp_grad_reduce = self.tp.active and self.sp
        self.encoder = TransformerEncoder(cfg.batch_size, cfg.num_layers, cfg.hidden_size, cfg.ffn_hidden_size,
                                          cfg.seq_length, cfg.num_heads, cfg.dropout_rate, cfg.dropout_rate,
                                          cfg.hidden_act, param_init_type=cfg.dtype, moe_config=cfg.moe_config,
                                          parallel_config=pc)
        self.layernorm = _LayerNorm((cfg.hidden_size,), param_init_type=cfg.dtype, tp=self.tp,
                                    sequence_parallel=self.sp)
        self.use_moe = cfg.moe_config.expert_num > 1
        if pc.pipeline_stage > 1:
            self.word_embedding.pipeline_stage = 0
            self.layernorm.pipeline_stage = pc.pipeline_stage - 1

    def construct(self, tokens):
        batch, seq = tokens.shape
        x, table = self.word_embedding(tokens)
        pos = torch.arange(seq, device=tokens.device).repeat(batch)
        if self.tp.active and self.sp:
            n = pos.shape[0] // self.tp.size
            pos = pos[self.tp.rank * n:(self.tp.rank + 1) * n]
        x = x + fused.embedding(self.position_embedding, pos)
        out = self.encoder(x, batch, seq)
        aux = None
        if self.use_moe:
            out, aux = out
        return self.layernorm(out), table, aux


class GPTForCausalLM(Cell):
    """tokens [B, S+1] (or (inputs, labels)) -> mean next-token cross entropy (+ MoE load-balance loss)."""

    def __init__(self, cfg: GPTConfig):
        super().__init__()
        self.cfg = cfg
        self.backbone = GPTModel(cfg)
        self.tp, self.sp = self.backbone.tp, self.backbone.sp
        self.loss = CrossEntropyLoss(cfg.parallel_config, tp=self.tp if self.backbone.word_embedding.split_vocab
                                     else TP.TPGroup(name=None, size=1, rank=0))

    def construct(self, tokens, labels=None):
        if labels is None:
            tokens, labels = tokens[:, :-1], tokens[:, 1:]
        h, table, aux = self.backbone(tokens)
        if self.backbone.word_embedding.split_vocab:
            logits = TP.column_parallel_linear(h, table, self.tp, sequence_parallel=self.sp)
            lab = labels.reshape(-1)
        else:
            logits = fused.linear(h, table)
            lab = labels.reshape(-1)
            if self.tp.active and self.sp:
                n = lab.shape[0] // self.tp.size
                lab = lab[self.tp.rank * n:(self.tp.rank + 1) * n]
        loss = self.loss(logits, lab)
        if aux is not None:
            loss = loss + aux
        return _wrap_out(loss)


def shard_full_weights(full, cfg: GPTConfig, mp: int, rank: int):
    """Slices {name: full tensor} of the model_parallel=1 model into the shard of model-parallel rank ``rank``:
    q/k/v heads inside the fused qkv matrix, FFN mapping rows, projection columns, vocabulary rows of the
    embedding (when it is split); everything else is replicated."""
    hq = cfg.hidden_size
    out = {}
    for name, w in full.items():
        if name.endswith("qkv.weight") or name.endswith("qkv.bias"):
            q, k, v = w[:hq], w[hq:2 * hq], w[2 * hq:]
            out[name] = torch.cat([torch.chunk(t, mp, 0)[rank] for t in (q, k, v)], 0)
        elif name.endswith("mapping.weight") or name.endswith("mapping.bias"):
            out[name] = torch.chunk(w, mp, 0)[rank]
        elif name.endswith("attention.projection.weight") or name.endswith("output.projection.weight"):
            out[name] = torch.chunk(w, mp, 1)[rank]
        elif name.endswith("embedding_table") and not cfg.parallel_config.vocab_emb_dp:
            out[name] = torch.chunk(w, mp, 0)[rank]
        else:
            out[name] = w
    return {k: v.contiguous() for k, v in out.items()}
