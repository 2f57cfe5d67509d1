"""The reference's import paths for the transformer building blocks (``mindspore.parallel._transformer`` and its
sub-modules ``transformer`` / ``layers`` / ``loss`` / ``moe`` / ``op_parallel_config``): everything lives in
``parallel.transformer`` and ``parallel.moe`` here."""
from ..moe import MoE, MoEConfig, Router, TopkRouter, calculate_expert_capacity, default_moe_config
from ..transformer import (AttentionMask, CrossAttention, CrossEntropyLoss, EmbeddingOpParallelConfig, FeedForward,
                           FixedSparseAttention, MultiHeadAttention, Transformer, TransformerDecoder,
                           TransformerDecoderLayer, TransformerEncoder, TransformerEncoderLayer,
                           TransformerOpParallelConfig, TransformerRecomputeConfig, VocabEmbedding, _LayerNorm,
                           _Linear, default_transformer_config)
from .. import moe, transformer
from .. import transformer as layers
from .. import transformer as loss
from .. import transformer as op_parallel_config

OpParallelConfig = TransformerOpParallelConfig

__all__ = ["AttentionMask", "VocabEmbedding", "MultiHeadAttention", "FeedForward", "TransformerEncoder",
           "TransformerDecoder", "TransformerEncoderLayer", "TransformerDecoderLayer", "Transformer",
           "TransformerOpParallelConfig", "EmbeddingOpParallelConfig", "TransformerRecomputeConfig", "MoEConfig",
           "OpParallelConfig", "CrossEntropyLoss", "FixedSparseAttention", "MoE", "Router", "TopkRouter"]

import sys as _sys

for _name, _mod in (("moe", moe), ("transformer", transformer), ("layers", layers), ("loss", loss),
                    ("op_parallel_config", op_parallel_config)):
    _sys.modules.setdefault(__name__ + "." + _name, _mod)      # `from ..._transformer.moe import MoE` resolves
