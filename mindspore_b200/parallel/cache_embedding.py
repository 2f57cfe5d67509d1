"""Host-device embedding cache: the full table lives in (pinned) host memory, the device holds ``vocab_cache_size``
rows - the ones used most recently - as the trainable parameter.  Before each lookup the ids of the batch are
mapped to cache slots; rows that are missing are loaded, and the rows they push out (least recently used, never one
needed by the current batch) are written back to the host table first, so updates made by the optimizer on the
device are not lost.

    emb = CachedEmbedding(vocab_size=50_000_000, embedding_size=64, vocab_cache_size=1_000_000)
    y = emb(ids)              # [..., 64]; gradients flow into emb.cache_table (a [cache, 64] Parameter)
    emb.flush()               # write every cached row back (before saving the host table)

The reference does this with a pair of passes and host-side hash maps (frontend/parallel/cache_embedding/
cache_embedding.cc: ``AddCacheEmbedding`` inserts MapCacheIdx / UpdateCache / swap ops around ``EmbeddingLookup``
when ``nn.EmbeddingLookup(vocab_cache_size>0)``; plugin/device/gpu/kernel/... map_cache_idx).  Here slot lookup,
victim choice and the swaps are tensor operations on the device; the only host work per step is the copy of the
missing / evicted rows."""
from __future__ import annotations

import torch

from ..common import dtype as mstype
from ..common.initializer import initializer
from ..common.parameter import Parameter
from ..common.tensor import Tensor
from ..nn.cell import Cell
from ..ops.primitive import _wrap_out


class CachedEmbedding(Cell):
    def __init__(self, vocab_size, embedding_size, vocab_cache_size, param_init="normal", dtype=mstype.float32,
                 device=None):
        super().__init__()
        if not 0 < vocab_cache_size <= vocab_size:
            raise ValueError("'vocab_cache_size' must be in (0, vocab_size], but got %d" % vocab_cache_size)
        self.vocab_size, self.embedding_size, self.cache_size = int(vocab_size), int(embedding_size), int(vocab_cache_size)
        dev = torch.device(device) if device is not None else torch.device("cuda" if torch.cuda.is_available() else "cpu")
        host = torch.as_tensor(initializer(param_init, (vocab_size, embedding_size), dtype)).detach().to("cpu")
        self.host_table = host.pin_memory() if torch.cuda.is_available() else host
        self.cache_table = Parameter(Tensor(torch.zeros(self.cache_size, embedding_size, dtype=host.dtype, device=dev)),
                                     name="cache_table")
        # id -> slot (-1: not cached), slot -> id (-1: free), slot -> step of last use
        self._slot_of = torch.full((vocab_size,), -1, dtype=torch.int64, device=dev)
        self._id_of = torch.full((self.cache_size,), -1, dtype=torch.int64, device=dev)
        self._last_use = torch.zeros(self.cache_size, dtype=torch.int64, device=dev)
        self._step = 0
        self.hits = self.misses = 0

    # ------------------------------------------------------------------ cache maintenance
    def _admit(self, ids):
        """Makes every id of ``ids`` resident and returns their slots."""
        dev = self._slot_of.device
        self._step += 1
        uniq = torch.unique(ids.reshape(-1))
        if uniq.numel() > self.cache_size:
            raise RuntimeError("a batch uses %d distinct ids, more than the cache holds (%d)"
                               % (uniq.numel(), self.cache_size))
        slots = self._slot_of[uniq]
        missing = uniq[slots < 0]
        self.hits += int(uniq.numel() - missing.numel())
        self.misses += int(missing.numel())
        self._last_use[slots[slots >= 0]] = self._step
        if missing.numel():
            # victims: free slots first, then least recently used; slots touched in this step are never chosen
            age = self._last_use.clone()
            age[self._id_of < 0] = -1
            age[self._last_use == self._step] = torch.iinfo(torch.int64).max
            victims = torch.topk(age, missing.numel(), largest=False).indices
            old_ids = self._id_of[victims]
            live = old_ids >= 0
            with torch.no_grad():
                table = self.cache_table.detach()
                if bool(live.any()):
                    rows = table[victims[live]].to("cpu")
                    self.host_table[old_ids[live].to("cpu")] = rows
                    self._slot_of[old_ids[live]] = -1
                table[victims] = self.host_table[missing.to("cpu")].to(dev, non_blocking=True)
            self._slot_of[missing] = victims
            self._id_of[victims] = missing
            self._last_use[victims] = self._step
        return self._slot_of[ids]

    def flush(self):
        """Writes every cached row back into the host table."""
        live = self._id_of >= 0
        with torch.no_grad():
            self.host_table[self._id_of[live].to("cpu")] = self.cache_table.detach()[live].to("cpu")

    def full_table(self):
        self.flush()
        return Tensor(self.host_table.clone())

    # ------------------------------------------------------------------ forward
    def construct(self, indices):
        ids = indices.long()
        if bool(((ids < 0) | (ids >= self.vocab_size)).any()):
            raise ValueError("embedding ids must be in [0, %d)" % self.vocab_size)
        slots = self._admit(ids.to(self._slot_of.device))
        return _wrap_out(torch.nn.functional.embedding(slots, self.cache_table))
