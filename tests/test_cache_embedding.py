"""Host-device embedding cache: training through a small cache gives the same table as training the full table."""
import numpy as np
import pytest
import torch

import mindspore_b200 as ms
from mindspore_b200 import nn
from mindspore_b200.parallel.cache_embedding import CachedEmbedding


def test_cached_training_matches_full_table():
    ms.set_seed(0)
    vocab, dim, cache = 50, 4, 8
    emb = CachedEmbedding(vocab, dim, cache, device="cpu")
    ref = torch.nn.Embedding(vocab, dim)
    with torch.no_grad():
        ref.weight.copy_(emb.host_table)
    opt = nn.SGD([emb.cache_table], 0.5)
    ropt = torch.optim.SGD(ref.parameters(), 0.5)
    g = torch.Generator().manual_seed(1)
    for step in range(30):
        ids = torch.randint(0, vocab, (6,), generator=g)
        tgt = torch.randn(6, dim, generator=g)
        out = emb(ms.Tensor(ids))
        torch.testing.assert_close(out.detach().as_subclass(torch.Tensor), ref(ids).detach())
        loss = ((out - tgt) ** 2).sum()
        emb.cache_table.grad = None
        loss.backward()
        opt((ms.Tensor(emb.cache_table.grad),))
        ropt.zero_grad()
        ((ref(ids) - tgt) ** 2).sum().backward()
        ropt.step()
    torch.testing.assert_close(emb.full_table().as_subclass(torch.Tensor), ref.weight.detach())
    assert emb.misses > cache and emb.hits > 0            # rows were evicted and reloaded along the way


def test_limits():
    emb = CachedEmbedding(20, 2, 4, device="cpu")
    with pytest.raises(RuntimeError):
        emb(ms.Tensor(torch.arange(6)))
    with pytest.raises(ValueError):
        emb(ms.Tensor(torch.tensor([25])))
    with pytest.raises(ValueError):
        CachedEmbedding(10, 2, 11)
    out = emb(ms.Tensor(torch.tensor([[1, 2], [2, 3]])))
    assert out.shape == (2, 2, 2)
