"""parallel.transformer beyond the GPT stack: decoder layer with attention over the encoder output, the
encoder-decoder Transformer, FixedSparseAttention's pattern, and the dense Router / TopkRouter tensors."""
import math

import numpy as np
import pytest
import torch

import mindspore_b200 as ms
from mindspore_b200.parallel import moe as MOE
from mindspore_b200.parallel import transformer as T


def _manual_attention(x, mem, wq, bq, wkv, bkv, wo, bo, heads, batch, tq, ts):
    H = x.shape[-1]
    d = H // heads
    q = (x @ wq.t() + bq).reshape(batch, tq, heads, d).permute(0, 2, 1, 3)
    kv = mem @ wkv.t() + bkv
    k = kv[:, :H].reshape(batch, ts, heads, d).permute(0, 2, 1, 3)
    v = kv[:, H:].reshape(batch, ts, heads, d).permute(0, 2, 1, 3)
    p = torch.softmax(q @ k.transpose(-1, -2) / math.sqrt(d), -1)
    o = (p @ v).permute(0, 2, 1, 3).reshape(batch * tq, H)
    return o @ wo.t() + bo


def test_cross_attention_matches_manual_formula():
    ms.set_seed(0)
    B, TQ, TS, H, heads = 2, 6, 10, 32, 4
    att = T.CrossAttention(H, heads)
    with torch.no_grad():
        for p in att.get_parameters():
            p.copy_(torch.randn(p.shape) * 0.2)
    x, mem = torch.randn(B * TQ, H), torch.randn(B * TS, H)
    got = att(ms.Tensor(x), ms.Tensor(mem), B, TQ, TS)
    t = lambda p: p.detach().as_subclass(torch.Tensor)
    ref = _manual_attention(x, mem, t(att.wq), t(att.bq), t(att.wkv), t(att.bkv), t(att.wo), t(att.bo), heads, B, TQ,
                            TS)
    np.testing.assert_allclose(got.detach().numpy(), ref.numpy(), rtol=1e-4, atol=1e-5)


def test_transformer_encoder_is_bidirectional_and_decoder_causal():
    ms.set_seed(1)
    B, S_SRC, S_TGT, H = 2, 8, 6, 32
    net = T.Transformer(hidden_size=H, batch_size=B, ffn_hidden_size=64, src_seq_length=S_SRC, tgt_seq_length=S_TGT,
                        encoder_layers=2, decoder_layers=2, num_heads=4)
    names = [p.name for p in net.get_parameters()]
    assert any("cross_attention" in n for n in names) and len(set(names)) == len(names)
    enc = torch.randn(B * S_SRC, H)
    dec = torch.randn(B * S_TGT, H)
    out, memory = net(ms.Tensor(enc), ms.Tensor(dec), B)
    assert out.shape == (B * S_TGT, H) and memory.shape == (B * S_SRC, H)
    # encoder: changing the LAST source token changes the memory of the FIRST one (no causal mask)
    enc2 = enc.clone()
    enc2[S_SRC - 1] += torch.randn(H)            # (a constant shift would vanish in the layer norm)
    out2, memory2 = net(ms.Tensor(enc2), ms.Tensor(dec), B)
    plain = lambda t: t.detach().as_subclass(torch.Tensor)
    out, memory, out2, memory2 = plain(out), plain(memory), plain(out2), plain(memory2)
    assert float((memory2[0] - memory[0]).abs().max()) > 1e-6
    # every decoder token of batch 0 sees the changed memory; batch 1 does not
    assert float((out2[:S_TGT] - out[:S_TGT]).abs().min(0).values.max()) > 1e-7
    np.testing.assert_allclose(out2[S_TGT:].numpy(), out[S_TGT:].numpy(), atol=1e-6)
    # decoder: changing the LAST target token leaves the earlier outputs alone (causal self-attention)
    dec2 = dec.clone()
    dec2[S_TGT - 1] += torch.randn(H)
    out3 = plain(net(ms.Tensor(enc), ms.Tensor(dec2), B)[0])
    np.testing.assert_allclose(out3[:S_TGT - 1].numpy(), out[:S_TGT - 1].numpy(), atol=1e-6)
    assert float((out3[S_TGT - 1] - out[S_TGT - 1]).abs().max()) > 1e-6
    # gradients reach encoder and decoder parameters
    net(ms.Tensor(enc), ms.Tensor(dec), B)[0].float().sum().backward()
    assert all(p.grad is not None for p in net.trainable_params())
    # encoder alone
    only = T.Transformer(hidden_size=H, batch_size=B, ffn_hidden_size=64, src_seq_length=S_SRC, tgt_seq_length=S_TGT,
                         encoder_layers=1, decoder_layers=0, num_heads=4)
    a, b = only(ms.Tensor(enc))
    assert a is b and a.shape == (B * S_SRC, H)


def test_fixed_sparse_attention_pattern_and_values():
    ms.set_seed(2)
    B, heads, D, S, blk = 2, 8, 16, 64, 16
    layer = T.FixedSparseAttention(B, heads, D, blk, seq_length=S, num_different_global_patterns=4)
    lay = layer.layout()
    assert lay.shape == (heads, S, S)
    # causal: nothing above the diagonal; own block fully visible below it
    assert not bool(torch.triu(lay, 1).any())
    assert bool(lay[0, 21, 16:22].all())
    # earlier blocks: only the head's summary slice (pattern 0: last 4 tokens of a block; pattern 1: the 4 before)
    assert lay[0, 40, :32].nonzero().flatten().tolist() == [12, 13, 14, 15, 28, 29, 30, 31]
    assert lay[1, 40, :32].nonzero().flatten().tolist() == [8, 9, 10, 11, 24, 25, 26, 27]
    assert bool((lay[4] == lay[0]).all())                       # heads cycle through the patterns
    q, k, v = (torch.randn(B, S, heads * D) for _ in range(3))
    out = layer(ms.Tensor(q), ms.Tensor(k), ms.Tensor(v), ms.Tensor(torch.ones(B, S, S)))
    assert out.shape == (B, S, heads * D)
    sp = lambda t: t.reshape(B, S, heads, D).permute(0, 2, 1, 3)
    scores = sp(q) @ sp(k).transpose(-1, -2) / math.sqrt(D)
    scores = scores.masked_fill(~lay[None], float("-inf"))
    ref = (torch.softmax(scores, -1) @ sp(v)).permute(0, 2, 1, 3).reshape(B, S, heads * D)
    np.testing.assert_allclose(out.detach().numpy(), ref.numpy(), rtol=1e-4, atol=1e-5)
    with pytest.raises(ValueError):
        T.FixedSparseAttention(B, heads, D, 24, seq_length=S)


def test_topk_router_dense_tensors_agree_with_index_form():
    ms.set_seed(3)
    cfg = MOE.MoEConfig(expert_num=4, capacity_factor=1.0, num_experts_chosen=2)
    router = T.Router(16, cfg)
    x = torch.randn(3, 12, 16)                                  # three routing groups of 12 tokens
    dispatch, combine, loss = router(ms.Tensor(x))
    C = MOE.calculate_expert_capacity(2, 12, 1.0, 4)
    assert dispatch.shape == (3, 12, 4, C) and combine.shape == dispatch.shape and loss.ndim == 0
    d = dispatch.detach()
    assert float(d.sum((0, 1)).max()) <= 3.0                    # one token per (group, expert, slot)
    assert float(d.sum(1).max()) <= 1.0
    assert float(d.sum((2, 3)).max()) <= 2.0                    # at most k experts per token
    logits = x[1] @ router.weight.detach().as_subclass(torch.Tensor).t()
    expert, slot, weight, l1 = MOE.router_reference(logits, 2, C)
    for t in range(12):
        for j in range(2):
            if int(slot[t, j]) >= 0:
                assert float(d[1, t, int(expert[t, j]), int(slot[t, j])]) == 1.0
                assert float(combine[1, t, int(expert[t, j]), int(slot[t, j])]) == pytest.approx(float(weight[t, j]),
                                                                                                 rel=1e-5)
    assert float(combine.sum()) == pytest.approx(float(sum(MOE.router_reference(
        x[g] @ router.weight.detach().as_subclass(torch.Tensor).t(), 2, C)[2].sum() for g in range(3))), rel=1e-4)
    loss.backward()
    assert router.weight.grad is not None and float(router.weight.grad.abs().sum()) > 0
