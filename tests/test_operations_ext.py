"""Second-tier primitives against numpy / scipy / torch restatements of the documented semantics."""
import numpy as np
import pytest
import scipy.special as sp
import torch

import mindspore_b200 as ms
from mindspore_b200.ops import operations as P
from mindspore_b200.parallel import operator_info as OI


def T(a, dtype=None):
    return ms.Tensor(np.asarray(a, dtype=dtype))


def test_registry_maps_names_to_classes():
    assert len(OI._REGISTRY) >= 290
    assert all(isinstance(v, type) and issubclass(v, OI.OperatorInfo) for v in OI._REGISTRY.values())
    for name in ("Add", "Mul", "PagedAttention", "ScatterNdAdd", "FFN", "Conv3D"):
        assert OI.get_info_class(name) is not None


def test_special_functions():
    a = np.array([0.5, 2.0, 3.5, 7.0]); b = np.array([1.5, 0.7, 2.0, 3.0]); x = np.array([0.1, 0.5, 0.9, 0.3])
    np.testing.assert_allclose(P.Betainc()(T(a), T(b), T(x)).numpy(), sp.betainc(a, b, x), rtol=1e-6)
    np.testing.assert_allclose(P.Igamma()(T(a), T(x)).numpy(), sp.gammainc(a, x), rtol=1e-6)
    np.testing.assert_allclose(P.BesselJ0()(T(x)).numpy(), sp.j0(x), rtol=1e-6)
    assert P.PopulationCount()(T([0, 1, 255, -1], np.int16)).tolist() == [0, 1, 8, 16]
    assert P.Gcd()(T([12, 18], np.int32), T([8, 27], np.int32)).tolist() == [4, 9]


def test_scatter_families():
    x = ms.Parameter(T(np.zeros((4, 3), np.float32)), name="x")
    P.ScatterAdd()(x, T([[0, 2], [2, 3]], np.int32), T(np.ones((2, 2, 3), np.float32)))
    assert x.numpy()[:, 0].tolist() == [1, 0, 2, 1]
    P.ScatterMax()(x, T([1], np.int32), T(np.full((1, 3), 5, np.float32)))
    assert x.numpy()[1].tolist() == [5, 5, 5]
    base = T(np.arange(12, dtype=np.float32).reshape(3, 4))
    out = P.TensorScatterMul()(base, T([[0, 0], [2, 3]], np.int32), T([10.0, 2.0], np.float32))
    exp = np.arange(12, dtype=np.float32).reshape(3, 4); exp[0, 0] *= 10; exp[2, 3] *= 2
    np.testing.assert_allclose(out.numpy(), exp)
    seg = P.UnsortedSegmentMax()(T([[1., 5.], [3., 2.], [4., 9.]], np.float32), T([0, 1, 0], np.int32), 2)
    assert seg.numpy().tolist() == [[4, 9], [3, 2]]
    assert P.InplaceAdd((0, 2))(T(np.zeros((3, 2), np.float32)), T(np.ones((2, 2), np.float32))).numpy().sum() == 4


def test_conv3d_and_pool3d_match_torch():
    g = torch.Generator().manual_seed(0)
    x = torch.randn(2, 3, 5, 6, 7, generator=g); w = torch.randn(4, 3, 3, 3, 3, generator=g)
    y = P.Conv3D(4, 3, pad_mode="same", stride=1)(ms.Tensor(x), ms.Tensor(w))
    torch.testing.assert_close(torch.as_tensor(y.numpy()), torch.nn.functional.conv3d(x, w, padding=1), rtol=1e-4,
                               atol=1e-4)
    p = P.MaxPool3D(kernel_size=2, strides=2)(ms.Tensor(x))
    torch.testing.assert_close(torch.as_tensor(p.numpy()), torch.nn.functional.max_pool3d(x, 2, 2))
    dx = P.Conv2DBackpropInput(4, 3, pad_mode="pad", pad=1)(ms.Tensor(torch.randn(1, 4, 5, 5, generator=g)),
                                                            ms.Tensor(torch.randn(4, 2, 3, 3, generator=g)), (1, 2, 5, 5))
    assert tuple(dx.shape) == (1, 2, 5, 5)


def test_quantisation_round_trip():
    x = T(np.linspace(-2, 2, 17), np.float32)
    q = P.Quant(scale=50.0, offset=0.0)(x)
    assert q.dtype == torch.int8 and q.tolist()[0] == -100 and q.tolist()[-1] == 100
    back = P.AntiQuant(scale=1 / 50.0, offset=0.0, dtype=torch.float32)(q)
    np.testing.assert_allclose(back.numpy(), x.numpy(), atol=0.011)
    xq, sc = P.DynamicQuantExt()(T(np.random.default_rng(0).normal(size=(4, 64)), np.float32))
    assert xq.dtype == torch.int8 and sc.shape == (4,) and int(xq.abs().max()) == 127
    xin = ms.Tensor(torch.linspace(-3, 3, 50).requires_grad_(True))
    y = P.FakeQuantPerLayer(num_bits=8)(xin, T([-1.0], np.float32), T([1.0], np.float32))
    assert float(y.max()) <= 1.01 and float(y.min()) >= -1.01
    a = torch.randint(-128, 127, (3, 16), dtype=torch.int8); b = torch.randint(-128, 127, (16, 5), dtype=torch.int8)
    out = P.QuantBatchMatmul(dtype=torch.float32)(ms.Tensor(a), ms.Tensor(b), T([0.5], np.float32))
    np.testing.assert_allclose(out.numpy(), (a.double() @ b.double() * 0.5).numpy())
    w = torch.randint(-8, 8, (16, 6), dtype=torch.int8)
    o2 = P.WeightQuantBatchMatmul(antiquant_group_size=8)(ms.Tensor(torch.randn(2, 16)), ms.Tensor(w),
                                                          ms.Tensor(torch.full((2, 6), 0.1)))
    assert tuple(o2.shape) == (2, 6)


def _attn_ref(q, k, v, scale, causal):
    s = torch.einsum("bhqd,bhkd->bhqk", q, k) * scale
    if causal:
        Sq, Sk = s.shape[-2:]
        s = s.masked_fill(torch.arange(Sk)[None] > torch.arange(Sk - Sq, Sk)[:, None], float("-inf"))
    return torch.softmax(s, -1) @ v


def test_paged_and_incremental_attention():
    g = torch.Generator().manual_seed(1)
    B, H, KVH, D, bs, L = 2, 4, 2, 8, 4, 10
    k = torch.randn(B, L, KVH, D, generator=g); v = torch.randn(B, L, KVH, D, generator=g)
    q = torch.randn(B, 1, H * D, generator=g)
    nblocks = 8
    kc = torch.zeros(nblocks, bs, KVH, D); vc = torch.zeros(nblocks, bs, KVH, D)
    tables = torch.tensor([[5, 1, 7], [0, 3, 2]])
    slots = torch.stack([torch.tensor([tables[b, t // bs] * bs + t % bs for t in range(L)]) for b in range(B)])
    P.ReshapeAndCache()(ms.Tensor(k.reshape(B * L, KVH * D)), ms.Tensor(v.reshape(B * L, KVH * D)), ms.Tensor(kc),
                        ms.Tensor(vc), ms.Tensor(slots.reshape(-1)))
    lens = torch.tensor([L, 7])
    out = P.PagedAttention(H, scale_value=D ** -0.5, kv_head_num=KVH)(ms.Tensor(q), ms.Tensor(kc), ms.Tensor(vc),
                                                                     ms.Tensor(tables), ms.Tensor(lens))
    for b in range(B):
        n = int(lens[b])
        kk = k[b, :n].repeat_interleave(H // KVH, 1).permute(1, 0, 2)[None]
        vv = v[b, :n].repeat_interleave(H // KVH, 1).permute(1, 0, 2)[None]
        ref = _attn_ref(q[b].reshape(1, 1, H, D).permute(0, 2, 1, 3), kk, vv, D ** -0.5, False)
        torch.testing.assert_close(torch.as_tensor(out.numpy())[b].reshape(H, D), ref[0, :, 0], rtol=1e-4, atol=1e-5)
    # dense-cache decode, BSH layout, same numbers for batch 0
    inc = P.IncreFlashAttention(H, "BSH", D ** -0.5, KVH)(ms.Tensor(q), ms.Tensor(k.reshape(B, L, KVH * D)),
                                                          ms.Tensor(v.reshape(B, L, KVH * D)), None, [L, 7])
    torch.testing.assert_close(torch.as_tensor(inc.numpy()), torch.as_tensor(out.numpy()), rtol=1e-4, atol=1e-5)
    # prefill, causal
    qf = torch.randn(B, L, H * D, generator=g)
    pf = P.PromptFlashAttention(H, D ** -0.5, next_tokens=0, input_layout="BSH", num_key_value_heads=KVH)(
        ms.Tensor(qf), ms.Tensor(k.reshape(B, L, KVH * D)), ms.Tensor(v.reshape(B, L, KVH * D)))
    ref = _attn_ref(qf.reshape(B, L, H, D).permute(0, 2, 1, 3), k.repeat_interleave(2, 2).permute(0, 2, 1, 3),
                    v.repeat_interleave(2, 2).permute(0, 2, 1, 3), D ** -0.5, True)
    torch.testing.assert_close(torch.as_tensor(pf.numpy()), ref.permute(0, 2, 1, 3).reshape(B, L, H * D), rtol=1e-4,
                               atol=1e-5)


def test_kv_cache_updates():
    cache = ms.Tensor(torch.zeros(2, 3, 6, 4))
    P.DecoderKVCache()(cache, ms.Tensor(torch.ones(2, 3, 1, 4)), ms.Tensor(torch.tensor([2, 5])), None, 2)
    c = cache.numpy()
    assert c[0, :, 2].sum() == 12 and c[1, :, 5].sum() == 12 and c.sum() == 24
    P.PromptKVCache()(cache, ms.Tensor(torch.full((1, 3, 4, 4), 2.0)), ms.Tensor(torch.tensor([4])),
                      ms.Tensor(torch.tensor([1])), 2)
    assert cache.numpy()[1, :, :4].sum() == 2 * 3 * 4 * 4


def test_ffn_grouped_matmul_and_routing():
    g = torch.Generator().manual_seed(2)
    x = torch.randn(6, 8, generator=g); w1 = torch.randn(8, 16, generator=g); w2 = torch.randn(8, 8, generator=g)
    y = P.FFN("swiglu")(ms.Tensor(x), ms.Tensor(w1), ms.Tensor(w2))
    a, gt = (x @ w1).chunk(2, -1)
    torch.testing.assert_close(torch.as_tensor(y.numpy()), (a * torch.nn.functional.silu(gt)) @ w2, rtol=1e-4,
                               atol=1e-4)
    ws = torch.randn(3, 8, 5, generator=g)
    out = P.GroupedMatmul(split_item=3, group_type=0)(ms.Tensor(x), ms.Tensor(ws), None, None, None, None, None,
                                                      ms.Tensor(torch.tensor([2, 2, 6])))
    ref = torch.cat([x[:2] @ ws[0], x[2:6] @ ws[2]])
    torch.testing.assert_close(torch.as_tensor(out.numpy()), ref, rtol=1e-4, atol=1e-4)
    T_, K = 3, 2
    ex = torch.randn(T_ * K, 4, generator=g); scales = torch.rand(T_, K, generator=g)
    row = torch.randperm(T_ * K, generator=g)
    fin = P.MoeFinalizeRouting()(ms.Tensor(ex), ms.Tensor(torch.zeros(T_, 4)), None, None, ms.Tensor(scales),
                                 ms.Tensor(row), ms.Tensor(torch.zeros(T_, K, dtype=torch.int64)))
    ref = sum(scales[:, k:k + 1] * ex[row[k * T_:(k + 1) * T_]] for k in range(K))
    torch.testing.assert_close(torch.as_tensor(fin.numpy()), ref, rtol=1e-5, atol=1e-5)


def test_detection_helpers_and_masks():
    anchors = T([[0, 0, 9, 9], [5, 5, 14, 14]], np.float32); gt = T([[0, 0, 9, 9]], np.float32)
    iou = P.IOU()(anchors, gt).numpy()
    np.testing.assert_allclose(iou, [[1.0, 25 / 175]], rtol=1e-5)
    enc = P.BoundingBoxEncode()(anchors, T([[0, 0, 9, 9], [5, 5, 14, 14]], np.float32))
    assert np.abs(enc.numpy()).max() < 1e-6
    dec = P.BoundingBoxDecode(max_shape=(100, 100))(anchors, enc)
    np.testing.assert_allclose(dec.numpy(), anchors.numpy(), atol=1e-4)
    pos, mask = P.GenerateEodMask(eod_token_id=9)(T([[1, 2, 9, 3, 4, 9, 5]], np.int64))
    assert pos.tolist() == [[0, 1, 2, 0, 1, 2, 0]]
    assert not bool(mask[0, 4, 3]) and bool(mask[0, 4, 1]) and bool(mask[0, 3, 4])
    m = P.DropoutGenMask()((4, 50), 0.8)
    y = P.DropoutDoMask()(ms.Tensor(torch.ones(4, 50)), m, 0.8)
    kept = float((y > 0).float().mean())
    assert 0.6 < kept < 0.95 and abs(float(y.max()) - 1.25) < 1e-6


def test_custom_pyfunc_with_bprop():
    op = P.Custom(lambda a, b: a * b, bprop=lambda a, b, out, dout: (dout * b, dout * a))
    a = ms.Tensor(torch.tensor([1.0, 2.0])).requires_grad_(True)
    b = ms.Tensor(torch.tensor([3.0, 4.0])).requires_grad_(True)
    op(a, b).sum().backward()
    assert a.grad.tolist() == [3.0, 4.0] and b.grad.tolist() == [1.0, 2.0]
