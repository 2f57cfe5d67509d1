"""The last tier of primitives against plain PyTorch references."""
import numpy as np
import pytest
import torch
import torch.nn.functional as F

import mindspore_b200 as ms
from mindspore_b200 import ops

P = ops.operations


def _plain(x):
    return x.as_subclass(torch.Tensor) if isinstance(x, torch.Tensor) else x


def test_recurrent_cells_match_torch_layers():
    torch.manual_seed(0)
    T, B, I, H = 5, 3, 4, 6
    x = torch.randn(T, B, I)
    lstm = torch.nn.LSTM(I, H)
    # torch packs gates (i, f, g, o) as rows; the primitive takes [I + H, 4H] columns in order (i, g, f, o)
    w = torch.cat([lstm.weight_ih_l0, lstm.weight_hh_l0], 1).detach()
    b = (lstm.bias_ih_l0 + lstm.bias_hh_l0).detach()
    order = torch.cat([torch.arange(0, H), torch.arange(2 * H, 3 * H), torch.arange(H, 2 * H), torch.arange(3 * H, 4 * H)])
    w2, b2 = w[order].t().contiguous(), b[order]
    h0, c0 = torch.randn(1, B, H), torch.randn(1, B, H)
    want, (hn, cn) = lstm(x, (h0, c0))
    outs = P.DynamicRNN()(x, w2, b2, None, h0, c0)
    assert len(outs) == 8
    assert torch.allclose(_plain(outs[0]), want, atol=1e-5) and torch.allclose(_plain(outs[2])[-1], cn[0], atol=1e-5)
    lens = torch.tensor([5, 2, 3])
    masked = P.DynamicRNN()(x, w2, b2, lens, h0, c0)
    assert float(_plain(masked[0])[3, 1].abs().sum()) == 0.0
    ref2, _ = lstm(x[:2, 1:2], (h0[:, 1:2], c0[:, 1:2]))
    assert torch.allclose(_plain(masked[1])[-1, 1], ref2[-1, 0], atol=1e-5)          # the state froze at step 2
    cell = P.BasicLSTMCell(forget_bias=0.0)(x[0], h0[0], c0[0], w2, b2)
    assert torch.allclose(_plain(cell[1]), want[0], atol=1e-5)

    gru = torch.nn.GRU(I, H)
    g0 = torch.randn(B, H)
    want, _ = gru(x, g0.unsqueeze(0))
    outs = P.DynamicGRUV2()(x, gru.weight_ih_l0.t().detach(), gru.weight_hh_l0.t().detach(), gru.bias_ih_l0.detach(),
                            gru.bias_hh_l0.detach(), None, g0)
    assert len(outs) == 6 and torch.allclose(_plain(outs[0]), want, atol=1e-5)
    # torch's update gate multiplies the old state, as here: h' = (1 - z) * n + z * h
    assert torch.allclose(_plain(outs[1])[-1], want[-1], atol=1e-5)


def test_adafactor_update_and_transducer_loss():
    torch.manual_seed(1)
    p = torch.randn(4, 3)
    g = torch.randn(4, 3)
    row, col = torch.zeros(4), torch.zeros(3)
    p0 = p.clone()
    eps = torch.tensor([1e-30, 1e-3])
    P.FusedAdaFactor()(eps, 1.0, 0.9, 0.8, 0.0, 0.1, g, p, torch.zeros(4, 3), row, col, torch.zeros(4, 3))
    sq = g * g + 1e-30
    r, c = 0.2 * sq.mean(-1), 0.2 * sq.mean(-2)
    upd = g * (r / r.mean()).rsqrt().unsqueeze(-1) * c.rsqrt().unsqueeze(0)
    upd = upd / max(1.0, float(upd.pow(2).mean().sqrt()))
    assert torch.allclose(p, p0 - 0.1 * upd, atol=1e-5) and torch.allclose(row, r, atol=1e-6)
    v, gv, full = torch.ones(5), torch.full((5,), 2.0), torch.zeros(5)
    P.FusedAdaFactorWithGlobalNorm()(eps, 1.0, 0.9, 0.0, 0.0, 0.5, gv, v, torch.zeros(5), torch.zeros(1),
                                     torch.zeros(1), full, torch.tensor(4.0))
    assert torch.allclose(v, torch.full((5,), 0.5), atol=1e-5)           # g / 4 -> update g / |g| = 1, lr 0.5

    acts = torch.randn(2, 3, 3, 4)
    labels = torch.tensor([[1, 2], [3, 0]])
    costs, grads = P.RNNTLoss(blank_label=0)(acts, labels, torch.tensor([3, 2]), torch.tensor([2, 1]))
    costs, grads = _plain(costs), _plain(grads)
    logp = torch.log_softmax(acts, -1)

    def brute(b, T, U, lab):
        # sum over all monotone paths from (0, 0) to (T - 1, U - 1), then the final blank
        def walk(t, u):
            if t == T - 1 and u == U - 1:
                return logp[b, t, u, 0]
            terms = []
            if t < T - 1:
                terms.append(logp[b, t, u, 0] + walk(t + 1, u))
            if u < U - 1:
                terms.append(logp[b, t, u, lab[u]] + walk(t, u + 1))
            return torch.logsumexp(torch.stack(terms), 0)
        return -walk(0, 0)
    assert abs(float(costs[0]) - float(brute(0, 3, 3, [1, 2]))) < 1e-4
    assert abs(float(costs[1]) - float(brute(1, 2, 2, [3]))) < 1e-4
    assert grads.shape == acts.shape and float(grads[1, 2].abs().sum()) == 0.0     # past the input length
    assert abs(float(grads[0].sum())) < 1e-4                               # softmax gradients sum to zero


def test_replay_buffer_and_cache_bookkeeping():
    buf = (torch.zeros(4, 2), torch.zeros(4, dtype=torch.int64))
    count, head = torch.zeros(1, dtype=torch.int64), torch.zeros(1, dtype=torch.int64)
    append = P.BufferAppend(4, [(2,), ()], [ms.float32, ms.int64])
    for k in range(6):
        append(buf, (torch.full((2,), float(k)), torch.tensor(k)), count, head)
    assert int(count) == 4 and int(head) == 2 and sorted(buf[1].tolist()) == [2, 3, 4, 5]
    get = P.BufferGetItem(4, [(2,), ()], [ms.float32, ms.int64])
    assert int(_plain(get(buf, count, head, torch.tensor(0))[1])) == 2
    assert int(_plain(get(buf, count, head, torch.tensor(-1))[1])) == 5
    sample = P.BufferSample(4, 3, [(2,), ()], [ms.float32, ms.int64], seed=3, unique=True)(buf, count, head)
    picked = _plain(sample[1]).tolist()
    assert len(set(picked)) == 3 and set(picked) <= {2, 3, 4, 5}
    assert _plain(sample[0])[:, 0].tolist() == [float(v) for v in picked]

    res, idx = P.SubAndFilter()(torch.tensor([1, 5, 9, 12]), 8, 2)
    assert _plain(res).tolist() == [3, 7] and _plain(idx).tolist() == [1, 2]
    assert _plain(P.MapUniform()(torch.tensor([0, 1, 2, 3, 4, 5]), 3, 2)).tolist() == [0, 3, 1, 4, 2, 5]
    table = torch.zeros(8, 4, dtype=torch.int64)
    cache, old, miss, swap = P.MapCacheIdx()(table, torch.tensor([10, 11, 10, 99]), 1, 50, 0)
    assert _plain(cache).tolist() == [0, 1, 0, -1] and _plain(miss).tolist() == [10, 11] and _plain(old).numel() == 0
    cache, _, miss, _ = P.MapCacheIdx()(table, torch.tensor([11, 12]), 2, 50, 0)
    assert _plain(cache).tolist() == [1, 2] and _plain(miss).tolist() == [12]
    key = P.Push("ApplyMomentum")((torch.ones(2),), ((2,),))
    assert int(_plain(key)) >= 0 and P.Pull()(key, torch.ones(2)).tolist() == [1.0, 1.0]


def test_patches_pooling_and_resampling():
    torch.manual_seed(2)
    x = torch.randn(1, 2, 4, 5, 6)
    out = _plain(P.ExtractVolumePatches([1, 1, 2, 2, 2], [1, 1, 2, 1, 1], "VALID")(x))
    assert out.shape == (1, 16, 2, 4, 5)
    # channel = ((kd * 2 + kh) * 2 + kw) * C + c
    assert torch.equal(out[0, ((1 * 2 + 0) * 2 + 1) * 2 + 1, 1, 2, 3], x[0, 1, 2 * 1 + 1, 2 + 0, 3 + 1])
    same = _plain(P.ExtractVolumePatches([1, 1, 3, 3, 3], [1, 1, 1, 1, 1], "SAME")(x))
    assert same.shape == (1, 54, 4, 5, 6)

    img = torch.randn(2, 3, 9, 9)
    samples = torch.rand(2, 3, 2)
    y, arg = P.FractionalMaxPoolWithFixedKsize(2, (4, 4))(img, samples)
    want, widx = F.fractional_max_pool2d(img, 2, output_size=(4, 4), return_indices=True, _random_samples=samples)
    assert torch.equal(_plain(y), want) and torch.equal(_plain(arg), widx)
    vol = torch.randn(1, 2, 7, 7, 7)
    y3, _ = P.FractionalMaxPool3DWithFixedKsize(2, (3, 3, 3))(vol, torch.rand(1, 2, 3))
    assert _plain(y3).shape == (1, 2, 3, 3, 3)
    nhwc = torch.randn(1, 9, 9, 2)
    y, rows, cols = P.FractionalMaxPool([1.0, 1.5, 1.5, 1.0], seed=1)(nhwc)
    rows, cols = _plain(rows).tolist(), _plain(cols).tolist()
    assert _plain(y).shape == (1, 6, 6, 2) and rows[0] == 0 and rows[-1] == 9 and len(rows) == 7
    assert all(1 <= b - a <= 2 for a, b in zip(rows, rows[1:]))
    assert torch.equal(_plain(y)[0, 0, 0], nhwc[0, rows[0]:rows[1], cols[0]:cols[1]].amax((0, 1)))
    ya, rows, cols = P.FractionalAvgPool([1.0, 2.0, 2.0, 1.0], pseudo_random=True, seed=4)(nhwc)
    rows, cols = _plain(rows).tolist(), _plain(cols).tolist()
    assert torch.allclose(_plain(ya)[0, 1, 2], nhwc[0, rows[1]:rows[2], cols[2]:cols[3]].mean((0, 1)), atol=1e-6)

    pic = torch.rand(1, 6, 8, 3)
    same = P.ScaleAndTranslate("triangle", antialias=True)(pic, torch.tensor([6, 8]), torch.tensor([1.0, 1.0]),
                                                           torch.tensor([0.0, 0.0]))
    assert torch.allclose(_plain(same), pic, atol=1e-6)
    half = P.ScaleAndTranslate("box", antialias=True)(pic, torch.tensor([3, 4]), torch.tensor([0.5, 0.5]),
                                                      torch.tensor([0.0, 0.0]))
    assert torch.allclose(_plain(half), F.avg_pool2d(pic.permute(0, 3, 1, 2), 2).permute(0, 2, 3, 1), atol=1e-6)
    shifted = P.ScaleAndTranslate("triangle")(pic, torch.tensor([6, 8]), torch.tensor([1.0, 1.0]),
                                              torch.tensor([0.0, 2.0]))
    assert torch.allclose(_plain(shifted)[:, :, 2:], pic[:, :, :-2], atol=1e-6)
    for kind in ("lanczos1", "lanczos3", "lanczos5", "gaussian", "keyscubic", "mitchellcubic"):
        up = _plain(P.ScaleAndTranslate(kind)(torch.ones(1, 4, 4, 1), torch.tensor([8, 8]), torch.tensor([2.0, 2.0]),
                                              torch.tensor([0.0, 0.0])))
        assert torch.allclose(up, torch.ones(1, 8, 8, 1), atol=1e-5)       # the weights of a sample sum to one


def test_detection_deformable_and_sparse():
    overlaps = torch.tensor([[1.0, 0.8, 0.1], [0.8, 1.0, 0.2], [0.1, 0.2, 1.0]])
    keep = P.NonMaxSuppressionWithOverlaps()(overlaps, torch.tensor([0.9, 0.8, 0.7]), 3, 0.5, 0.0)
    assert _plain(keep).tolist() == [0, 2]
    boxes = torch.tensor([[[[0.0, 0.0, 0.5, 0.5]], [[0.0, 0.0, 0.52, 0.5]], [[0.5, 0.5, 1.2, 1.0]]]])
    scores = torch.tensor([[[0.9, 0.1], [0.8, 0.7], [0.3, 0.6]]])
    nb, ns, nc, valid = P.CombinedNonMaxSuppression()(boxes, scores, 2, 4, 0.5, 0.2)
    assert int(_plain(valid)[0]) == 4
    assert [round(v, 2) for v in _plain(ns)[0].tolist()] == [0.9, 0.7, 0.6, 0.3]
    assert _plain(nc)[0].tolist() == [0.0, 1.0, 1.0, 0.0] and float(_plain(nb)[0, 2, 2]) == 1.0     # clipped

    torch.manual_seed(3)
    x = torch.randn(2, 4, 6, 7)
    w = torch.randn(5, 4, 3, 3)
    off = torch.zeros(2, 3 * 1 * 9, 6, 7)
    off[:, 18:] = 1.0                                                      # masks
    sampled = P.DeformableOffsets((1, 1, 1, 1), (1, 1, 1, 1), (3, 3))(x, off)
    assert _plain(sampled).shape == (2, 4, 18, 21)
    assert torch.allclose(F.conv2d(_plain(sampled), w, stride=3), F.conv2d(x, w, padding=1), atol=1e-4)
    off[:, 0:9] = 1.0                                                      # every tap one pixel to the right
    moved = P.DeformableOffsets((1, 1, 1, 1), (1, 1, 1, 1), (3, 3))(x, off)
    assert torch.allclose(F.conv2d(_plain(moved), w, stride=3)[..., :-1], F.conv2d(x, w, padding=1)[..., 1:], atol=1e-4)

    begin, size, box = P.SampleDistortedBoundingBoxV2(seed=5, area_range=(0.3, 0.6))(
        torch.tensor([40, 60, 3]), torch.tensor([[[0.1, 0.1, 0.9, 0.9]]]), torch.tensor([0.1]))
    begin, size, box = _plain(begin).tolist(), _plain(size).tolist(), _plain(box)
    assert size[2] == -1 and 0.3 * 2400 * 0.9 <= size[0] * size[1] <= 0.6 * 2400 * 1.1
    assert begin[0] + size[0] <= 40 and begin[1] + size[1] <= 60 and 0.7 <= (size[1] / size[0]) <= 1.4
    assert abs(float(box[0, 0, 0]) - begin[0] / 40) < 1e-6

    idx = torch.tensor([[0, 1], [1, 2], [2, 3], [3, 0]])
    yi, yv, ys = P.SparseSlice()(idx, torch.tensor([1.0, 2.0, 3.0, 4.0]), torch.tensor([4, 4]), torch.tensor([1, 1]),
                                 torch.tensor([2, 5]))
    assert _plain(yi).tolist() == [[0, 1], [1, 2]] and _plain(yv).tolist() == [2.0, 3.0] and _plain(ys).tolist() == [2, 3]
    assert P.Partial is ops.Partial and float(P.identity(ms.Tensor(np.array([2.0], np.float32)))[0]) == 2.0
