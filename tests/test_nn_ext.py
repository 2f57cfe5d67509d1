"""Extended layers and optimizers: RNN cells against torch.nn cells with the same weights, transposed / 3-D
convolutions against torch.nn.functional, the Transformer stack end to end, LazyAdam / AdamOffload against Adam,
THOR's preconditioner, AdaSum on two CPU ranks."""
import numpy as np
import torch

import mindspore_b200 as ms
from mindspore_b200 import nn
from _mp import run_ranks


def _t(x):
    return ms.Tensor(x)


def test_rnn_cells_match_torch():
    torch.manual_seed(0)
    x, h, c = torch.randn(3, 5), torch.randn(3, 7), torch.randn(3, 7)
    for ours, ref in ((nn.LSTMCell(5, 7), torch.nn.LSTMCell(5, 7)), (nn.GRUCell(5, 7), torch.nn.GRUCell(5, 7)),
                      (nn.RNNCell(5, 7), torch.nn.RNNCell(5, 7))):
        with torch.no_grad():
            for n in ("weight_ih", "weight_hh", "bias_ih", "bias_hh"):
                getattr(ref, n).copy_(getattr(ours, n))
        if isinstance(ours, nn.LSTMCell):
            (h1, c1), (h2, c2) = ours(_t(x), (_t(h), _t(c))), ref(x, (h, c))
            torch.testing.assert_close(torch.as_tensor(h1.detach().numpy()), h2.detach(), rtol=1e-5, atol=1e-5)
            torch.testing.assert_close(torch.as_tensor(c1.detach().numpy()), c2.detach(), rtol=1e-5, atol=1e-5)
        else:
            torch.testing.assert_close(torch.as_tensor(ours(_t(x), _t(h)).detach().numpy()), ref(x, h).detach(),
                                       rtol=1e-5, atol=1e-5)


def test_conv_variants_match_torch():
    torch.manual_seed(1)
    x3 = torch.randn(2, 3, 4, 5, 6)
    c3 = nn.Conv3d(3, 4, 3, pad_mode="pad", padding=1, has_bias=True)
    ref = torch.nn.functional.conv3d(x3, c3.weight.detach(), c3.bias.detach(), padding=1)
    torch.testing.assert_close(torch.as_tensor(c3(_t(x3)).detach().numpy()), torch.as_tensor(ref.numpy()), rtol=1e-4,
                               atol=1e-4)
    t1 = nn.Conv1dTranspose(3, 2, 4, stride=2, pad_mode="same")
    assert tuple(t1(_t(torch.randn(2, 3, 9))).shape) == (2, 2, 18)
    t3 = nn.Conv3dTranspose(3, 2, 3, stride=2, pad_mode="pad", padding=1, output_padding=1)
    ref = torch.nn.functional.conv_transpose3d(x3, t3.weight.detach(), None, 2, 1, 1)
    torch.testing.assert_close(torch.as_tensor(t3(_t(x3)).detach().numpy()), torch.as_tensor(ref.numpy()), rtol=1e-4,
                               atol=1e-4)
    u = nn.Unfold([1, 2, 2, 1], [1, 2, 2, 1], [1, 1, 1, 1])(_t(torch.arange(32.0).reshape(1, 2, 4, 4)))
    f = nn.Fold((4, 4), 2, stride=2)(u)
    assert torch.equal(torch.as_tensor(f.numpy()), torch.arange(32.0).reshape(1, 2, 4, 4))


def test_transformer_trains():
    ms.set_seed(3)
    model = nn.Transformer(d_model=16, nhead=4, num_encoder_layers=1, num_decoder_layers=1, dim_feedforward=32,
                           dropout=0.0, batch_first=True)
    src, tgt = _t(torch.randn(4, 6, 16)), _t(torch.randn(4, 5, 16))
    mask = _t(torch.triu(torch.ones(5, 5, dtype=torch.bool), 1))

    class Net(nn.Cell):
        def __init__(self):
            super().__init__()
            self.m = model

        def construct(self, s, t):
            return (self.m(s, t, tgt_mask=mask) ** 2).mean()
    net = Net()
    step = nn.TrainOneStepCell(net, nn.Adam(net.trainable_params(), 1e-2))
    step.set_train()
    first = float(step(src, tgt))
    for _ in range(20):
        last = float(step(src, tgt))
    assert last < first * 0.7


def test_multifield_embedding_sum_and_max():
    m = nn.MultiFieldEmbeddingLookup(6, 2, 2, param_init="ones", operator="SUM")
    out = m(_t(torch.tensor([[1, 2, 3]])), _t(torch.tensor([[1.0, 2.0, 3.0]])), _t(torch.tensor([[0, 0, 1]])))
    assert out.tolist() == [[[3.0, 3.0], [3.0, 3.0]]]
    m2 = nn.MultiFieldEmbeddingLookup(6, 2, 2, param_init="ones", operator="MAX")
    out = m2(_t(torch.tensor([[1, 2, 3]])), _t(torch.tensor([[1.0, 2.0, 3.0]])), _t(torch.tensor([[0, 0, -1]])))
    assert out.tolist() == [[[2.0, 2.0], [0.0, 0.0]]]


def _train(opt_fn, steps=5):
    ms.set_seed(7)
    net = nn.WithLossCell(nn.SequentialCell([nn.Dense(6, 8), nn.Tanh(), nn.Dense(8, 1)]), nn.MSELoss())
    g = torch.Generator().manual_seed(0)
    x, y = _t(torch.randn(32, 6, generator=g)), _t(torch.randn(32, 1, generator=g))
    step = nn.TrainOneStepCell(net, opt_fn(net))
    step.set_train()
    losses = [float(step(x, y)) for _ in range(steps)]
    return losses, [p.detach().numpy().copy() for p in net.trainable_params()]


def test_lazy_and_offload_adam_equal_adam_on_dense_gradients():
    ref_l, ref_p = _train(lambda n: nn.Adam(n.trainable_params(), 1e-2))
    for cls in (nn.LazyAdam, nn.AdamOffload):
        l, p = _train(lambda n: cls(n.trainable_params(), 1e-2))
        np.testing.assert_allclose(l, ref_l, rtol=1e-5)
        for a, b in zip(p, ref_p):
            np.testing.assert_allclose(a, b, rtol=1e-4, atol=1e-6)


def test_lazy_adam_touches_only_rows_with_gradient():
    emb = ms.Parameter(_t(torch.ones(16, 4)), name="emb")
    opt = nn.LazyAdam([emb], 0.1)
    g = torch.zeros(16, 4); g[3] = 1.0
    opt((_t(g),))
    w = emb.detach().numpy()
    assert (w[3] < 1).all() and (np.delete(w, 3, 0) == 1).all()
    assert float(opt.moment1[0].abs().sum()) == float(opt.moment1[0][3].abs().sum())


def test_thor_preconditions_dense_layers():
    losses, _ = _train(lambda n: nn.THOR(n, 0.05, 0.05, 0.9, frequency=2), steps=25)
    base, _ = _train(lambda n: nn.Momentum(n.trainable_params(), 0.05, 0.9), steps=25)
    assert losses[-1] < losses[0] * 0.7
    assert np.isfinite(losses).all() and losses[-1] < base[-1] * 1.5


def _adasum_rank(rank, world):
    import torch.distributed as dist
    import mindspore_b200 as ms
    from mindspore_b200 import nn
    from mindspore_b200.communication import init
    ms.set_context(device_target="CPU")
    init("gloo")
    p = ms.Parameter(ms.Tensor(torch.zeros(2)), name="w")
    opt = nn.AdaSumByGradWrapCell(nn.SGD([p], 1.0))
    grad = torch.tensor([1.0, 0.0]) if rank == 0 else torch.tensor([0.0, 1.0])
    opt((ms.Tensor(grad),))
    a = p.detach().numpy().tolist()
    p2 = ms.Parameter(ms.Tensor(torch.zeros(2)), name="w2")
    opt2 = nn.AdaSumByDeltaWeightWrapCell(nn.SGD([p2], 1.0))
    opt2((ms.Tensor(torch.tensor([2.0, 2.0])),))
    dist.barrier()
    return a, p2.detach().numpy().tolist()


def test_adasum_two_ranks():
    res = run_ranks(_adasum_rank, 2)
    for a, b in res:
        np.testing.assert_allclose(a, [-1.0, -1.0])          # orthogonal gradients add
        np.testing.assert_allclose(b, [-2.0, -2.0])          # identical deltas average


def test_simple_layers_match_torch_functional():
    import torch.nn.functional as F
    torch.manual_seed(0)
    x = torch.randn(2, 4, 6, 6)
    X = _t(x)

    def same(a, b):
        torch.testing.assert_close(torch.as_tensor(a.detach().numpy()), b, rtol=1e-5, atol=1e-6)
    same(nn.ReflectionPad2d(1)(X), F.pad(x, (1, 1, 1, 1), mode="reflect"))
    same(nn.ReplicationPad2d((1, 0, 2, 0))(X), F.pad(x, (1, 0, 2, 0), mode="replicate"))
    same(nn.ConstantPad2d(1, 3.0)(X), F.pad(x, (1, 1, 1, 1), value=3.0))
    same(nn.ZeroPad2d((1, 2, 0, 0))(X), F.pad(x, (1, 2, 0, 0)))
    x5 = torch.randn(1, 2, 4, 4, 4)
    same(nn.MaxPool3d(2)(_t(x5)), F.max_pool3d(x5, 2))
    same(nn.AvgPool3d(2, 2)(_t(x5)), F.avg_pool3d(x5, 2, 2))
    same(nn.AdaptiveAvgPool1d(3)(_t(x5[0, :, 0])), F.adaptive_avg_pool1d(x5[0, :, 0], 3))
    same(nn.Softmin()(X), F.softmin(x, -1))
    same(nn.Hardswish()(X), F.hardswish(x))
    same(nn.CELU(0.5)(X), F.celu(x, 0.5))
    same(nn.HShrink(0.3)(X), F.hardshrink(x, 0.3))
    same(nn.Roll(2, 1)(X), torch.roll(x, 2, 1))
    same(nn.Unflatten(1, (2, 2))(X), x.unflatten(1, (2, 2)))
    same(nn.Norm(axis=1)(X), x.norm(dim=1))
    same(nn.CosineSimilarity()(X, _t(x * 2)), F.cosine_similarity(x, x * 2))
    same(nn.LRN(2, 1.0, 1e-4, 0.75)(X), F.local_response_norm(x, 5, 5e-4, 0.75, 1.0))
    a, b = torch.randn(3, 5), torch.randn(3, 7)
    bd = nn.BiDense(5, 7, 4)
    same(bd(_t(a), _t(b)), F.bilinear(a, b, bd.weight.detach().as_subclass(torch.Tensor),
                                      bd.bias.detach().as_subclass(torch.Tensor)))
    assert abs(float(nn.ClipByNorm()(_t(torch.ones(4) * 3), 1.0).norm()) - 1.0) < 1e-6
    d = nn.Dropout2d(0.5)
    d.set_train(False)
    same(d(X), x)
    y, idx = F.max_pool2d(x, 2, return_indices=True)
    same(nn.MaxUnpool2d(2)(_t(y), _t(idx)), F.max_unpool2d(y, idx, 2))


def test_math_image_and_wrapper_cells():
    torch.manual_seed(0)
    a = torch.rand(2, 3, 32, 32)
    b = (a + 0.1 * torch.rand(2, 3, 32, 32)).clamp(0, 1)
    s_same, s_diff = nn.SSIM()(_t(a), _t(a)), nn.SSIM()(_t(a), _t(b))
    assert torch.allclose(s_same.as_subclass(torch.Tensor), torch.ones(2), atol=1e-6) and float(s_diff.max()) < 1.0
    assert float(nn.MSSSIM(power_factors=(0.5, 0.5), filter_size=5)(_t(a), _t(a)).min()) > 0.9999
    mse = ((a - b) ** 2).mean((1, 2, 3))
    torch.testing.assert_close(nn.PSNR()(_t(a), _t(b)).as_subclass(torch.Tensor), 10 * torch.log10(1 / mse))
    dy, dx = nn.ImageGradients()(_t(torch.arange(12.0).reshape(1, 1, 3, 4)))
    assert dy[0, 0, 0].tolist() == [4.0] * 4 and dy[0, 0, 2].tolist() == [0.0] * 4 and dx[0, 0, 0].tolist() == [1, 1, 1, 0]
    td = nn.TimeDistributed(nn.Dense(4, 2), 1)
    x = torch.randn(3, 5, 4)
    ref = torch.stack([td.layer(_t(x[:, i])).detach().as_subclass(torch.Tensor) for i in range(5)], 1)
    torch.testing.assert_close(td(_t(x)).detach().as_subclass(torch.Tensor), ref)
    assert nn.CentralCrop(0.5)(_t(a)).shape == (2, 3, 16, 16)
    m, v = nn.Moments(axis=0)(_t(a))
    torch.testing.assert_close(v.as_subclass(torch.Tensor), a.var(0, unbiased=False))
    assert nn.MatrixSetDiag()(_t(torch.ones(2, 2)), _t(torch.tensor([5., 6.]))).tolist() == [[5, 1], [1, 6]]
    p = ms.Parameter(_t(torch.tensor(0.1)), name="lr")
    nn.ParameterUpdate(p)(_t(torch.tensor(0.5)))
    assert float(p.detach()) == 0.5
    out, g = nn.Vjp(lambda t: t ** 2)(_t(torch.tensor([1., 2.])), _t(torch.ones(2)))
    assert out.tolist() == [1.0, 4.0] and torch.as_tensor(g[0] if isinstance(g, tuple) else g).tolist() == [2.0, 4.0]
    from mindspore_b200 import ops
    assert ops.argsort(_t(torch.tensor([3., 1., 2.]))).tolist() == [1, 2, 0]
    assert ops.cummax(_t(torch.tensor([1., 3., 2.])), 0)[0].tolist() == [1, 3, 3]
    assert sorted(ops.shuffle(_t(torch.arange(5)), seed=1).tolist()) == [0, 1, 2, 3, 4]


def test_cell_state_dict_scopes_and_hooks():
    ms.set_seed(0)
    net = nn.SequentialCell([nn.Dense(2, 3), nn.ReLU(), nn.Dense(3, 1)])
    other = nn.SequentialCell([nn.Dense(2, 3), nn.ReLU(), nn.Dense(3, 1)])
    sd = net.state_dict()
    assert list(sd) == ["0.weight", "0.bias", "2.weight", "2.bias"]
    assert other.load_state_dict({k: v.detach().clone() for k, v in sd.items()}) == ([], [])
    x = _t(torch.ones(1, 2))
    assert torch.equal(net(x), other(x))
    import pytest
    with pytest.raises(RuntimeError):
        other.load_state_dict({"0.weight": sd["0.weight"]})
    assert other.load_state_dict({"0.weight": sd["0.weight"]}, strict=False)[0] == ["0.bias", "2.weight", "2.bias"]
    net.generate_scope()
    assert net[0].get_scope() == "Default/0-Dense" and net[2].get_scope() == "Default/2-Dense"
    net.check_names()
    net.eval()
    assert not net.training and len(list(net.parameters())) == 4 and dict(net.named_parameters()).keys() == sd.keys()
    seen = []
    net[2].register_backward_pre_hook(lambda c, g: seen.append(tuple(g.shape)))
    net.train()
    net(x).sum().backward()
    assert seen == [(1, 1)]
    assert net.cast_inputs((x, 3), torch.bfloat16)[0].dtype == torch.bfloat16
    net.set_param_ps()
    assert all(p.is_param_ps for p in net.get_parameters())
