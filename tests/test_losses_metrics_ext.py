"""Further losses against torch.nn.functional and further metrics against hand-computed values."""
import numpy as np
import torch
import torch.nn.functional as F

import mindspore_b200 as ms
import mindspore_b200.train.metrics as M
from mindspore_b200 import nn


def T(x):
    return ms.Tensor(x)


def test_losses_match_torch():
    g = torch.Generator().manual_seed(0)
    x, y = torch.randn(6, 5, generator=g), torch.randint(0, 5, (6,), generator=g)
    assert abs(float(nn.MultiMarginLoss()(T(x), T(y))) - float(F.multi_margin_loss(x, y))) < 1e-6
    sign = torch.where(torch.rand(6, 5, generator=g) > 0.5, 1.0, -1.0)
    assert abs(float(nn.SoftMarginLoss()(T(x), T(sign))) - float(F.soft_margin_loss(x, sign))) < 1e-6
    assert abs(float(nn.HingeEmbeddingLoss(0.7)(T(x), T(sign))) - float(F.hinge_embedding_loss(x, sign, 0.7))) < 1e-6
    t01 = (sign > 0).float()
    assert abs(float(nn.MultiLabelSoftMarginLoss()(T(x), T(t01))) - float(F.multilabel_soft_margin_loss(x, t01))) < 1e-6
    tgt = torch.rand(6, 5, generator=g) * 3
    assert abs(float(nn.PoissonNLLLoss()(T(x), T(tgt))) - float(F.poisson_nll_loss(x, tgt))) < 1e-6
    var = torch.rand(6, 5, generator=g) + 0.1
    assert abs(float(nn.GaussianNLLLoss()(T(x), T(tgt), T(var))) - float(F.gaussian_nll_loss(x, tgt, var))) < 1e-6
    ml = torch.tensor([[3, 0, -1, 1, 2], [1, 2, -1, 0, 0]])
    assert abs(float(nn.MultilabelMarginLoss()(T(x[:2]), T(ml))) - float(F.multilabel_margin_loss(x[:2], ml))) < 1e-6
    onehot = F.one_hot(y, 5).float().reshape(6, 5, 1)
    d = float(nn.MultiClassDiceLoss()(T(x.reshape(6, 5, 1)), T(onehot)))
    assert 0 < d < 1


def test_sampled_softmax_equals_full_softmax_when_all_classes_are_sampled():
    g = torch.Generator().manual_seed(1)
    C, D, B = 7, 4, 5
    w, b = torch.randn(C, D, generator=g), torch.randn(C, generator=g)
    h, y = torch.randn(B, D, generator=g), torch.randint(0, C, (B,), generator=g)
    loss = nn.SampledSoftmaxLoss(num_sampled=C, num_classes=C, sampled_values=(torch.arange(C), None, None))
    got = loss(T(w), T(b), T(y), T(h))
    ref = F.cross_entropy(h @ w.t() + b, y, reduction="none")     # accidental hits are masked, so each class counts once
    torch.testing.assert_close(torch.as_tensor(got.numpy()), ref, rtol=1e-4, atol=1e-4)


def test_metrics():
    r = M.ROC(pos_label=1)
    r.update(np.array([0.1, 0.4, 0.35, 0.8]), np.array([0, 0, 1, 1]))
    fpr, tpr, thr = r.eval()
    assert fpr.tolist() == [0, 0, 0.5, 0.5, 1] and tpr.tolist() == [0, 0.5, 0.5, 1, 1] and M.auc(fpr, tpr) == 0.75
    b = M.BleuScore()
    b.update([["the", "cat", "sat", "on", "the", "mat"]], [[["the", "cat", "sat", "on", "a", "mat"]]])
    assert 0.4 < b.eval() < 0.6
    b.clear()
    b.update([["a", "b", "c", "d"]], [[["a", "b", "c", "d"]]])
    assert abs(b.eval() - 1.0) < 1e-12
    a = np.zeros((8, 8)); a[2:5, 2:5] = 1
    c = np.zeros((8, 8)); c[3:6, 3:6] = 1
    h = M.HausdorffDistance(); h.update(a, c, 1)
    assert abs(h.eval() - 2 ** 0.5) < 1e-9
    m = M.MeanSurfaceDistance(symmetric=True); m.update(a, c, 1)
    assert 0 < m.eval() < 2 ** 0.5
    cs = M.CosineSimilarity(); cs.update(np.array([[1.0, 0], [0, 1.0], [1.0, 1.0]]))
    s = cs.eval()
    assert abs(s[0, 2] - 2 ** -0.5) < 1e-9 and s[0, 1] == 0 and s[0, 0] == 0
    cm = M.ConfusionMatrixMetric(skip_channel=False, metric_name="f1 score", calculation_method=True)
    cm.update(np.array([[[1, 1, 0, 0]]]), np.array([[[1, 0, 1, 0]]]))
    assert abs(cm.eval() - 0.5) < 1e-9
    net = lambda x: torch.stack([x[:, :, :2].sum((1, 2, 3)), x.sum((1, 2, 3))], 1)      # class 0 looks at the top rows
    oc = M.OcclusionSensitivity(margin=0)
    oc.update(net, torch.ones(1, 1, 4, 4), np.array([0]))
    mp = oc.eval()
    assert mp[:2].min() == 1 and mp[2:].max() == 0
    assert isinstance(M.get_metric_fn("roc", pos_label=1), M.ROC)
