"""hypercomplex layers against complex arithmetic / the defining algebra."""
import numpy as np
import pytest
import torch

import mindspore_b200 as ms
from mindspore_b200 import hypercomplex as hc
from mindspore_b200.hypercomplex.utils import get_x_and_y, to_2channel


def test_complex_dense_and_conv_match_complex_arithmetic():
    ms.set_seed(0)
    d = hc.complex.Dense(6, 4)
    with torch.no_grad():
        for p in d.get_parameters():
            p.copy_(torch.randn(p.shape))
    xr, xi = torch.randn(5, 6), torch.randn(5, 6)
    yr, yi = get_x_and_y(d(to_2channel(xr, xi)))
    t = lambda p: p.detach().as_subclass(torch.Tensor)
    w = torch.complex(t(d.weight_x), t(d.weight_y))
    ref = torch.complex(xr, xi) @ w.t() + torch.complex(t(d.bias_x), t(d.bias_y))
    np.testing.assert_allclose(yr.detach().numpy(), ref.real.numpy(), rtol=1e-4, atol=1e-5)
    np.testing.assert_allclose(yi.detach().numpy(), ref.imag.numpy(), rtol=1e-4, atol=1e-5)
    c = hc.complex.Conv2d(3, 5, 3, stride=2, pad_mode="same", has_bias=True)
    x = torch.randn(2, 2, 3, 9, 9)
    out = c(ms.Tensor(x)).detach().as_subclass(torch.Tensor)
    assert out.shape == (2, 2, 5, 5, 5)
    # (a + ib)(c + id): real part = conv(xr, wx) - conv(xi, wy)
    wx, wy = t(c.weight_x), t(c.weight_y)
    pad = torch.nn.functional.pad
    conv = lambda a, k: torch.nn.functional.conv2d(pad(a, [1, 1, 1, 1]), k, None, 2)
    real = conv(x[0], wx) - conv(x[1], wy) + t(c.bias_x).reshape(1, -1, 1, 1)
    np.testing.assert_allclose(out[0].numpy(), real.numpy(), rtol=1e-4, atol=1e-4)
    out.sum()
    loss = c(ms.Tensor(x)).sum()
    loss.backward()
    assert c.weight_y.grad is not None


def test_dual_and_double_algebras():
    ms.set_seed(1)
    xr, xi = torch.randn(3, 4), torch.randn(3, 4)
    for mod, sq in ((hc.dual, 0.0), (hc.double, 1.0)):
        d = mod.Dense(4, 2, has_bias=False)
        with torch.no_grad():
            for p in d.get_parameters():
                p.copy_(torch.randn(p.shape))
        wx, wy = (p.detach().as_subclass(torch.Tensor) for p in (d.weight_x, d.weight_y))
        yr, yi = get_x_and_y(d(to_2channel(xr, xi)))
        np.testing.assert_allclose(yr.detach().numpy(), (xr @ wx.t() + sq * xi @ wy.t()).numpy(), rtol=1e-4, atol=1e-5)
        np.testing.assert_allclose(yi.detach().numpy(), (xr @ wy.t() + xi @ wx.t()).numpy(), rtol=1e-4, atol=1e-5)


def test_norm_pool_relu_and_shape_checks():
    x = ms.Tensor(torch.randn(2, 4, 3, 8, 8))
    bn = hc.complex.BatchNorm2d(3)
    bn.set_train()
    y = bn(x).detach().as_subclass(torch.Tensor)
    assert y.shape == x.shape and abs(float(y[0].mean())) < 1e-4 and abs(float(y[1].var()) - 1) < 0.05
    assert hc.complex.AvgPool2d(kernel_size=2, stride=2)(x).shape == (2, 4, 3, 4, 4)
    assert hc.dual.AdaptiveAvgPool2d(1)(x).shape == (2, 4, 3, 1, 1)
    assert float(hc.double.ReLU()(x).min()) >= 0
    with pytest.raises(ValueError):
        hc.complex.Dense(4, 2)(ms.Tensor(torch.randn(3, 4)))
    with pytest.raises(ValueError):
        to_2channel(torch.zeros(2), torch.zeros(3))
