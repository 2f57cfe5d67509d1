"""Implicit-GEMM convolution, fused BatchNorm / ReLU and pooling kernels against PyTorch fp32 references."""
import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def CK():
    from mindspore_b200 import _native
    from mindspore_b200.ops import conv_kernel
    assert _native.cuda() is not None and conv_kernel.available()
    torch.manual_seed(0)
    return conv_kernel


def _close(got, exp, tol=2e-2):
    got, exp = got.float(), exp.float()
    err = (got - exp).abs().max().item()
    scale = exp.abs().max().item()
    assert err <= tol * scale + 1e-3, "max err %g vs scale %g" % (err, scale)


def _status_ok():
    from mindspore_b200 import _native
    torch.cuda.synchronize()
    assert _native.device_status() == 0


CASES = [  # N, Cin, H, W, Cout, k, stride
    (4, 64, 56, 56, 64, 3, 1), (4, 64, 56, 56, 256, 1, 1), (2, 128, 28, 28, 128, 3, 2), (2, 256, 56, 56, 512, 1, 2),
    (8, 512, 7, 7, 512, 3, 1), (3, 64, 30, 22, 72, 3, 1), (2, 256, 14, 14, 1024, 1, 1), (2, 3, 64, 64, 64, 7, 2),
]


@pytest.mark.parametrize("N,Cin,H,W,Cout,k,stride", CASES)
def test_conv_forward_and_gradients(CK, N, Cin, H, W, Cout, k, stride):
    x = torch.randn(N, Cin, H, W, device="cuda").bfloat16().requires_grad_(Cin >= 64)
    w = (torch.randn(Cout, Cin, k, k, device="cuda") / (Cin * k * k) ** 0.5).bfloat16().requires_grad_(True)
    pad = k // 2
    y, stats = CK._ConvFn.apply(x, w, stride, pad, pad, True)
    xr, wr = x.detach().float().requires_grad_(True), w.detach().float().requires_grad_(True)
    yr = F.conv2d(xr, wr, None, stride, pad)
    _close(y, yr)
    yb = y.detach().float()
    _close(stats[:Cout], yb.sum((0, 2, 3)), 1e-2)
    _close(stats[Cout:], (yb * yb).sum((0, 2, 3)), 1e-2)
    dy = torch.randn_like(yr).bfloat16()
    y.backward(dy)
    yr.backward(dy.float())
    _close(w.grad, wr.grad, 3e-2)
    if Cin >= 64:
        _close(x.grad, xr.grad, 3e-2)
    _status_ok()


@pytest.mark.parametrize("relu,res", [(True, False), (True, True), (False, False)])
def test_conv_bn_act_unit(CK, relu, res):
    N, Cin, H, W, Cout = 4, 64, 28, 28, 128
    x = torch.randn(N, Cin, H, W, device="cuda").bfloat16().requires_grad_(True)
    w = (torch.randn(Cout, Cin, 3, 3, device="cuda") / 24).bfloat16().requires_grad_(True)
    gamma = (1 + 0.1 * torch.randn(Cout, device="cuda")).requires_grad_(True)
    beta = (0.1 * torch.randn(Cout, device="cuda")).requires_grad_(True)
    r = torch.randn(N, Cout, H, W, device="cuda").bfloat16().requires_grad_(True) if res else None
    mm, mv = torch.zeros(Cout, device="cuda"), torch.ones(Cout, device="cuda")
    y = CK.conv_bn_act(x, w, gamma, beta, mm, mv, 1, 1, relu, r, 1e-5, 0.9)
    leaves = [t.detach().float().requires_grad_(True) for t in (x, w, gamma, beta)]
    rr = r.detach().float().requires_grad_(True) if res else None
    mm2, mv2 = torch.zeros(Cout, device="cuda"), torch.ones(Cout, device="cuda")
    c = F.conv2d(leaves[0], leaves[1], None, 1, 1).bfloat16().float()      # the kernel normalises the stored bf16
    yr = F.batch_norm(c, mm2, mv2, leaves[2], leaves[3], True, 0.1, 1e-5)
    if res:
        yr = yr + rr
    if relu:
        yr = torch.relu(yr)
    _close(y, yr, 3e-2)
    _close(mm, mm2, 2e-2)
    _close(mv, mv2, 2e-2)
    dy = torch.randn_like(yr).bfloat16()
    y.backward(dy)
    yr.backward(dy.float())
    _close(gamma.grad, leaves[2].grad, 3e-2)
    _close(beta.grad, leaves[3].grad, 3e-2)
    _close(w.grad, leaves[1].grad, 5e-2)
    _close(x.grad, leaves[0].grad, 5e-2)
    if res:
        _close(r.grad, rr.grad, 2e-2)
    _status_ok()


def test_pooling(CK):
    x = torch.randn(4, 64, 30, 26, device="cuda").bfloat16().requires_grad_(True)
    y = CK.maxpool3x3s2(x)
    xr = x.detach().float().requires_grad_(True)
    yr = F.max_pool2d(xr, 3, 2, 1)
    _close(y, yr, 1e-3)
    dy = torch.randn_like(yr).bfloat16()
    y.backward(dy)
    yr.backward(dy.float())
    _close(x.grad, xr.grad, 1e-2)
    z = torch.randn(8, 256, 7, 7, device="cuda").bfloat16().requires_grad_(True)
    a = CK.global_avgpool(z)
    zr = z.detach().float().requires_grad_(True)
    ar = zr.mean((2, 3))
    _close(a, ar, 1e-2)
    da = torch.randn_like(ar).bfloat16()
    a.backward(da)
    ar.backward(da.float())
    _close(z.grad, zr.grad, 1e-2)
    _status_ok()


def test_resnet50_train_step_runs_on_kernels():
    import mindspore_b200 as ms
    from mindspore_b200 import _native, nn
    from mindspore_b200.models.resnet import ResNetWithLoss, resnet50
    ms.set_context(device_target="GPU")
    ms.set_seed(0)
    net = ResNetWithLoss(resnet50(1000, dtype=torch.bfloat16))
    opt = nn.Momentum(net.trainable_params(), 0.05, 0.9)
    step = nn.TrainOneStepCell(net, opt)
    step.set_train()
    x = torch.randn(8, 3, 224, 224, device="cuda").bfloat16()
    y = torch.randint(0, 1000, (8,), device="cuda")
    before = _native.launch_count
    losses = [float(step(ms.Tensor(x), ms.Tensor(y))) for _ in range(4)]
    assert _native.launch_count - before > 4 * 300          # convolutions, BN and pooling ran as our kernels
    assert all(l == l for l in losses) and losses[-1] < losses[0]
    _status_ok()
