"""The fp16 builds of the sm_100a kernels (GEMM, norms, activations, RoPE, FlashAttention, convolution, BatchNorm)
against plain PyTorch fp32 references, and the reference-style fp16 + loss-scale recipe landing on them."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda"
H16 = torch.float16


@pytest.fixture(scope="module")
def K():
    from mindspore_b200 import _native
    from mindspore_b200.ops import kernels
    assert _native.cuda() is not None, "native CUDA library is not loaded"
    torch.manual_seed(0)
    return kernels


def _close(got, exp, tol=1e-2, abs_tol=1e-3):
    got, exp = got.float(), exp.float()
    err = (got - exp).abs().max().item()
    scale = exp.abs().max().item()
    assert err <= tol * scale + abs_tol, "max err %g vs scale %g" % (err, scale)


def _status_ok():
    from mindspore_b200 import _native
    torch.cuda.synchronize()
    assert _native.device_status() == 0


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, True)])
@pytest.mark.parametrize("shape", [(128, 128, 64), (200, 136, 72), (1024, 1536, 320), (2048, 4096, 4096)])
def test_gemm_fp16(K, a_mn, b_mn, shape):
    M, N, Kd = shape
    a = torch.randn((Kd, M) if a_mn else (M, Kd), device=DEV).half()
    b = torch.randn((Kd, N) if b_mn else (N, Kd), device=DEV).half()
    bias = torch.randn(N, device=DEV).half()
    A = a.float().t() if a_mn else a.float()
    B = b.float().t() if b_mn else b.float()
    ref = A @ B.t()
    before = K._native.launch_count
    c = K.gemm(a, b, a_mn=a_mn, b_mn=b_mn, bias=bias, alpha=0.5)
    assert c.dtype == H16 and K._native.launch_count == before + 1
    _close(c, 0.5 * ref + bias.float(), 2e-3)         # fp16 rounding of the output only: 10 mantissa bits
    acc = torch.ones(M, N, device=DEV)
    K.gemm(a, b, a_mn=a_mn, b_mn=b_mn, out=acc, accumulate=True)
    _close(acc, ref + 1, 1e-4)
    acc16 = torch.ones(M, N, device=DEV).half()
    K.gemm(a, b, a_mn=a_mn, b_mn=b_mn, out=acc16, accumulate=True)
    _close(acc16, ref + 1, 2e-3)
    _status_ok()


def test_norms_fp16(K):
    rows, H = 512, 4096
    x, res, dy, dres = (torch.randn(rows, H, device=DEV).half() for _ in range(4))
    w = (1 + 0.1 * torch.randn(H, device=DEV)).half()
    y, rstd, xs = K.rmsnorm_fwd(x, w, 1e-5, residual=res)
    assert y.dtype == H16
    xf = (x.float() + res.float()).half().float()
    r = torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-5)
    _close(y, xf * r * w.float(), 2e-3)
    _close(xs, xf, 1e-3)
    xl, wl = xf.clone().requires_grad_(True), w.float().clone().requires_grad_(True)
    (xl * torch.rsqrt(xl.pow(2).mean(-1, keepdim=True) + 1e-5) * wl).backward(dy.float())
    dx, dw = K.rmsnorm_bwd(dy, xs, w, rstd, dresidual=dres)
    _close(dx, xl.grad + dres.float(), 2e-3)
    _close(dw, wl.grad, 2e-3)
    b = torch.randn(H, device=DEV).half()
    y, mean, rs = K.layernorm_fwd(x, w, b, 1e-5)
    xl, wl, bl = (t.float().clone().requires_grad_(True) for t in (x, w, b))
    yl = torch.nn.functional.layer_norm(xl, (H,), wl, bl, 1e-5)
    _close(y, yl, 2e-3)
    yl.backward(dy.float())
    dx, dw, db = K.layernorm_bwd(dy, x, w, mean, rs)
    _close(dx, xl.grad, 2e-3)
    _close(dw, wl.grad, 2e-3)
    _close(db, bl.grad, 2e-3)
    _status_ok()


def test_activations_rope_fp16(K):
    rows, F = 256, 2752
    gu = torch.randn(rows, 2 * F, device=DEV).half()
    gl = gu.float().clone().requires_grad_(True)
    ol = torch.nn.functional.silu(gl[:, :F]) * gl[:, F:]
    _close(K.swiglu_fwd(gu), ol, 2e-3)
    do = torch.randn(rows, F, device=DEV).half()
    ol.backward(do.float())
    _close(K.swiglu_bwd(gu, do), gl.grad, 2e-3)
    xg, bg, dg = torch.randn(rows, 1024, device=DEV).half(), torch.randn(1024, device=DEV).half(), \
        torch.randn(rows, 1024, device=DEV).half()
    xl = (xg.float() + bg.float()).requires_grad_(True)
    yl = torch.nn.functional.gelu(xl, approximate="tanh")
    _close(K.gelu_fwd(xg, bg), yl, 2e-3)
    yl.backward(dg.float())
    _close(K.gelu_bwd(xg, dg, bg), xl.grad, 2e-3)
    S, nh, D = 256, 8, 128
    q = torch.randn(2 * S, nh * D, device=DEV).half()
    inv = 1.0 / (10000 ** (torch.arange(0, D, 2, device=DEV).float() / D))
    fr = torch.outer(torch.arange(S, device=DEV).float(), inv)
    cos, sin = fr.cos().contiguous(), fr.sin().contiguous()
    qf = q.float().view(2, S, nh, D)
    c, s = cos[None, :, None, :], sin[None, :, None, :]
    a, b = qf[..., :D // 2], qf[..., D // 2:]
    ref = torch.cat([a * c - b * s, b * c + a * s], -1).view(2 * S, nh * D)
    q2 = q.clone()
    K.rope_(q2, cos, sin, nh, D, S)
    _close(q2, ref, 2e-3)
    _status_ok()


@pytest.mark.parametrize("B,S,H,causal", [(1, 256, 2, False), (2, 512, 4, True)])
def test_flash_attention_fp16(K, B, S, H, causal):
    from mindspore_b200.ops import flash_attn_kernel as FK
    from mindspore_b200.ops.attention import reference_attention
    D = 128
    q, k, v, do = (torch.randn(B, S, H, D, device=DEV).half() for _ in range(4))
    assert FK.supports(q, k, v)
    sc = 1 / math.sqrt(D)
    o, lse, q2, k2, v2 = FK.fwd(q, k, v, causal, sc)
    assert o.dtype == H16
    dq, dk, dv = FK.bwd(do, q2, k2, v2, o, lse, causal, sc)
    qf, kf, vf = (t.float().detach().requires_grad_(True) for t in (q, k, v))
    ref = reference_attention(qf, kf, vf, causal)
    ref.backward(do.float())
    _close(o, ref, 5e-3)
    _close(dq, qf.grad, 1e-2)
    _close(dk, kf.grad, 1e-2)
    _close(dv, vf.grad, 1e-2)
    _status_ok()


@pytest.mark.parametrize("relu", [False, True])
def test_conv_bn_relu_fp16(K, relu):
    from mindspore_b200.ops import conv_kernel as CK
    n, cin, cout, h = 8, 64, 128, 28
    x = torch.randn(n, cin, h, h, device=DEV).half().contiguous(memory_format=torch.channels_last)
    w = (torch.randn(cout, cin, 3, 3, device=DEV) * 0.05).half()
    gamma, beta = torch.rand(cout, device=DEV) + 0.5, torch.randn(cout, device=DEV) * 0.1
    mm, mv = torch.zeros(cout, device=DEV), torch.ones(cout, device=DEV)
    xg, wg = x.clone().requires_grad_(True), w.clone().requires_grad_(True)
    gg, bg = gamma.clone().requires_grad_(True), beta.clone().requires_grad_(True)
    assert CK.supports(xg, wg)
    before = K._native.launch_count
    y = CK.conv_bn_act(xg, wg, gg, bg, mm, mv, stride=1, pad=1, relu=relu)
    assert y.dtype == H16 and K._native.launch_count > before
    dy = torch.randn_like(y)
    y.backward(dy)
    xr, wr = x.float().clone().requires_grad_(True), w.float().clone().requires_grad_(True)
    gr, br = gamma.clone().requires_grad_(True), beta.clone().requires_grad_(True)
    yr = torch.nn.functional.batch_norm(torch.nn.functional.conv2d(xr, wr, None, 1, 1), None, None, gr, br, True, 0.1,
                                        1e-5)
    if relu:
        yr = torch.relu(yr)
    yr.backward(dy.float())
    _close(y, yr, 1e-2)
    # with the ReLU, outputs next to zero fall on the other side of the mask in fp16 than in the fp32 reference:
    # single gradient elements then differ by a whole term, whatever the precision of the rest
    tol = 6e-2 if relu else 2e-2
    _close(xg.grad, xr.grad, tol)
    _close(wg.grad, wr.grad, tol)
    _close(gg.grad, gr.grad, tol)
    _close(bg.grad, br.grad, tol)
    _status_ok()


def test_fp16_loss_scale_recipe_runs_on_the_kernels():
    """The reference's mixed-precision recipe (fp16 compute, fp32 parameters, dynamic loss scale): Dense / LayerNorm /
    GELU of an fp16 network launch the fp16 kernel builds, the loss falls, and no step overflows."""
    import mindspore_b200 as ms
    from mindspore_b200 import _native, nn, ops
    ms.set_context(mode=ms.PYNATIVE_MODE, device_target="GPU")
    ms.set_seed(0)

    class Net(nn.Cell):
        def __init__(self):
            super().__init__()
            self.fc1, self.fc2 = nn.Dense(256, 1024), nn.Dense(1024, 16)
            self.norm, self.act = nn.LayerNorm((1024,)), nn.GELU()

        def construct(self, x):
            return self.fc2(self.act(self.norm(self.fc1(x))))

    net = Net().to_float(ms.float16)
    loss_fn = nn.SoftmaxCrossEntropyWithLogits(sparse=True, reduction="mean")
    opt = nn.Momentum(net.trainable_params(), learning_rate=0.05, momentum=0.9)
    step = nn.TrainOneStepWithLossScaleCell(nn.WithLossCell(net, loss_fn), opt,
                                            nn.DynamicLossScaleUpdateCell(2.0 ** 10, 2.0, 100))
    step.set_train()
    g = torch.Generator().manual_seed(1)
    x = ms.Tensor(torch.randn(512, 256, generator=g).cuda())
    y = ms.Tensor(torch.randint(0, 16, (512,), generator=g).cuda())
    before = _native.launch_count
    losses = []
    for _ in range(12):
        loss, overflow, _scale = step(x, y)
        assert not bool(overflow)
        losses.append(float(loss))
    assert _native.launch_count - before >= 12 * 6, "the fp16 network did not run on the native kernels"
    assert losses[-1] < 0.7 * losses[0], losses
    torch.cuda.synchronize()
    assert _native.device_status() == 0
