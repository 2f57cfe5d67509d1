"""Numerics of the sm_100a kernels against plain PyTorch fp32 references of the same operation.

Every test fails if the native CUDA library is not loaded (no silent eager fallback) and checks the per-device
status word, which the kernels set when one of their bounded waits gives up."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda"


@pytest.fixture(scope="module")
def K():
    from mindspore_b200 import _native
    from mindspore_b200.ops import kernels
    assert _native.cuda() is not None, "native CUDA library is not loaded"
    torch.manual_seed(0)
    return kernels


def _close(got, exp, tol=2e-2, abs_tol=1e-3):
    got, exp = got.float(), exp.float()
    err = (got - exp).abs().max().item()
    scale = exp.abs().max().item()
    assert err <= tol * scale + abs_tol, "max err %g vs scale %g" % (err, scale)


def _status_ok():
    from mindspore_b200 import _native
    torch.cuda.synchronize()
    assert _native.device_status() == 0


def _gemm_ref(a, b, a_mn, b_mn):
    A = a.float().transpose(-1, -2) if a_mn else a.float()
    B = b.float().transpose(-1, -2) if b_mn else b.float()
    return A @ B.transpose(-1, -2)


@pytest.mark.parametrize("a_mn", [False, True])
@pytest.mark.parametrize("b_mn", [False, True])
@pytest.mark.parametrize("bn", [128, 256])
@pytest.mark.parametrize("shape", [(128, 128, 64), (256, 512, 512), (200, 136, 72), (1024, 1536, 320)])
def test_gemm_layouts(K, a_mn, b_mn, bn, shape):
    M, N, Kd = shape
    a = torch.randn((Kd, M) if a_mn else (M, Kd), device=DEV).bfloat16()
    b = torch.randn((Kd, N) if b_mn else (N, Kd), device=DEV).bfloat16()
    c = K.gemm(a, b, a_mn=a_mn, b_mn=b_mn, bn_hint=bn)
    _close(c, _gemm_ref(a, b, a_mn, b_mn))
    _status_ok()


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, True)])
def test_gemm_cta_pair(K, a_mn, b_mn):
    """Problems of at least 64 tiles of 256 x 256 go to the CTA-pair kernel (tcgen05.mma.cta_group::2); ragged M / N
    edges, a bias, fp32 accumulation into an existing output."""
    assert K._PAIR_GEMM, "the CTA-pair GEMM is expected to be on by default"
    M, N, Kd = 2048 + 72, 2048 + 136, 448
    a = torch.randn((Kd, M) if a_mn else (M, Kd), device=DEV).bfloat16()
    b = torch.randn((Kd, N) if b_mn else (N, Kd), device=DEV).bfloat16()
    bias = torch.randn(N, device=DEV).bfloat16()
    ref = _gemm_ref(a, b, a_mn, b_mn)
    assert K._pair_gemm_ok(M, N, Kd, 1, torch.empty(M, N, device=DEV, dtype=torch.bfloat16),
                           torch.empty(M, N, device=DEV, dtype=torch.bfloat16), False, 0)
    _close(K.gemm(a, b, a_mn=a_mn, b_mn=b_mn, bias=bias), ref + bias.float())
    out = torch.randn(M, N, device=DEV)
    exp = out + 0.5 * ref
    _close(K.gemm(a, b, a_mn=a_mn, b_mn=b_mn, out=out, out_dtype=torch.float32, accumulate=True, alpha=0.5), exp)
    _status_ok()


def test_gemm_batched_accumulate_bias(K):
    a = torch.randn(3, 256, 192, device=DEV).bfloat16()
    b = torch.randn(3, 384, 192, device=DEV).bfloat16()
    _close(K.gemm(a, b), _gemm_ref(a, b, False, False))
    at = torch.randn(3, 192, 256, device=DEV).bfloat16()
    bt = torch.randn(3, 192, 384, device=DEV).bfloat16()
    out = torch.randn(3, 256, 384, device=DEV)
    exp = out + _gemm_ref(at, bt, True, True)
    got = K.gemm(at, bt, a_mn=True, b_mn=True, out=out, out_dtype=torch.float32, accumulate=True)
    _close(got, exp)
    a2 = torch.randn(512, 256, device=DEV).bfloat16()
    b2 = torch.randn(256, 1024, device=DEV).bfloat16()
    bias = torch.randn(1024, device=DEV).bfloat16()
    out2 = torch.randn(512, 1024, device=DEV).bfloat16()
    exp2 = out2.float() + _gemm_ref(a2, b2, False, True) + bias.float()
    got2 = K.gemm(a2, b2, b_mn=True, out=out2, accumulate=True, bias=bias)
    _close(got2, exp2)
    _status_ok()


def test_linear_fwd_dgrad_wgrad(K):
    x = torch.randn(384, 512, device=DEV).bfloat16()
    w = torch.randn(768, 512, device=DEV).bfloat16()
    dy = torch.randn(384, 768, device=DEV).bfloat16()
    _close(K.linear_fwd(x, w), x.float() @ w.float().t())
    _close(K.linear_dgrad(dy, w), dy.float() @ w.float())
    main_grad = torch.ones(768, 512, device=DEV)
    K.linear_wgrad(dy, x, out=main_grad, accumulate=True)
    _close(main_grad, 1 + dy.float().t() @ x.float())
    _status_ok()


def test_rmsnorm_fwd_bwd(K):
    rows, H = 512, 4096
    x = torch.randn(rows, H, device=DEV).bfloat16()
    res = torch.randn(rows, H, device=DEV).bfloat16()
    w = (1 + 0.1 * torch.randn(H, device=DEV)).bfloat16()
    y, rstd, xs = K.rmsnorm_fwd(x, w, 1e-5, residual=res)
    xf = (x.float() + res.float()).bfloat16().float()
    r = torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-5)
    _close(y, xf * r * w.float())
    _close(rstd, r.flatten(), 1e-3)
    _close(xs, xf)
    dy = torch.randn(rows, H, device=DEV).bfloat16()
    dres = torch.randn(rows, H, device=DEV).bfloat16()
    xl = xf.clone().requires_grad_(True)
    wl = w.float().clone().requires_grad_(True)
    (xl * torch.rsqrt(xl.pow(2).mean(-1, keepdim=True) + 1e-5) * wl).backward(dy.float())
    dx, dw = K.rmsnorm_bwd(dy, xs, w, rstd, dresidual=dres)
    _close(dx, xl.grad + dres.float())
    _close(dw, wl.grad)
    dwf = torch.ones(H, device=DEV)
    K.rmsnorm_bwd(dy, xs, w, rstd, dw_out=dwf, accumulate=True)
    _close(dwf, wl.grad + 1)
    _status_ok()


def test_layernorm_fwd_bwd(K):
    rows, H = 300, 1024
    x = torch.randn(rows, H, device=DEV).bfloat16()
    w = (1 + 0.1 * torch.randn(H, device=DEV)).bfloat16()
    b = torch.randn(H, device=DEV).bfloat16()
    dy = torch.randn(rows, H, device=DEV).bfloat16()
    y, mean, rs = K.layernorm_fwd(x, w, b, 1e-5)
    xl, wl, bl = (t.float().clone().requires_grad_(True) for t in (x, w, b))
    yl = torch.nn.functional.layer_norm(xl, (H,), wl, bl, 1e-5)
    _close(y, yl)
    yl.backward(dy.float())
    dx, dw, db = K.layernorm_bwd(dy, x, w, mean, rs)
    _close(dx, xl.grad)
    _close(dw, wl.grad)
    _close(db, bl.grad)
    _status_ok()


def test_swiglu_gelu(K):
    rows, F = 256, 2752
    gu = torch.randn(rows, 2 * F, device=DEV).bfloat16()
    gl = gu.float().clone().requires_grad_(True)
    ol = torch.nn.functional.silu(gl[:, :F]) * gl[:, F:]
    _close(K.swiglu_fwd(gu), ol)
    do = torch.randn(rows, F, device=DEV).bfloat16()
    ol.backward(do.float())
    _close(K.swiglu_bwd(gu, do), gl.grad)
    xg = torch.randn(rows, 1024, device=DEV).bfloat16()
    bg = torch.randn(1024, device=DEV).bfloat16()
    xl = (xg.float() + bg.float()).requires_grad_(True)
    yl = torch.nn.functional.gelu(xl, approximate="tanh")
    _close(K.gelu_fwd(xg, bg), yl)
    dg = torch.randn(rows, 1024, device=DEV).bfloat16()
    yl.backward(dg.float())
    _close(K.gelu_bwd(xg, dg, bg), xl.grad)
    _status_ok()


def test_rope(K):
    S, nh, D = 256, 8, 128
    q = torch.randn(2 * S, nh * D, device=DEV).bfloat16()
    inv = 1.0 / (10000 ** (torch.arange(0, D, 2, device=DEV).float() / D))
    fr = torch.outer(torch.arange(S, device=DEV).float(), inv)
    cos, sin = fr.cos().contiguous(), fr.sin().contiguous()
    qf = q.float().view(2, S, nh, D)
    c, s = cos[None, :, None, :], sin[None, :, None, :]
    a, b = qf[..., :D // 2], qf[..., D // 2:]
    ref = torch.cat([a * c - b * s, b * c + a * s], -1).view(2 * S, nh * D)
    q2 = q.clone()
    K.rope_(q2, cos, sin, nh, D, S)
    _close(q2, ref)
    K.rope_(q2, cos, sin, nh, D, S, backward=True)
    _close(q2, q, 3e-2)
    _status_ok()


def test_cross_entropy(K):
    V = 32000
    lg = (torch.randn(64, V, device=DEV) * 3).bfloat16()
    lab = torch.randint(0, V, (64,), device=DEV, dtype=torch.int32)
    lab[3] = -100
    st = K.ce_stats(lg, lab)
    gs = torch.tensor([0.5], device=DEV)
    loss, dl = K.ce_loss_grad(lg, lab, st, gs)
    ll = lg.float().clone().requires_grad_(True)
    lr = torch.nn.functional.cross_entropy(ll, lab.long(), ignore_index=-100, reduction="none")
    _close(loss, lr, 1e-3)
    (lr.sum() * 0.5).backward()
    _close(dl, ll.grad)
    _status_ok()


def test_adamw_and_grad_norm(K):
    n = 1000003
    p = torch.randn(n, device=DEV)
    g = torch.randn(n, device=DEV)
    m, v = torch.zeros(n, device=DEV), torch.zeros(n, device=DEV)
    plp = torch.empty(n, device=DEV, dtype=torch.bfloat16)
    lr, b1, b2, eps, wd = 1e-3, 0.9, 0.95, 1e-8, 0.1
    hy = torch.tensor([lr, b1, b2, eps, wd, 1 - b1, 1 - b2, 1.0], device=DEV)
    ref = p * (1 - lr * wd) - lr * g / (g.abs() + eps)
    K.adamw_step(p, m, v, g, plp, hy)
    _close(p, ref, 1e-4)
    _close(plp, ref, 1e-2)
    _close(m, (1 - b1) * g, 1e-5)
    out = torch.zeros(1, device=DEV)
    nf = torch.zeros(1, device=DEV, dtype=torch.int32)
    K.sumsq_finite(g, out, nf)
    _close(out, g.pow(2).sum().view(1), 1e-3)
    assert nf.item() == 0
    g[5] = float("inf")
    K.sumsq_finite(g, out, nf)
    assert nf.item() != 0
    _status_ok()


def test_embedding(K):
    tab = torch.randn(1000, 512, device=DEV).bfloat16()
    ids = torch.randint(0, 1000, (4, 64), device=DEV, dtype=torch.int32)
    _close(K.embedding_fwd(tab, ids), tab[ids.long()])
    dt = torch.zeros(1000, 512, device=DEV)
    de = torch.randn(4, 64, 512, device=DEV).bfloat16()
    K.embedding_bwd(de, ids, dt)
    ref = torch.zeros(1000, 512, device=DEV).index_add_(0, ids.flatten().long(), de.float().view(-1, 512))
    _close(dt, ref, 1e-3)
    _status_ok()


@pytest.mark.parametrize("B,S,H,causal,packed", [(1, 128, 1, True, False), (1, 256, 2, False, False),
                                                  (2, 512, 4, True, False), (1, 1024, 4, True, True)])
def test_flash_attention_fwd_bwd(K, B, S, H, causal, packed):
    from mindspore_b200.ops import flash_attn_kernel as FK
    from mindspore_b200.ops.attention import reference_attention
    assert FK.available()
    D = 128
    if packed:
        qkv = torch.randn(B, S, 3 * H * D, device=DEV).bfloat16()
        q, k, v = (qkv[..., i * H * D:(i + 1) * H * D].view(B, S, H, D) for i in range(3))
    else:
        q, k, v = (torch.randn(B, S, H, D, device=DEV).bfloat16() for _ in range(3))
    do = torch.randn(B, S, H, D, device=DEV).bfloat16()
    sc = 1 / math.sqrt(D)
    o, lse, q2, k2, v2 = FK.fwd(q, k, v, causal, sc)
    dq, dk, dv = FK.bwd(do, q2, k2, v2, o, lse, causal, sc)
    qf, kf, vf = (t.float().detach().requires_grad_(True) for t in (q, k, v))
    ref = reference_attention(qf, kf, vf, causal)
    ref.backward(do.float())
    _close(o, ref, 2e-2)
    _close(dq, qf.grad, 3e-2)
    _close(dk, kf.grad, 3e-2)
    _close(dv, vf.grad, 3e-2)
    _status_ok()


def test_llama_kernel_path_matches_fp32_reference():
    """Loss and every parameter gradient of a small Llama on the kernel path vs the same model in fp32 on CPU."""
    import mindspore_b200 as ms
    from mindspore_b200.models.llama import LlamaConfig, LlamaForCausalLM
    ms.set_context(device_target="GPU")
    ms.set_seed(0)
    cfg = LlamaConfig(vocab_size=2048, hidden_size=512, num_layers=2, num_heads=4, num_kv_heads=4,
                      ffn_hidden_size=1408, seq_length=256)
    net = LlamaForCausalLM(cfg)
    tokens = torch.randint(0, 2048, (2, 257), dtype=torch.int32, device=DEV)
    loss = net(ms.Tensor(tokens))
    loss.backward()
    got = {p.name: p.grad.float().cpu() for p in net.get_parameters()}
    ms.set_context(device_target="CPU")
    ref_net = LlamaForCausalLM(cfg)
    for a, b in zip(net.get_parameters(), ref_net.get_parameters()):
        b.set_data(a.detach().float().cpu(), slice_shape=True)
    ref_loss = ref_net(ms.Tensor(tokens.cpu()))
    ref_loss.backward()
    assert abs(float(loss) - float(ref_loss)) < 2e-2
    for p in ref_net.get_parameters():
        _close(got[p.name], p.grad, 6e-2, 1e-4)
    _status_ok()



@pytest.mark.parametrize("B,S,H,causal", [(1, 128, 1, True), (1, 256, 2, False), (2, 512, 4, True), (1, 1024, 4, True)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_flash_attention_forward_lse(K, B, S, H, causal, dtype):
    """Forward output and log-sum-exp against the fp32 reference, both element types."""
    from mindspore_b200.ops import flash_attn_kernel as FK
    from mindspore_b200.ops.attention import reference_attention
    D = 128
    q, k, v = (torch.randn(B, S, H, D, device=DEV).to(dtype) for _ in range(3))
    sc = 1 / math.sqrt(D)
    qf, kf, vf = q.float(), k.float(), v.float()
    ref = reference_attention(qf, kf, vf, causal)
    scores = torch.einsum("bqhd,bkhd->bhqk", qf, kf) * sc
    if causal:
        scores = scores.masked_fill(torch.ones(S, S, device=DEV, dtype=torch.bool).triu(1), float("-inf"))
    o, lse, *_ = FK.fwd(q, k, v, causal, sc)
    _close(o, ref, 2e-2)
    _close(lse, torch.logsumexp(scores, -1), 1e-3, 1e-3)
    _status_ok()


@pytest.mark.parametrize("tb", [True, False])
def test_matmul_primitive_accumulates_into_main_grad(K, tb):
    """MatMul whose weight owns an fp32 accumulator: two backward passes leave 2 x the weight gradient there (added
    by the wgrad GEMM epilogue) and no ``.grad``; the input gradient is returned as usual."""
    from mindspore_b200.ops import fused
    M, N, Kd = 512, 384, 256
    a = torch.randn(M, Kd, device=DEV).bfloat16().requires_grad_(True)
    w = torch.randn((N, Kd) if tb else (Kd, N), device=DEV).bfloat16().requires_grad_(True)
    w.main_grad = torch.zeros(w.shape, dtype=torch.float32, device=DEV)
    dy = torch.randn(M, N, device=DEV).bfloat16()
    for _ in range(2):
        fused.matmul(a, w, False, tb).backward(dy)
    assert w.grad is None
    wf = w.detach().float()
    ref_w = dy.float().t() @ a.detach().float() if tb else a.detach().float().t() @ dy.float()
    ref_a = dy.float() @ wf if tb else dy.float() @ wf.t()
    _close(w.main_grad, 2 * ref_w, 1e-2)
    _close(a.grad, 2 * ref_a, 2e-2)
    _status_ok()
