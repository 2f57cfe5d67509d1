"""Checks that stand in for memory / race tooling on the GPU kernels: model-sized GEMM shapes with a per-element
tolerance, split-K accumulation, canary regions around outputs (an out-of-bounds store shows up as a changed
canary), and run-twice bitwise equality for the kernels that claim a fixed reduction order."""
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


def _status_ok():
    from mindspore_b200 import _native
    torch.cuda.synchronize()
    assert _native.device_status() == 0


def _elementwise_close(got, exp, k, rel=2e-2):
    """bf16 inputs, fp32 accumulation: the error of one output element is bounded by the rounding of the result
    (2^-8 relative) plus accumulation-order noise that grows like sqrt(K) times the size of one product."""
    got, exp = got.float(), exp.float()
    tol = rel * exp.abs() + 4e-3 * (k ** 0.5)
    bad = (got - exp).abs() > tol
    assert not bool(bad.any()), "%d of %d elements off, worst %g" % (int(bad.sum()), bad.numel(),
                                                                     float(((got - exp).abs() - tol).max()))


@pytest.mark.parametrize("M,N,Kd", [(4096, 4096, 4096), (2048, 22016, 4096), (2048, 4096, 11008), (4096, 512, 4096),
                                    (4096, 4096, 512), (4096, 1536, 4096), (4096, 4096, 1376)])
def test_gemm_model_shapes_per_element(K, M, N, Kd):
    a = torch.randn(M, Kd, device=DEV).bfloat16()
    b = torch.randn(N, Kd, device=DEV).bfloat16()
    _elementwise_close(K.gemm(a, b), a.float() @ b.float().t(), Kd)
    dy = torch.randn(M, N, device=DEV).bfloat16()
    _elementwise_close(K.linear_dgrad(dy, b), dy.float() @ b.float(), N)
    _status_ok()


@pytest.mark.parametrize("rows,N,Kd", [(4096, 4096, 512), (4096, 1536, 4096), (4096, 4096, 1376), (4096, 2752, 4096),
                                       (8192, 4096, 4096)])
def test_wgrad_split_k_accumulates_exactly_once(K, rows, N, Kd):
    """dW[N, K] += dY[rows, N]^T X[rows, K] into an fp32 accumulator, twice: shapes whose tile count is a poor
    multiple of the SM-pair count run with split-K, the partial products meeting in the TMA reduce epilogue."""
    dy = torch.randn(rows, N, device=DEV).bfloat16()
    x = torch.randn(rows, Kd, device=DEV).bfloat16()
    acc = torch.full((N, Kd), 0.5, device=DEV)
    K.linear_wgrad(dy, x, out=acc, accumulate=True)
    K.linear_wgrad(dy, x, out=acc, accumulate=True)
    _elementwise_close(acc, 0.5 + 2 * (dy.float().t() @ x.float()), rows)
    from mindspore_b200 import _native
    lib = _native.cuda()
    lib.msb_gemm_pair_set_splitk(0)
    try:
        ref = torch.full((N, Kd), 0.5, device=DEV)
        K.linear_wgrad(dy, x, out=ref, accumulate=True)
        K.linear_wgrad(dy, x, out=ref, accumulate=True)
    finally:
        lib.msb_gemm_pair_set_splitk(1)
    _elementwise_close(acc, ref, rows, rel=1e-3)
    _status_ok()


def _with_canaries(shape, dtype, pad=4096):
    n = 1
    for s in shape:
        n *= s
    flat = torch.full((n + 2 * pad,), 7.0, device=DEV, dtype=dtype)
    return flat, flat[pad:pad + n].view(shape), pad


def _canaries_intact(flat, pad):
    return bool((flat[:pad] == 7).all()) and bool((flat[-pad:] == 7).all())


def test_outputs_stay_inside_their_buffers(K):
    """GEMM (ragged edges, both epilogues), RMSNorm, SwiGLU and cross entropy write into views surrounded by
    canary elements; none of the canaries may change."""
    M, N, Kd = 1000, 1352, 328
    a = torch.randn(M, Kd, device=DEV).bfloat16()
    b = torch.randn(N, Kd, device=DEV).bfloat16()
    flat, out, pad = _with_canaries((M, N), torch.bfloat16)
    K.gemm(a, b, out=out)
    assert _canaries_intact(flat, pad)
    torch.testing.assert_close(out.float(), a.float() @ b.float().t(), rtol=2e-2, atol=0.5)
    flat32, out32, pad = _with_canaries((N, Kd), torch.float32)
    out32.zero_()
    K.linear_wgrad(torch.randn(M, N, device=DEV).bfloat16(), a, out=out32, accumulate=True)
    assert _canaries_intact(flat32, pad)
    # big enough for the CTA-pair kernel with split-K
    flat32, out32, pad = _with_canaries((4096, 1536), torch.float32)
    out32.zero_()
    K.linear_wgrad(torch.randn(4096, 4096, device=DEV).bfloat16(), torch.randn(4096, 1536, device=DEV).bfloat16(),
                   out=out32, accumulate=True)
    assert _canaries_intact(flat32, pad)
    _status_ok()


def test_norm_backward_is_bitwise_repeatable(K):
    """The weight gradient of RMSNorm / LayerNorm is reduced in two stages with a fixed order: two runs on the same
    data give identical bits (an atomic reduction would not)."""
    rows, H = 3000, 4096
    x = torch.randn(rows, H, device=DEV).bfloat16()
    dy = torch.randn(rows, H, device=DEV).bfloat16()
    w = torch.randn(H, device=DEV).bfloat16()
    y, rstd, _ = K.rmsnorm_fwd(x, w, 1e-5)
    outs = []
    for _ in range(3):
        dw = torch.zeros(H, device=DEV)
        dx, _ = K.rmsnorm_bwd(dy, x, w, rstd, dw_out=dw, accumulate=True)
        outs.append((dx.clone(), dw.clone()))
    for dx, dw in outs[1:]:
        assert torch.equal(dx, outs[0][0]) and torch.equal(dw, outs[0][1])
    xf = x.float().requires_grad_(True)
    wf = w.float().requires_grad_(True)
    ref = (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-5) * wf)
    ref.backward(dy.float())
    torch.testing.assert_close(outs[0][1], wf.grad, rtol=2e-2, atol=2e-1)
    b = torch.randn(H, device=DEV).bfloat16()
    _, mean, rstd2 = K.layernorm_fwd(x, w, b, 1e-5)
    ln = []
    for _ in range(2):
        dw = torch.zeros(H, device=DEV)
        db = torch.zeros(H, device=DEV)
        dx, _, _ = K.layernorm_bwd(dy, x, w, mean, rstd2, dw_out=dw, db_out=db, accumulate=True)
        ln.append((dx.clone(), dw.clone(), db.clone()))
    assert all(torch.equal(a_, b_) for a_, b_ in zip(ln[0], ln[1]))
    torch.testing.assert_close(ln[0][2], dy.float().sum(0), rtol=2e-2, atol=2e-1)
    _status_ok()


def test_flash_attention_backward_is_bitwise_repeatable():
    from mindspore_b200.ops import flash_attn_kernel as FK
    if not FK.available():
        pytest.skip("attention kernels not built")
    B, S, H, D = 2, 1024, 4, 128
    q, k, v = (torch.randn(B, S, H, D, device=DEV).bfloat16() for _ in range(3))
    do = torch.randn(B, S, H, D, device=DEV).bfloat16()
    sc = D ** -0.5
    o, lse = FK.fwd(q, k, v, True, sc)[:2]
    first = [t.clone() for t in FK.bwd(do, q, k, v, o, lse, True, sc)]
    for _ in range(2):
        again = FK.bwd(do, q, k, v, o, lse, True, sc)
        assert all(torch.equal(a_, b_) for a_, b_ in zip(first, again))
    o2, lse2 = FK.fwd(q, k, v, True, sc)[:2]
    assert torch.equal(o, o2) and torch.equal(lse, lse2)
    _status_ok()
