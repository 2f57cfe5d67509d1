"""Mixture of experts: routing arithmetic, row dispatch/combine vs the dense one-hot (GShard) formulation,
expert parallelism over gloo ranks, and the CUDA router / scatter / gather kernels."""
import pytest
import torch

import mindspore_b200 as ms
from mindspore_b200.parallel import moe as MOE

from _mp import run_ranks


def _layer(E, k, H, F, cf=1.5, act="gelu", group=None, dtype=torch.float32, seed=3):
    torch.manual_seed(seed)
    ms.set_seed(seed)
    cfg = MOE.MoEConfig(expert_num=E, capacity_factor=cf, num_experts_chosen=k, aux_loss_factor=0.05)
    return MOE.MoE(H, F, hidden_act=act, moe_config=cfg, expert_parallel_group=group, param_init_type=dtype)


def test_capacity_and_config_checks():
    assert MOE.calculate_expert_capacity(2, 64, 1.0, 8) == 16
    assert MOE.calculate_expert_capacity(1, 10, 1.1, 4) == 3
    with pytest.raises(ValueError):
        MOE.MoEConfig(expert_num=4, capacity_factor=0.5)
    with pytest.raises(ValueError):
        MOE.MoEConfig(expert_num=2, num_experts_chosen=3)


@pytest.mark.parametrize("k,cf", [(1, 1.0), (2, 1.0), (2, 2.0)])
def test_router_reference_invariants(k, cf):
    torch.manual_seed(0)
    T, E = 96, 8
    logits = torch.randn(T, E) * 2
    cap = MOE.calculate_expert_capacity(k, T, cf, E)
    expert, slot, weight, loss = MOE.router_reference(logits, k, cap)
    kept = slot >= 0
    assert int(slot.max()) < cap
    # a slot of an expert is used at most once
    flat = (expert.long() * cap + slot.long())[kept]
    assert flat.unique().numel() == flat.numel()
    assert torch.all(weight[~kept] == 0)
    if k > 1:
        s = weight.sum(-1)
        assert torch.allclose(s[kept.any(-1)], torch.ones_like(s[kept.any(-1)]), atol=1e-5)
    assert float(loss) > 0


@pytest.mark.parametrize("k,act", [(1, "gelu"), (2, "gelu"), (2, "swiglu")])
def test_moe_layer_matches_dense_formulation(k, act):
    E, H, F, T = 4, 16, 32, 40
    net = _layer(E, k, H, F, cf=1.25, act=act)
    x = ms.Tensor(torch.randn(T, H)).requires_grad_(True)
    out, aux = net(x)
    (out.sum() + aux).backward()
    xr = x.detach().clone().as_subclass(torch.Tensor).requires_grad_(True)
    ps = {n: p.detach().clone().requires_grad_(True) for n, p in
          (("r", net.router_weight), ("w1", net.w1), ("w2", net.w2), ("b1", net.b1), ("b2", net.b2))}
    ref, aux_ref = MOE.moe_reference_forward(xr, ps["r"], ps["w1"], ps["w2"], ps["b1"], ps["b2"], k, 1.25, act)
    (ref.sum() + aux_ref * 0.05).backward()
    torch.testing.assert_close(out.as_subclass(torch.Tensor), ref, rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(float(aux), float(aux_ref) * 0.05, rtol=1e-5, atol=1e-7)
    torch.testing.assert_close(x.grad.as_subclass(torch.Tensor), xr.grad, rtol=1e-4, atol=1e-5)
    for name, p in (("r", net.router_weight), ("w1", net.w1), ("w2", net.w2)):
        torch.testing.assert_close(p.grad.as_subclass(torch.Tensor), ps[name].grad, rtol=1e-3, atol=1e-5)


def _ep_worker(rank, world):
    from mindspore_b200.communication import init
    ms.set_context(device_target="CPU")
    init("mccl")
    E, H, F, T, k = 4, 16, 32, 24, 2
    full = _layer(E, k, H, F, cf=2.0)                     # same seed on every rank: identical full weights
    net = _layer(E, k, H, F, cf=2.0, group=ms.communication.GlobalComm.WORLD_COMM_GROUP)
    el = E // world
    with torch.no_grad():
        full.b1.copy_(torch.randn(full.b1.shape, generator=torch.Generator().manual_seed(5)) * 0.2)
        full.b2.copy_(torch.randn(full.b2.shape, generator=torch.Generator().manual_seed(6)) * 0.2)
        net.router_weight.copy_(full.router_weight)
        for a, b in ((net.w1, full.w1), (net.w2, full.w2), (net.b1, full.b1), (net.b2, full.b2)):
            a.copy_(b[rank * el:(rank + 1) * el])
    g = torch.Generator().manual_seed(100 + rank)
    x = ms.Tensor(torch.randn(T, H, generator=g)).requires_grad_(True)
    out, aux = net(x)
    (out.sum() + aux).backward()
    # the same tokens through the full single-rank layer: capacity per (source rank, expert) is the same
    xr = ms.Tensor(x.detach().clone()).requires_grad_(True)
    ref, aux_ref = full(xr)
    (ref.sum() + aux_ref).backward()
    err_out = float((out - ref).abs().max())
    err_dx = float((x.grad - xr.grad).abs().max())
    # expert gradients on the owner sum the contributions of every rank's tokens
    gw = full.w1.grad.as_subclass(torch.Tensor).clone()
    torch.distributed.all_reduce(gw)
    err_dw = float((net.w1.grad.as_subclass(torch.Tensor) - gw[rank * el:(rank + 1) * el]).abs().max())
    torch.distributed.barrier()
    return err_out, err_dx, err_dw, float(aux), float(aux_ref)


def test_expert_parallel_over_gloo_matches_single_rank():
    for err_out, err_dx, err_dw, aux, aux_ref in run_ranks(_ep_worker, 2):
        assert err_out < 1e-5 and err_dx < 1e-5 and err_dw < 1e-4
        assert aux == pytest.approx(aux_ref, rel=1e-5)


def test_grad_reducer_leaves_expert_parameters_local():
    from mindspore_b200 import nn
    net = _layer(4, 1, 8, 16)
    net.w1.dp_local = True
    red = nn.DistributedGradReducer(list(net.get_parameters()), mean=True, degree=4)
    idx = [i for i, p in enumerate(red.params) if p is net.w1]
    assert idx and idx[0] in red.local_only and all(idx[0] not in b for b in red.buckets)


# ------------------------------------------------------------------------------------------------ CUDA kernels
@pytest.mark.gpu
@pytest.mark.parametrize("T,E,k,cf", [(300, 8, 2, 1.0), (4096, 64, 2, 1.25), (1000, 16, 1, 1.0), (777, 160, 4, 2.0)])
def test_router_kernel_matches_reference(T, E, k, cf):
    from mindspore_b200 import _native
    torch.manual_seed(1)
    logits = (torch.randn(T, E, device="cuda") * 2).requires_grad_(True)
    cap = MOE.calculate_expert_capacity(k, T, cf, E)
    expert, slot, weight, loss = MOE.route(logits, k, cap)
    dw = torch.randn_like(weight)
    (weight * dw).sum().add(loss * 0.3).backward()
    lr = logits.detach().clone().requires_grad_(True)
    e2, s2, w2, l2 = MOE.router_reference(lr, k, cap)
    ((w2 * dw).sum() + l2 * 0.3).backward()
    assert torch.equal(expert, e2) and torch.equal(slot, s2)
    torch.testing.assert_close(weight, w2, rtol=1e-4, atol=1e-6)
    torch.testing.assert_close(loss, l2, rtol=1e-4, atol=1e-6)
    torch.testing.assert_close(logits.grad, lr.grad, rtol=2e-3, atol=1e-6)
    torch.cuda.synchronize()
    assert _native.device_status() == 0


@pytest.mark.gpu
@pytest.mark.parametrize("k,act", [(2, "gelu"), (2, "swiglu"), (1, "gelu")])
def test_moe_layer_kernels_match_dense_formulation(k, act):
    from mindspore_b200 import _native
    ms.set_context(device_target="GPU")
    E, H, F, T = 8, 256, 512, 1024
    net = _layer(E, k, H, F, cf=1.25, act=act, dtype=torch.bfloat16)
    assert net.w1.is_cuda
    x = ms.Tensor(torch.randn(T, H, device="cuda").bfloat16()).requires_grad_(True)
    out, aux = net(x)
    assert isinstance(next(iter(net._transports.values())), MOE._KernelTransport)
    dy = torch.randn_like(out.as_subclass(torch.Tensor))
    ((out.as_subclass(torch.Tensor).float() * dy.float()).sum() + aux).backward()
    xr = x.detach().float().as_subclass(torch.Tensor).requires_grad_(True)
    ps = {n: p.detach().float().clone().requires_grad_(True) for n, p in
          (("r", net.router_weight), ("w1", net.w1), ("w2", net.w2), ("b1", net.b1), ("b2", net.b2))}
    cap_factor = ((MOE.calculate_expert_capacity(k, T, 1.25, E) + 7) // 8 * 8) * E / (k * T)
    ref, aux_ref = MOE.moe_reference_forward(xr, ps["r"], ps["w1"], ps["w2"], ps["b1"], ps["b2"], k, cap_factor, act)
    ((ref * dy.float()).sum() + aux_ref * 0.05).backward()
    scale = ref.abs().max().item()
    assert (out.as_subclass(torch.Tensor).float() - ref).abs().max().item() <= 3e-2 * scale + 1e-3
    assert (x.grad.float() - xr.grad).abs().max().item() <= 5e-2 * xr.grad.abs().max().item() + 1e-3
    g1 = net.w1.grad if net.w1.grad is not None else net.w1.main_grad
    assert (g1.float() - ps["w1"].grad).abs().max().item() <= 5e-2 * ps["w1"].grad.abs().max().item() + 1e-3
    torch.cuda.synchronize()
    assert _native.device_status() == 0


def _ep_gpu_worker(rank, world, fused, drops=False):
    from mindspore_b200 import _native
    from mindspore_b200.communication import init
    torch.cuda.set_device(rank)
    ms.set_context(device_target="GPU", device_id=rank)
    init("nccl")
    E, H, F, T, k = 8, 256, 512, 512, 2
    cf = 2.0
    if drops:                                   # capacity 256 for 2048 choices over 8 experts: tokens are dropped
        H, F, T, cf = 512, 1024, 1024, 1.0
    full = _layer(E, k, H, F, cf=cf, dtype=torch.bfloat16)
    net = _layer(E, k, H, F, cf=cf, group=ms.communication.GlobalComm.WORLD_COMM_GROUP, dtype=torch.bfloat16)
    net.fused_transport = fused
    net.fused_gemm = fused
    el = E // world
    with torch.no_grad():
        full.b1.copy_(torch.randn(full.b1.shape, generator=torch.Generator().manual_seed(5)) * 0.2)
        full.b2.copy_(torch.randn(full.b2.shape, generator=torch.Generator().manual_seed(6)) * 0.2)
        net.router_weight.copy_(full.router_weight)
        for a, b in ((net.w1, full.w1), (net.w2, full.w2), (net.b1, full.b1), (net.b2, full.b2)):
            a.copy_(b[rank * el:(rank + 1) * el])
    g = torch.Generator().manual_seed(100 + rank)
    x = ms.Tensor(torch.randn(T, H, generator=g).bfloat16().cuda()).requires_grad_(True)
    out, aux = net(x)
    kind = type(next(iter(net._transports.values()))).__name__
    (out.float().sum() + aux).backward()
    xr = ms.Tensor(x.detach().clone()).requires_grad_(True)
    ref, aux_ref = full(xr)
    (ref.float().sum() + aux_ref).backward()
    scale = float(ref.float().abs().max())
    err_out = float((out.float() - ref.float()).abs().max()) / scale
    err_dx = float((x.grad.float() - xr.grad.float()).abs().max()) / float(xr.grad.float().abs().max())
    # expert weights see the tokens of every rank: the full layer's gradients summed over the ranks, sliced
    err_dw = 0.0
    for a, b in ((net.w1, full.w1), (net.w2, full.w2), (net.b1, full.b1), (net.b2, full.b2)):
        gf = (b.grad if b.grad is not None else b.main_grad).float().clone()
        torch.distributed.all_reduce(gf)
        ga = (a.grad if a.grad is not None else a.main_grad).float()
        ref_slice = gf[rank * el:(rank + 1) * el]
        err_dw = max(err_dw, float((ga - ref_slice).abs().max()) / (float(ref_slice.abs().max()) + 1e-6))
    torch.cuda.synchronize()
    status = _native.device_status()
    torch.distributed.barrier()
    ms.communication.release()
    return kind, err_out, err_dx, err_dw, float(aux), float(aux_ref), status


@pytest.mark.gpu
@pytest.mark.parametrize("fused,drops", [(True, False), (False, False), (True, True)])
def test_expert_parallel_on_2_gpus(fused, drops):
    """fused: the expert GEMMs run the row exchange themselves (gather form in front of the first, push form behind
    the second, and the mirrored forms in backward); otherwise torch all_to_all around batched GEMMs."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    for kind, err_out, err_dx, err_dw, aux, aux_ref, status in run_ranks(_ep_gpu_worker, 2, fused, drops):
        assert kind == ("_KernelTransport" if fused else "_TorchTransport")
        assert status == 0
        assert err_out < 3e-2 and err_dx < 5e-2 and err_dw < 5e-2, (err_out, err_dx, err_dw)
        assert aux == pytest.approx(aux_ref, rel=1e-3)
