"""Data parallelism on the parameter arena and the sharded (ZeRO-style) optimizer step: gloo ranks must end with
the parameters a single process gets on the whole batch."""
import pytest
import torch

from _mp import run_ranks


def _net(ms, nn):
    torch.manual_seed(21)
    ms.set_seed(21)

    class Net(nn.Cell):
        def __init__(self):
            super().__init__()
            self.a = nn.Dense(24, 40)
            self.b = nn.Dense(40, 8)
            self.loss = nn.MSELoss()

        def construct(self, x, y):
            return self.loss(self.b(torch.tanh(self.a(x))), y)

    return Net()


def _data():
    g = torch.Generator().manual_seed(9)
    return torch.randn(16, 24, generator=g), torch.randn(16, 8, generator=g)


def _opt(nn, net, clip):
    return nn.AdamWeightDecay(net.trainable_params(), learning_rate=1e-2, weight_decay=0.1, use_arena=True,
                              max_grad_norm=clip)


def _single(clip):
    import mindspore_b200 as ms
    from mindspore_b200 import nn
    net = _net(ms, nn)
    step = nn.TrainOneStepCell(net, _opt(nn, net, clip))
    x, y = _data()
    for _ in range(3):
        step(ms.Tensor(x), ms.Tensor(y))
    return {p.name: p.detach().clone() for p in net.get_parameters()}


def _worker(rank, world, shard, clip):
    import mindspore_b200 as ms
    from mindspore_b200 import nn
    from mindspore_b200.communication import GlobalComm, init
    ms.set_context(device_target="CPU")
    init("mccl")
    net = _net(ms, nn)
    opt = _opt(nn, net, clip)
    opt.set_data_parallel_group(GlobalComm.WORLD_COMM_GROUP, mean=True, shard=shard)
    step = nn.TrainOneStepCell(net, opt)
    x, y = _data()
    n = x.shape[0] // world
    for _ in range(3):
        step(ms.Tensor(x[rank * n:(rank + 1) * n]), ms.Tensor(y[rank * n:(rank + 1) * n]))
    sharded_state = opt._dp.shard and opt._dp.master.numel() < opt.arena.total
    torch.distributed.barrier()
    return {p.name: p.detach().clone() for p in net.get_parameters()}, sharded_state


@pytest.mark.parametrize("shard,clip", [(False, 0.0), (True, 0.0), (True, 0.05), (False, 0.05)])
def test_data_parallel_arena_matches_single_process(shard, clip):
    ref = _single(clip)
    for params, sharded_state in run_ranks(_worker, 2, shard, clip):
        assert sharded_state == shard
        for name, value in params.items():
            torch.testing.assert_close(value, ref[name], rtol=1e-5, atol=1e-6)


def _gpu_worker(rank, world, fused):
    import mindspore_b200 as ms
    from mindspore_b200 import _native, nn
    from mindspore_b200.communication import GlobalComm, init
    torch.cuda.set_device(rank)
    ms.set_context(device_target="GPU", device_id=rank)
    init("nccl")

    def build():
        torch.manual_seed(4)
        ms.set_seed(4)
        net = nn.SequentialCell([nn.Dense(256, 512), nn.Tanh(), nn.Dense(512, 256)]).to_float(torch.bfloat16)
        for p in net.get_parameters():
            p.set_data(p.detach().to(torch.bfloat16).cuda())
        return net

    def run(net, opt, x, y, steps=3):
        for _ in range(steps):
            opt.zero_grad()
            out = net(ms.Tensor(x))
            loss = ((out.float() - y) ** 2).mean()
            loss.backward()
            for p in net.get_parameters():
                if p.grad is not None:
                    p.main_grad.add_(p.grad.float())
                    p.grad = None
            opt.sync_data_parallel_grads()
            opt.fused_step()
        return {p.name: p.detach().float().clone() for p in net.get_parameters()}

    g = torch.Generator().manual_seed(8)
    x = torch.randn(64, 256, generator=g).bfloat16().cuda()
    y = torch.randn(64, 256, generator=g).cuda()
    ref_net = build()
    ref_opt = nn.AdamWeightDecay(ref_net.trainable_params(), learning_rate=1e-3, weight_decay=0.1, max_grad_norm=1.0)
    ref = run(ref_net, ref_opt, x, y)
    net = build()
    opt = nn.AdamWeightDecay(net.trainable_params(), learning_rate=1e-3, weight_decay=0.1, max_grad_norm=1.0)
    opt.set_data_parallel_group(GlobalComm.WORLD_COMM_GROUP, mean=True, shard=True, fused=fused)
    n = x.shape[0] // world
    got = run(net, opt, x[rank * n:(rank + 1) * n], y[rank * n:(rank + 1) * n])
    worst = max(float((got[k] - ref[k]).abs().max() / (ref[k].abs().max() + 1e-6)) for k in ref)
    torch.cuda.synchronize()
    status = _native.device_status()
    used_symm = opt._dp.symm is not None
    torch.distributed.barrier()
    ms.communication.release()
    return worst, status, used_symm


@pytest.mark.gpu
@pytest.mark.parametrize("fused", [True, False])
def test_sharded_optimizer_on_2_gpus(fused):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    for worst, status, used_symm in run_ranks(_gpu_worker, 2, fused):
        assert status == 0 and used_symm == fused
        assert worst < 2e-2


def _overlap_worker(rank, world, clip):
    from mindspore_b200.parallel import zero
    zero._OVERLAP_BUCKET_ELEMS = 512                      # several buckets even for this small net
    params, _ = _worker(rank, world, False, clip)
    import mindspore_b200  # noqa: F401
    return params, zero._last_overlapped


def test_allreduce_overlapped_with_backward_matches_single_process():
    """Buckets are all-reduced from inside backward as soon as their gradients are complete; the result must not
    change and at least one bucket must really have been launched early."""
    ref = _single(0.05)
    for params, overlapped in run_ranks(_overlap_worker, 2, 0.05):
        assert overlapped > 0
        for name, value in params.items():
            torch.testing.assert_close(value, ref[name], rtol=1e-5, atol=1e-6)


def _gpu_overlap_worker(rank, world, overlap):
    import os
    os.environ["MSB200_DP_OVERLAP"] = "1" if overlap else "0"
    import mindspore_b200 as ms
    from mindspore_b200 import _native, nn
    from mindspore_b200.communication import GlobalComm, init
    from mindspore_b200.parallel import zero
    zero._OVERLAP_BUCKET_ELEMS = 16 * 1024
    torch.cuda.set_device(rank)
    ms.set_context(device_target="GPU", device_id=rank)
    init("nccl")
    torch.manual_seed(11)
    ms.set_seed(11)

    class Net(nn.Cell):
        def __init__(self):
            super().__init__()
            self.c1 = nn.Conv2d(64, 64, 3, dtype=torch.bfloat16)
            self.bn1 = nn.BatchNorm2d(64)
            self.c2 = nn.Conv2d(64, 128, 3, stride=2, dtype=torch.bfloat16)
            self.bn2 = nn.BatchNorm2d(128)
            self.fc = nn.Dense(128, 16, dtype=torch.bfloat16)
            self.loss = nn.SoftmaxCrossEntropyWithLogits(sparse=True, reduction="mean")

        def construct(self, x, y):
            h = torch.relu(self.bn1(self.c1(x)))
            h = torch.relu(self.bn2(self.c2(h)))
            return self.loss(self.fc(h.mean((2, 3))).float(), y)

    net = Net()
    for p in net.get_parameters():
        # trainable parameters share one dtype (flat arena); moving statistics stay fp32
        p.set_data(p.detach().to(torch.bfloat16).cuda() if p.requires_grad else p.detach().cuda())
    opt = nn.Momentum(net.trainable_params(), 0.05, 0.9, weight_decay=1e-4)
    assert opt.arena is not None
    opt.set_data_parallel_group(GlobalComm.WORLD_COMM_GROUP, mean=True)
    step = nn.TrainOneStepCell(net, opt)
    step.set_train()
    g = torch.Generator().manual_seed(100 + rank)
    x = torch.randn(8, 64, 16, 16, generator=g).bfloat16().cuda()
    y = torch.randint(0, 16, (8,), generator=g).cuda()
    losses = [float(step(ms.Tensor(x), ms.Tensor(y))) for _ in range(4)]
    torch.cuda.synchronize()
    out = {p.name: p.detach().float().cpu() for p in net.trainable_params()}
    status = _native.device_status()
    torch.distributed.barrier()
    ms.communication.release()
    return out, losses, status, zero._last_overlapped


@pytest.mark.gpu
def test_overlapped_allreduce_on_2_gpus():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    base = run_ranks(_gpu_overlap_worker, 2, False)
    over = run_ranks(_gpu_overlap_worker, 2, True)
    for (p0, l0, s0, n0), (p1, l1, s1, n1) in zip(base, over):
        assert s0 == 0 and s1 == 0 and n0 == 0 and n1 > 0
        assert l1[-1] < l1[0]
        for k in p0:
            torch.testing.assert_close(p1[k], p0[k], rtol=2e-2, atol=2e-3)
    for k in over[0][0]:                                   # both ranks hold the same weights
        torch.testing.assert_close(over[0][0][k], over[1][0][k], rtol=0, atol=0)


class _KernelStyleLinear(torch.autograd.Function):
    """Stands in for the GPU kernel path on CPU ranks: backward accumulates the weight gradient straight into
    ``main_grad`` and reports it, like ops/fused.py::_LinearFn and _EmbeddingFn do."""

    @staticmethod
    def forward(ctx, x, w):
        ctx.save_for_backward(x, w.detach())
        ctx.w_ref = w
        return x @ w.detach().t()

    @staticmethod
    def backward(ctx, dy):
        from mindspore_b200.nn.optim import notify_grad_written
        x, w = ctx.saved_tensors
        ctx.w_ref.main_grad.add_(dy.t() @ x)
        notify_grad_written(ctx.w_ref)
        return dy @ w, None


def _tied_worker(rank, world, overlap):
    """A weight used twice in one step (tied table): its bucket may only be reduced after the second write."""
    import os
    os.environ["MSB200_DP_OVERLAP"] = "1" if overlap else "0"
    import mindspore_b200 as ms
    from mindspore_b200 import nn
    from mindspore_b200.communication import GlobalComm, init
    from mindspore_b200.common.parameter import Parameter
    from mindspore_b200.nn.optim import note_grad_producer
    from mindspore_b200.parallel import zero
    ms.set_context(device_target="CPU")
    init("mccl")
    torch.manual_seed(5)

    class Tied(nn.Cell):
        def __init__(self):
            super().__init__()
            self.table = Parameter(torch.randn(12, 12) * 0.3, name="table")
            self.mid = nn.Dense(12, 12)

        def construct(self, x):
            note_grad_producer(self.table)
            h = _KernelStyleLinear.apply(x, self.table)            # first use (its backward runs last)
            h = torch.tanh(self.mid(h))
            note_grad_producer(self.table)
            return _KernelStyleLinear.apply(h, self.table).pow(2).mean()   # second use (backward runs first)

    net = Tied()
    opt = nn.AdamWeightDecay(net.trainable_params(), learning_rate=1e-2, use_arena=True)
    opt.set_data_parallel_group(GlobalComm.WORLD_COMM_GROUP, mean=True, shard=False)
    step = nn.TrainOneStepCell(net, opt)
    g = torch.Generator().manual_seed(40 + rank)
    for _ in range(2):
        step(ms.Tensor(torch.randn(6, 12, generator=g)))
    torch.distributed.barrier()
    return {p.name: p.detach().clone() for p in net.get_parameters()}, zero._last_overlapped


def test_overlap_waits_for_the_last_write_of_a_shared_parameter():
    on = run_ranks(_tied_worker, 2, True)
    off = run_ranks(_tied_worker, 2, False)
    assert on[0][1] > 0, "the overlap path did not run"
    for (p_on, _), (p_off, _) in zip(on, off):
        for name in p_on:
            torch.testing.assert_close(p_on[name], p_off[name], rtol=0, atol=0)
    for name in on[0][0]:                       # replicas stay identical
        torch.testing.assert_close(on[0][0][name], on[1][0][name], rtol=0, atol=0)


def _loss_scale_worker(rank, world):
    import mindspore_b200 as ms
    from mindspore_b200 import nn
    from mindspore_b200.communication import GlobalComm, init
    ms.set_context(device_target="CPU")
    init("mccl")
    net = _net(ms, nn)
    opt = _opt(nn, net, 0.0)
    opt.set_data_parallel_group(GlobalComm.WORLD_COMM_GROUP, mean=True, shard=False)
    step = nn.TrainOneStepWithLossScaleCell(net, opt, nn.DynamicLossScaleUpdateCell(1024.0, 2.0, 1000))
    x, y = _data()
    n = x.shape[0] // world
    for _ in range(3):
        step(ms.Tensor(x[rank * n:(rank + 1) * n]), ms.Tensor(y[rank * n:(rank + 1) * n]))
    torch.distributed.barrier()
    return {p.name: p.detach().clone() for p in net.get_parameters()}


def test_loss_scale_cell_synchronises_gradients_over_the_data_parallel_group():
    ref = _single(0.0)
    for params in run_ranks(_loss_scale_worker, 2):
        for name, value in params.items():
            torch.testing.assert_close(value, ref[name], rtol=1e-4, atol=1e-5)


def test_overflow_step_does_not_advance_the_optimizer_step():
    import mindspore_b200 as ms
    from mindspore_b200 import nn
    net = _net(ms, nn)
    opt = _opt(nn, net, 0.0)
    step = nn.TrainOneStepWithLossScaleCell(net, opt, nn.DynamicLossScaleUpdateCell(1024.0, 2.0, 1000))
    x, y = _data()
    before = {p.name: p.detach().clone() for p in net.get_parameters()}
    bad = x.clone()
    bad[0, 0] = float("inf")
    _, overflow, scale = step(ms.Tensor(bad), ms.Tensor(y))
    assert bool(overflow) and opt._step_host == 0 and int(opt.global_step) == 0
    assert float(step.scale_sense) == 512.0
    for p in net.get_parameters():
        torch.testing.assert_close(p.detach(), before[p.name], rtol=0, atol=0)
    _, overflow, _ = step(ms.Tensor(x), ms.Tensor(y))
    assert not bool(overflow) and opt._step_host == 1 and int(opt.global_step) == 1
