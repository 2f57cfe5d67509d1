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
