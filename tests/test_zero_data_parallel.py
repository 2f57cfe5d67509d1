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
