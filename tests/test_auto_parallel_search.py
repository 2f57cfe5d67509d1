"""auto_parallel: strategy search (sharding propagation / dynamic programming) picks strategies that the SPMD
execution then runs; results equal the single-device computation."""
import pytest
import torch

from _mp import run_ranks


def _worker(rank, world, search_mode, configure_first):
    import mindspore_b200 as ms
    from mindspore_b200 import nn, ops
    from mindspore_b200.communication import init
    ms.set_context(device_target="CPU", mode=ms.GRAPH_MODE)
    init("mccl")
    ms.set_auto_parallel_context(parallel_mode="auto_parallel", search_mode=search_mode, device_num=world,
                                 global_rank=rank, full_batch=True)

    class Net(nn.Cell):
        def __init__(self):
            super().__init__()
            torch.manual_seed(5)
            self.w1 = ms.Parameter(ms.Tensor(torch.randn(32, 64) * 0.1), name="w1")
            self.w2 = ms.Parameter(ms.Tensor(torch.randn(64, 16) * 0.1), name="w2")
            self.m1 = ops.MatMul()
            if configure_first:
                self.m1.shard(((1, 1), (1, world)))
            self.m2 = ops.MatMul()
            self.relu = ops.ReLU()
            self.sum = ops.ReduceSum()

        def construct(self, x):
            return self.sum(self.m2(self.relu(self.m1(x, self.w1)), self.w2), ())

    net = Net()
    x = torch.randn(8, 32, generator=torch.Generator().manual_seed(1))
    out = float(net(ms.Tensor(x)))
    chosen = getattr(net, "_searched_strategies", {})
    torch.distributed.barrier()
    return out, net.m1.in_strategy, net.m2.in_strategy, net.relu.in_strategy, len(chosen)


@pytest.mark.parametrize("search_mode,configure_first", [("sharding_propagation", True),
                                                         ("dynamic_programming", False),
                                                         ("recursive_programming", True)])
def test_auto_parallel_search_and_run(search_mode, configure_first):
    torch.manual_seed(5)
    w1, w2 = torch.randn(32, 64) * 0.1, torch.randn(64, 16) * 0.1
    x = torch.randn(8, 32, generator=torch.Generator().manual_seed(1))
    expect = float((torch.relu(x @ w1) @ w2).sum())
    for out, s1, s2, s_relu, n in run_ranks(_worker, 2, search_mode, configure_first):
        assert out == pytest.approx(expect, rel=1e-4)
        assert s1 is not None and s2 is not None and s_relu is not None and n >= 3
        if configure_first:
            assert s1 == ((1, 1), (1, 2))
            # column-parallel first layer: the cheapest continuation keeps the activation split and makes the
            # second MatMul row-parallel (no redistribution in between)
            assert s_relu == ((1, 2),) and s2 == ((1, 2), (2, 1))
