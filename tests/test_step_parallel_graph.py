"""Graph mode under semi_auto_parallel: the traced graph holds the inserted collectives; the post-trace pass
publishes parameter layouts, fusion buckets, communication volume and the strategy checkpoint."""
import os

import pytest
import torch

from _mp import run_ranks


def _worker(rank, world, tmp):
    import mindspore_b200 as ms
    from mindspore_b200 import nn, ops
    from mindspore_b200.communication import init
    from mindspore_b200.parallel import strategy_ckpt as SC
    ms.set_context(device_target="CPU", mode=ms.GRAPH_MODE)
    init("mccl")
    path = os.path.join(tmp, "strategy_%d.ckpt" % rank)
    ms.set_auto_parallel_context(parallel_mode="semi_auto_parallel", device_num=world, global_rank=rank,
                                 full_batch=True, strategy_ckpt_save_file=path)

    class Net(nn.Cell):
        def __init__(self):
            super().__init__()
            torch.manual_seed(5)
            self.w1 = ms.Parameter(ms.Tensor(torch.randn(32, 64) * 0.1), name="w1")
            self.w2 = ms.Parameter(ms.Tensor(torch.randn(64, 16) * 0.1), name="w2")
            self.m1 = ops.MatMul().shard(((1, 1), (1, 2)))          # column parallel
            self.m2 = ops.MatMul().shard(((1, 2), (2, 1)))          # row parallel -> AllReduce
            self.relu = ops.ReLU()
            self.sum = ops.ReduceSum()

        def construct(self, x):
            return self.sum(self.m2(self.relu(self.m1(x, self.w1)), self.w2), ())

    net = Net()
    x = torch.randn(8, 32, generator=torch.Generator().manual_seed(1))
    out = float(net(ms.Tensor(x)))
    layouts = getattr(net, "parameter_layout_dict", None)
    vol = getattr(net, "_comm_volume", None)
    saved = SC.StrategyFile.load(path) if os.path.isfile(path) else None
    torch.distributed.barrier()
    return out, layouts, vol, None if saved is None else {k: v.as_list() for k, v in saved.layouts.items()}


def test_graph_mode_step_parallel_annotations(tmp_path):
    torch.manual_seed(5)
    w1, w2 = torch.randn(32, 64) * 0.1, torch.randn(64, 16) * 0.1
    x = torch.randn(8, 32, generator=torch.Generator().manual_seed(1))
    expect = float((torch.relu(x @ w1) @ w2).sum())
    for out, layouts, vol, saved in run_ranks(_worker, 2, str(tmp_path)):
        assert out == pytest.approx(expect, rel=1e-4)
        assert layouts is not None and set(layouts) == {"w1", "w2"}
        assert layouts["w1"]["tensor_map"][1] != -1 and layouts["w2"]["tensor_map"][0] != -1
        assert vol is not None and "AllReduce" in vol
        assert saved is not None and set(saved) == {"w1", "w2"}
