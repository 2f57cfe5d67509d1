"""Pipeline parallelism: stage-local execution with 1F1B / GPipe schedules over gloo ranks must give the
parameters a single process gets with the same micro-batching."""
import pytest
import torch

from _mp import run_ranks


def _build(ms, nn, stages):
    class Block(nn.Cell):
        def __init__(self, i):
            super().__init__()
            self.fc = nn.Dense(16, 16)
            self.act = nn.Tanh()

        def construct(self, x):
            return self.act(self.fc(x)) + x

    class Head(nn.Cell):
        def __init__(self):
            super().__init__()
            self.fc = nn.Dense(16, 4)
            self.loss = nn.MSELoss()

        def construct(self, x, y):
            return self.loss(self.fc(x), y)

    class Net(nn.Cell):
        def __init__(self):
            super().__init__()
            self.blocks = nn.CellList([Block(i) for i in range(4)])
            self.head = Head()
            per = 4 // stages
            for i, b in enumerate(self.blocks):
                b.pipeline_stage = min(i // per, stages - 1)
            self.head.pipeline_stage = stages - 1

        def construct(self, x, y):
            for b in self.blocks:
                x = b(x)
            return self.head(x, y)

    torch.manual_seed(11)
    ms.set_seed(11)
    return Net()


def _data():
    g = torch.Generator().manual_seed(5)
    return torch.randn(8, 16, generator=g), torch.randn(8, 4, generator=g)


def _single(micro):
    import mindspore_b200 as ms
    from mindspore_b200 import nn
    net = _build(ms, nn, 1)
    opt = nn.SGD(net.trainable_params(), learning_rate=0.1)
    step = nn.TrainOneStepCell(nn.GradAccumulationCell(net, micro), opt)
    x, y = _data()
    losses = [float(step(ms.Tensor(x), ms.Tensor(y))) for _ in range(2)]
    return losses, {p.name: p.detach().clone() for p in net.get_parameters()}


def _worker(rank, world, stages, micro, scheduler):
    import mindspore_b200 as ms
    from mindspore_b200 import nn
    from mindspore_b200.communication import init
    ms.set_context(device_target="CPU")
    init("mccl")
    ms.set_auto_parallel_context(parallel_mode="semi_auto_parallel", device_num=world, global_rank=rank,
                                 pipeline_stages=stages, pipeline_config={"pipeline_scheduler": scheduler})
    net = _build(ms, nn, stages)
    opt = nn.SGD(net.trainable_params(), learning_rate=0.1)
    step = nn.TrainOneStepCell(nn.PipelineCell(net, micro), opt)
    x, y = _data()
    losses = [float(step(ms.Tensor(x), ms.Tensor(y))) for _ in range(2)]
    stage = rank // (world // stages)
    mine = {p.name: p.detach().clone() for p in net.get_parameters() if stage in p._pipeline_stage_list}
    torch.distributed.barrier()
    return stage, losses, mine


@pytest.mark.parametrize("stages,micro,scheduler", [(2, 4, "1f1b"), (4, 4, "1f1b"), (2, 2, "gpipe")])
def test_pipeline_matches_single_process(stages, micro, scheduler):
    ref_losses, ref_params = _single(micro)
    res = run_ranks(_worker, stages, stages, micro, scheduler)
    seen = set()
    for stage, losses, params in res:
        if stage == stages - 1:
            assert losses == pytest.approx(ref_losses, rel=1e-5)
        for name, value in params.items():
            torch.testing.assert_close(value, ref_params[name], rtol=1e-5, atol=1e-6)
            seen.add(name)
    assert seen == set(ref_params)
