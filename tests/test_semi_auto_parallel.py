"""semi_auto_parallel: shard strategies on primitives execute as SPMD (2 CPU ranks over gloo) and reproduce the
single-device result and gradients; layouts and inserted communication follow the reference's rules."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _net_and_data():
    import mindspore_b200 as ms
    from mindspore_b200 import nn, ops
    from mindspore_b200.common.initializer import initializer

    class Net(nn.Cell):
        def __init__(self, s1, s2, out2=None):
            super().__init__()
            torch.manual_seed(5)
            self.w1 = ms.Parameter(ms.Tensor(torch.randn(32, 64) * 0.1), name="w1")
            self.w2 = ms.Parameter(ms.Tensor(torch.randn(64, 16) * 0.1), name="w2")
            self.m1 = ops.MatMul().shard(s1)
            self.m2 = ops.MatMul().shard(s2, out2)
            self.relu = ops.ReLU()
            self.sum = ops.ReduceSum()

        def construct(self, x):
            h = self.relu(self.m1(x, self.w1))
            y = self.m2(h, self.w2)
            return self.sum(y * y, ())
    x = torch.randn(8, 32, generator=torch.Generator().manual_seed(1))
    return Net, x


def _worker(rank, world, port, q, s1, s2, out2):
    sys.path.insert(0, ROOT)
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    import mindspore_b200 as ms
    from mindspore_b200.communication import init
    from mindspore_b200.parallel import spmd
    ms.set_context(device_target="CPU")
    Net, x = _net_and_data()
    ref = Net(None, None)
    ref.m1.in_strategy = ref.m2.in_strategy = None
    ms.set_auto_parallel_context(parallel_mode="stand_alone")
    xr = ms.Tensor(x)
    lr = ref(xr)
    gr = torch.autograd.grad(lr, [ref.w1, ref.w2])
    init("mccl")
    ms.set_auto_parallel_context(parallel_mode="semi_auto_parallel", device_num=world, global_rank=rank,
                                 full_batch=True)
    net = Net(s1, s2, out2)
    loss = net(ms.Tensor(x))
    loss_full = spmd.to_full(loss)
    # the scalar loss is replicated over the ranks: _VirtualDiv scales the incoming gradient by 1/replicas so that
    # summed (AllReduce) weight gradients are not counted several times
    g = torch.autograd.grad(spmd.virtual_div_loss(loss), [net.w1, net.w2])
    errs = []
    for p, gi, gf in zip([net.w1, net.w2], g, gr):
        lay = p.param_layout
        from mindspore_b200.parallel.layout import slice_for_rank
        want = slice_for_rank(gf, lay, rank) if lay is not None else gf
        errs.append(float((gi - want).abs().max()))
    q.put((rank, float(loss_full), float(lr), max(errs), {k: v.to_dict() for k, v in spmd.parameter_layouts.items()}))
    torch.distributed.barrier()


def _run(world, s1, s2, out2=None):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 23000 + (os.getpid() * 7 + abs(hash((s1, s2))) % 500) % 4000
    procs = [ctx.Process(target=_worker, args=(r, world, port, q, s1, s2, out2)) for r in range(world)]
    for p in procs:
        p.start()
    import queue as _q
    import time
    res, deadline = [], time.time() + 240
    while len(res) < world:
        try:
            res.append(q.get(timeout=2))
        except _q.Empty:
            if any(p.exitcode not in (None, 0) for p in procs) or time.time() > deadline:
                for p in procs:
                    p.kill()
                raise AssertionError("worker failed: %s" % [p.exitcode for p in procs])
    for p in procs:
        p.join(30)
    return res


@pytest.mark.parametrize("s1,s2,out2", [
    (((2, 1), (1, 1)), ((2, 1), (1, 1)), None),            # data parallel: batch split, weights mirrored
    (((1, 1), (1, 2)), ((1, 2), (2, 1)), None),            # column parallel then row parallel (AllReduce)
    (((1, 2), (2, 1)), ((1, 1), (1, 2)), None),            # K-split first matmul, column-parallel second
    (((1, 1), (1, 2)), ((1, 2), (2, 1)), ((2, 1),)),       # row parallel with ReduceScatter output (seq parallel)
])
def test_two_matmul_strategies_match_single(s1, s2, out2):
    for rank, loss, ref, gerr, layouts in _run(2, s1, s2, out2):
        assert abs(loss - ref) < 1e-3 * max(1.0, abs(ref)), (rank, loss, ref)
        assert gerr < 1e-4, (rank, gerr)
        assert set(layouts) == {"w1", "w2"}


def test_operator_info_matmul_layouts():
    import mindspore_b200 as ms
    from mindspore_b200 import ops
    from mindspore_b200.parallel.operator_info import MatMulInfo, StrategyError
    info = MatMulInfo(ops.MatMul(), [(64, 32), (32, 16)], ((2, 4), (4, 1)), None, stage_devices=8)
    assert info.dev_matrix == [2, 4, 1]
    assert info.inputs_tensor_map == [[2, 1], [1, -1]]
    assert info.outputs_tensor_map == [[2, -1]]
    assert info.forward_comm == ("AllReduce", [1])
    rs = MatMulInfo(ops.MatMul(), [(64, 32), (32, 16)], ((2, 4), (4, 1)), ((8, 1),), stage_devices=8)
    assert rs.forward_comm[0] == "ReduceScatter" and rs.output_layouts()[0].slice_shape() == (8, 16)
    rep = MatMulInfo(ops.MatMul(), [(64, 32), (32, 16)], ((2, 1), (1, 2)), None, stage_devices=8)
    assert rep.dev_matrix == [2, 2, 1, 2] and rep.repeat == 2 and rep.as_loss_divisor() == 2
    with pytest.raises(StrategyError):
        MatMulInfo(ops.MatMul(), [(64, 32), (32, 16)], ((2, 4), (2, 1)), None, stage_devices=8)
    with pytest.raises(StrategyError):
        MatMulInfo(ops.MatMul(), [(64, 32), (32, 16)], ((3, 1), (1, 1)), None, stage_devices=8)
