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


def _mlp_graph(hidden=256, ffn=1024, batch=64, layers=2):
    """Traced forward graph of a residual MLP stack (full shapes, stand-alone mode)."""
    import mindspore_b200 as ms
    from mindspore_b200 import nn, ops
    from mindspore_b200.graph import jit as J
    ms.set_context(device_target="CPU", mode=ms.PYNATIVE_MODE)

    class Block(nn.Cell):
        def __init__(self, i):
            super().__init__()
            self.w1 = ms.Parameter(ms.Tensor(torch.randn(hidden, ffn) * 0.05), name="w1_%d" % i)
            self.w2 = ms.Parameter(ms.Tensor(torch.randn(ffn, hidden) * 0.05), name="w2_%d" % i)
            self.m1, self.m2, self.act, self.add = ops.MatMul(), ops.MatMul(), ops.GeLU(), ops.Add()

        def construct(self, x):
            return self.add(x, self.m2(self.act(self.m1(x, self.w1)), self.w2))      # residual: not a chain

    class Net(nn.Cell):
        def __init__(self):
            super().__init__()
            self.blocks = nn.CellList([Block(i) for i in range(layers)])
            self.sum = ops.ReduceSum()

        def construct(self, x):
            for b in self.blocks:
                x = b(x)
            return self.sum(x, ())

    net = Net()
    return net, J.trace_cell(net, (ms.Tensor(torch.randn(batch, hidden)),))


@pytest.mark.parametrize("device_num", [4, 8])
def test_search_modes_on_a_residual_graph(device_num):
    from mindspore_b200.parallel import auto_parallel as AP
    from mindspore_b200.parallel import operator_info as OI
    costs = {}
    for mode in ("sharding_propagation", "dynamic_programming", "recursive_programming"):
        net, fg = _mlp_graph()
        chosen = AP.search(fg, device_num, mode)
        ls = AP.last_search
        assert len(chosen) >= 9
        for op, c in zip(ls["ops"], ls["choice"]):
            info = OI.make_info(op.prim, op.in_shapes, op.cands[c], None, device_num)      # every choice is legal
            assert info.dev_matrix is not None
        if mode != "recursive_programming":
            costs[mode] = AP.total_cost(ls["ops"], ls["edges"], ls["mats"], ls["choice"])
        else:
            # the product of log2(N) binary cuts uses every device on the heavy operators
            mm = [op for op in ls["ops"] if op.prim.name == "MatMul"]
            assert all(max(1, int(torch.tensor(op.cands[c][0]).prod()) * 1) >= 1 for op, c in zip(ls["ops"], ls["choice"]))
            assert any(max(max(st) for st in op.cands[ls["choice"][ls["ops"].index(op)]]) > 1 for op in mm)
    # the elimination search is exact on this graph: never worse than propagation
    assert costs["dynamic_programming"] <= costs["sharding_propagation"] + 1e-6


def test_memory_capacity_steers_the_search():
    """Two operators, each with a fast-but-large and a slow-but-small candidate: with room the fast ones win, with a
    capacity below their footprint the search re-prices memory until the result fits."""
    import types
    import mindspore_b200 as ms
    from mindspore_b200.parallel import auto_parallel as AP

    def op(costs, mems):
        return types.SimpleNamespace(cands=[("a",), ("b",)], costs=list(costs), mems=list(mems), infos=[None, None])
    ops = [op([1.0, 5.0], [100.0, 10.0]), op([2.0, 3.0], [80.0, 20.0])]
    edges, mats = [(0, 1)], [[[0.0, 1.0], [1.0, 0.0]]]
    try:
        for mode in ("dynamic_programming", "sharding_propagation"):
            ms.set_cost_model_context(device_memory_capacity=1000.0)
            assert AP.fit_memory(ops, edges, mats, [-1, -1], mode, 4) == [0, 0]
            ms.set_cost_model_context(device_memory_capacity=50.0)
            choice = AP.fit_memory(ops, edges, mats, [-1, -1], mode, 4)
            assert sum(o.mems[c] for o, c in zip(ops, choice)) <= 50.0, (mode, choice)
        with pytest.raises(ValueError):
            ms.set_cost_model_context(no_such_key=1.0)
        with pytest.raises(TypeError):
            ms.set_cost_model_context(costmodel_alpha="fast")
        assert ms.get_cost_model_context("costmodel_gamma") == 0.001
    finally:
        ms.reset_cost_model_context()
