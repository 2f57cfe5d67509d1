"""Graph passes: cast / arithmetic simplification keeps results and gradients, duplicate collectives merge,
gradient all-reduces are bucketed by the comm_fusion threshold, collectives are hoisted without crossing effect
chains, the executor reports a memory plan, and GRAPH_MODE data-parallel training all-reduces at every replay.
Reference passes: frontend/optimizer/irpass/{arithmetic_simplify,cast_eliminate}.cc, frontend/parallel/pass/
merge_comm.cc, allreduce_fusion/allreduce_fusion.cc, pass/overlap_grad_comm.cc."""
import os

import pytest
import torch

import mindspore_b200 as ms
from mindspore_b200 import nn, ops
from mindspore_b200.graph import jit as J
from mindspore_b200.graph import opt_passes as O
from mindspore_b200.graph.passes import run_default_passes

from _mp import run_ranks


def _names(fg):
    out = []
    for n in fg.graph.nodes:
        if n.op == "call_function":
            out.append(getattr(n.target, "name", None) or getattr(n.target, "__name__", "?"))
    return out


def test_simplification_keeps_values_and_gradients(tmp_path):
    ms.set_context(mode=ms.GRAPH_MODE, device_target="CPU", save_graphs=2, save_graphs_path=str(tmp_path))

    class Net(nn.Cell):
        def __init__(self):
            super().__init__()
            self.w = ms.Parameter(ms.Tensor(torch.randn(4, 4, generator=torch.Generator().manual_seed(0))), name="w")
            self.cast, self.mul, self.add, self.neg = ops.Cast(), ops.Mul(), ops.Add(), ops.Neg()
            self.tr, self.mm, self.sum = ops.Transpose(), ops.MatMul(), ops.ReduceSum()

        def construct(self, x):
            a = self.cast(self.cast(x, ms.float32), ms.float32)          # cast to the same dtype, twice
            a = self.add(self.mul(a, 1.0), 0.0)                          # * 1, + 0
            a = self.neg(self.neg(a))                                    # double negation
            a = self.tr(self.tr(a, (1, 0)), (1, 0))                      # transpose of a transpose
            return self.sum(self.mm(a, self.w), ())

    net = Net()
    grad = ops.GradOperation(get_by_list=True)(net, ms.ParameterTuple([net.w]))
    x = ms.Tensor(torch.randn(3, 4, generator=torch.Generator().manual_seed(1)))
    out = float(net(x))
    assert out == pytest.approx(float((x @ net.w.detach()).sum()), rel=1e-5)
    (cg,) = net._compiled.values()
    names = _names(cg.fg)
    assert "Cast" not in names and "Neg" not in names and "Transpose" not in names and "Mul" not in names, names
    assert os.path.isfile(tmp_path / "Net_01_cast_eliminate.ir") and os.path.isfile(tmp_path / "Net_memory_plan.txt")
    rep = cg.memory_report()
    assert rep["tensors"] >= 1 and 0 < rep["arena_bytes"] <= rep["sum_bytes"] + 512 * rep["tensors"]

    @ms.jit
    def g(x):
        return grad(x)
    (gw,) = g(x)
    torch.testing.assert_close(gw, x.sum(0)[:, None].expand(4, 4).contiguous(), rtol=1e-5, atol=1e-6)
    ms.set_context(mode=ms.PYNATIVE_MODE, save_graphs=0)


def _comm_graph(world=1):
    """A hand-built graph: two all-gathers of the same value, compute, and three in-place gradient all-reduces."""
    import torch.fx as fx
    from mindspore_b200.communication import comm_func as CF
    from mindspore_b200.graph.ir import FuncGraph
    fg = FuncGraph("comm")
    g = fg.graph
    x = g.placeholder("x")
    x.meta.update(shape=(4, 8), dtype=torch.float32)
    a = g.call_function(torch.tanh, (x,))
    b = g.call_function(torch.sigmoid, (a,))
    ag1 = g.call_function(CF.all_gather_node, (x, "grp"))
    ag2 = g.call_function(CF.all_gather_node, (x, "grp"))
    c = g.call_function(torch.add, (ag1, ag2))
    grads = []
    for i in range(3):
        gi = g.call_function(torch.mul, (b, float(i + 1)))
        gi.meta.update(shape=(4, 8), dtype=torch.float32)
        grads.append(g.call_function(CF.all_reduce_node, (gi, "sum", "grp")))
    for n in (a, b, ag1, ag2, c):
        n.meta.update(shape=(4, 8), dtype=torch.float32)
    fg.set_output((c,) + tuple(grads), None)
    return fg


def test_merge_comm_fusion_and_hoisting_on_a_graph():
    fg = _comm_graph()
    assert O.merge_comm(fg) == 1
    assert _names(fg).count("all_gather_node") == 1
    assert O.allreduce_fusion(fg, threshold_bytes=2 * 4 * 8 * 4) == 1        # two of the three fit one bucket
    names = _names(fg)
    assert names.count("fused_all_reduce") == 1 and names.count("all_reduce_node") == 1
    fused = next(n for n in fg.graph.nodes if n.op == "call_function" and n.target is O.fused_all_reduce)
    assert fused.meta["fusion"] == 1 and len(fused.args) == 3 + 2
    # the all-gather only needs x: it moves up in front of the tanh / sigmoid chain, and runs on the comm stream
    moved = O.comm_reorder(fg)
    order = _names(fg)
    assert moved >= 1 and order.index("all_gather_node") < order.index("tanh")
    assert O.mark_comm_stream(fg) >= 1
    ag = next(n for n in fg.graph.nodes if getattr(n.target, "__name__", "") == "all_gather_node")
    assert ag.meta.get("comm_stream") and ag.meta.get("hoisted")
    # collectives keep their relative order (one chain)
    chain = [n for n in fg.graph.nodes if O.is_collective(n)]
    pred = O.effect_chains(fg)
    for earlier, later in zip(chain, chain[1:]):
        assert earlier in pred[later]
    fg.graph.lint()


def test_effect_chain_orders_reads_after_writes():
    """Reads of a parameter that follow a write are chained behind it; a snapshot ``p * 1`` taken before a write is
    not folded into the parameter (its later readers would see the write)."""
    from mindspore_b200.graph.ir import FuncGraph
    fg = FuncGraph("effects")
    g = fg.graph
    x = g.placeholder("x")
    x.meta.update(shape=(), dtype=torch.float32)
    c = ms.Parameter(ms.Tensor(torch.zeros(())), name="c", requires_grad=False)
    pc = fg.param_node(c)
    pc.meta.update(shape=(), dtype=torch.float32)
    snap = g.call_function(torch.mul, (pc, 1.0))
    snap.meta.update(shape=(), dtype=torch.float32)
    write = g.call_function(ops.AssignAdd(), (pc, x))
    read = g.call_function(torch.add, (pc, 0.5))
    fg.set_output((snap, read), None)
    pred = O.effect_chains(fg)
    assert pred[read] == [write] and read.meta["after"] == [write.name]
    assert O.arithmetic_simplify(fg) == 0 and snap in list(fg.graph.nodes)
    # end to end: a counter cell keeps counting across replays of one compiled graph
    ms.set_context(mode=ms.GRAPH_MODE, device_target="CPU")

    class Counter(nn.Cell):
        def __init__(self):
            super().__init__()
            self.c = ms.Parameter(ms.Tensor(torch.zeros(())), name="c", requires_grad=False)
            self.assign_add = ops.AssignAdd()

        def construct(self, x):
            before = self.c * 1.0 + x
            self.assign_add(self.c, x)
            return before, self.c * 1.0

    net = Counter()
    outs = [tuple(float(v) for v in net(ms.Tensor(torch.tensor(2.0)))) for _ in range(3)]
    assert outs == [(2.0, 2.0), (4.0, 4.0), (6.0, 6.0)] and len(net._compiled) == 1
    ms.set_context(mode=ms.PYNATIVE_MODE)


def _dp_worker(rank, world, mode):
    import mindspore_b200 as ms
    from mindspore_b200 import nn
    from mindspore_b200.communication import init
    ms.set_context(device_target="CPU", mode=ms.GRAPH_MODE if mode == "graph" else ms.PYNATIVE_MODE)
    init("mccl")
    ms.set_auto_parallel_context(parallel_mode="data_parallel", gradients_mean=True, device_num=world)
    ms.set_seed(9)
    net = nn.SequentialCell([nn.Dense(6, 16), nn.Tanh(), nn.Dense(16, 3)])
    opt = nn.Momentum(net.trainable_params(), learning_rate=0.1, momentum=0.9)
    step = nn.TrainOneStepCell(nn.WithLossCell(net, nn.MSELoss()), opt)
    step.set_train()
    g = torch.Generator().manual_seed(100 + rank)            # every rank sees different data
    for _ in range(4):
        step(ms.Tensor(torch.randn(8, 6, generator=g)), ms.Tensor(torch.randn(8, 3, generator=g)))
    n_comm = 0
    if mode == "graph":
        (cg,) = step._compiled.values()
        n_comm = sum(1 for n in cg.fg.graph.nodes if O.is_collective(n))
    torch.distributed.barrier()
    return [p.detach().clone() for p in net.get_parameters()], n_comm


def test_graph_mode_data_parallel_all_reduces_on_every_replay():
    eager = run_ranks(_dp_worker, 2, "eager")
    graph = run_ranks(_dp_worker, 2, "graph")
    for (pe, _), (pg, n_comm) in zip(eager, graph):
        assert n_comm >= 1, "the traced step holds no collective node"
        for a, b in zip(pe, pg):
            torch.testing.assert_close(a, b, rtol=1e-5, atol=1e-6)
    for a, b in zip(graph[0][0], graph[1][0]):               # replicas stay identical
        torch.testing.assert_close(a, b, rtol=0, atol=0)


def test_pattern_fusion_keeps_training_results():
    """Reference-style small operators (Add + RmsNorm, Split + SiLU * up, MatMul + BiasAdd + GeLU) train to the same
    parameters in graph mode, where they are rewritten to the fused primitives, as eagerly."""
    def run(mode):
        ms.set_context(mode=mode, device_target="CPU")
        ms.set_seed(4)

        class Block(nn.Cell):
            def __init__(self):
                super().__init__()
                g = torch.Generator().manual_seed(2)
                self.gamma = ms.Parameter(ms.Tensor(torch.rand(16, generator=g) + 0.5), name="gamma")
                self.w_gu = ms.Parameter(ms.Tensor(torch.randn(64, 16, generator=g) * 0.2), name="w_gu")
                self.w_d = ms.Parameter(ms.Tensor(torch.randn(16, 32, generator=g) * 0.2), name="w_d")
                self.b_d = ms.Parameter(ms.Tensor(torch.randn(16, generator=g) * 0.1), name="b_d")
                self.b_gu = ms.Parameter(ms.Tensor(torch.randn(64, generator=g) * 0.1), name="b_gu")
                self.bias_gu = ops.BiasAdd()
                self.add, self.norm = ops.Add(), ops.RmsNorm(1e-5)
                self.mm1, self.mm2 = ops.MatMul(transpose_b=True), ops.MatMul(transpose_b=True)
                self.split, self.silu, self.mul = ops.Split(axis=-1, output_num=2), ops.SiLU(), ops.Mul()
                self.bias, self.gelu, self.sum = ops.BiasAdd(), ops.GeLU(), ops.ReduceSum()

            def construct(self, x, r):
                s = self.add(x, r)
                h = self.norm(s, self.gamma)[0]
                gate, up = self.split(self.bias_gu(self.mm1(h, self.w_gu), self.b_gu))
                y = self.gelu(self.bias(self.mm2(self.mul(self.silu(gate), up), self.w_d), self.b_d))
                return self.sum((y + s) * (y + s), ())

        net = Block()
        opt = nn.Momentum(net.trainable_params(), learning_rate=0.01, momentum=0.9)
        step = nn.TrainOneStepCell(net, opt)
        step.set_train()
        g = torch.Generator().manual_seed(7)
        losses = [float(step(ms.Tensor(torch.randn(8, 16, generator=g)), ms.Tensor(torch.randn(8, 16, generator=g))))
                  for _ in range(4)]
        names = []
        if mode == ms.GRAPH_MODE:
            (cg,) = step._compiled.values()
            names = _names(cg.fg)
        return losses, [p.detach().clone() for p in net.get_parameters()], names
    ref_l, ref_p, _ = run(ms.PYNATIVE_MODE)
    l, p, names = run(ms.GRAPH_MODE)
    ms.set_context(mode=ms.PYNATIVE_MODE)
    assert "AddRmsNorm" in names and "SwiGLU" in names and "RmsNorm" not in names and "SiLU" not in names, names
    assert "gelu_tanh" in names and "linear" in names and "BiasAdd" not in names, names
    assert l == pytest.approx(ref_l, rel=1e-5)
    for a, b in zip(p, ref_p):
        torch.testing.assert_close(a, b, rtol=1e-5, atol=1e-6)
