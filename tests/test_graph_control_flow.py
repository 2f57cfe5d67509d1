"""Graph mode keeps what depends on run-time values out of the trace: ``cond`` records a Switch whose branch is
chosen at every replay, the loss-scale cell's ``if not overflow`` becomes a predicated update, and the optimizer's
learning-rate schedule / Adam bias correction are computed from ``global_step`` by graph nodes.
Reference cases: python/mindspore/nn/wrap/loss_scale.py:404-422; tests/st/control/ (if / while in graph mode)."""
import pytest
import torch

import mindspore_b200 as ms
from mindspore_b200 import nn, ops
from mindspore_b200.graph.control_flow import Switch, cond


def test_cond_records_one_switch_and_replays_both_ways():
    ms.set_context(mode=ms.GRAPH_MODE, device_target="CPU")

    class Net(nn.Cell):
        def __init__(self):
            super().__init__()
            self.w = ms.Parameter(ms.Tensor(torch.tensor([1.0, 2.0, 3.0])), name="w")

        def construct(self, x):
            y = x * self.w
            return cond(y.sum() > 0, lambda a: a * 2 + y, lambda a: a - 1, x)

    net = Net()
    pos, neg = ms.Tensor(torch.ones(3)), ms.Tensor(-torch.ones(3))
    assert torch.allclose(net(pos), torch.tensor([3.0, 4.0, 5.0]))
    assert torch.allclose(net(neg), torch.tensor([-2.0, -2.0, -2.0]))       # same compiled graph, other branch
    assert torch.allclose(net(pos), torch.tensor([3.0, 4.0, 5.0]))
    (cg,) = net._compiled.values()
    switches = [n for n in cg.fg.graph.nodes if n.op == "call_function" and isinstance(n.target, Switch)]
    assert len(switches) == 1 and len(net._compiled) == 1
    # gradients flow through whichever branch ran
    g = ops.GradOperation(get_by_list=True)(net, ms.ParameterTuple([net.w]))
    ms.set_context(mode=ms.PYNATIVE_MODE)
    (gw,) = g(pos)
    assert torch.allclose(gw, torch.ones(3))             # d/dw sum(2x + x*w) = x


def _lenet_step(mode, dtype=torch.float32):
    ms.set_context(mode=mode, device_target="CPU")
    ms.set_seed(3)
    from mindspore_b200.models.lenet import LeNet5
    net = LeNet5()
    loss = nn.SoftmaxCrossEntropyWithLogits(sparse=True, reduction="mean")
    opt = nn.Momentum(net.trainable_params(), learning_rate=0.05, momentum=0.9)
    step = nn.TrainOneStepWithLossScaleCell(nn.WithLossCell(net, loss), opt,
                                            nn.DynamicLossScaleUpdateCell(2.0 ** 10, 2.0, 3))
    step.set_train()
    return net, step, opt


def _batches():
    g = torch.Generator().manual_seed(0)
    out = []
    for i in range(7):
        x = torch.randn(8, 1, 32, 32, generator=g)
        if i == 2:
            x[0, 0, 0, 0] = float("inf")              # one overflow step in the middle
        out.append((ms.Tensor(x), ms.Tensor(torch.randint(0, 10, (8,), generator=g).to(torch.int32))))
    return out


def test_lenet_dynamic_loss_scale_through_an_overflow_step_in_graph_mode():
    ref_net, ref_step, ref_opt = _lenet_step(ms.PYNATIVE_MODE)
    ref = []
    for x, y in _batches():
        l, ov, sc = ref_step(x, y)
        ref.append((float(l) if torch.isfinite(l) else None, bool(ov), float(ref_step.scale_sense)))
    net, step, opt = _lenet_step(ms.GRAPH_MODE)
    got = []
    for x, y in _batches():
        l, ov, sc = step(x, y)
        got.append((float(l) if torch.isfinite(l) else None, bool(ov), float(step.scale_sense)))
    assert len(step._compiled) == 1, "the step must be one graph, not one per branch outcome"
    assert [g[1] for g in got] == [r[1] for r in ref] == [False, False, True, False, False, False, False]
    assert [g[2] for g in got] == [r[2] for r in ref]           # halved at the overflow, doubled after 3 clean steps
    for g, r in zip(got, ref):
        if r[0] is not None:
            assert g[0] == pytest.approx(r[0], rel=1e-5)
    for p, q in zip(net.get_parameters(), ref_net.get_parameters()):
        torch.testing.assert_close(p.detach(), q.detach(), rtol=1e-5, atol=1e-6)
    assert int(opt.global_step) == int(ref_opt.global_step) == 6          # the skipped step does not count
    ms.set_context(mode=ms.PYNATIVE_MODE)


@pytest.mark.parametrize("optim", ["adam", "adamw", "sgd"])
def test_schedule_and_bias_correction_follow_global_step_in_graph_mode(optim):
    def run(mode):
        ms.set_context(mode=mode, device_target="CPU")
        ms.set_seed(5)
        net = nn.SequentialCell([nn.Dense(6, 8), nn.Tanh(), nn.Dense(8, 3)])
        lr = nn.ExponentialDecayLR(0.1, 0.5, 2)
        if optim == "sgd":
            opt = nn.SGD(net.trainable_params(), learning_rate=lr, momentum=0.9)
        elif optim == "adam":
            opt = nn.Adam(net.trainable_params(), learning_rate=lr)
        else:
            opt = nn.AdamWeightDecay(net.trainable_params(), learning_rate=lr, weight_decay=0.01, use_arena=False,
                                     bias_correction=True)
        step = nn.TrainOneStepCell(nn.WithLossCell(net, nn.MSELoss()), opt)
        step.set_train()
        g = torch.Generator().manual_seed(1)
        losses = []
        for _ in range(6):
            x, y = torch.randn(4, 6, generator=g), torch.randn(4, 3, generator=g)
            losses.append(float(step(ms.Tensor(x), ms.Tensor(y))))
        return losses, [p.detach().clone() for p in net.get_parameters()]
    ref_losses, ref_params = run(ms.PYNATIVE_MODE)
    losses, params = run(ms.GRAPH_MODE)
    ms.set_context(mode=ms.PYNATIVE_MODE)
    # graph mode evaluates beta ** t and the schedule in fp32 tensors, eager mode in host doubles
    assert losses == pytest.approx(ref_losses, rel=2e-4)
    for p, q in zip(params, ref_params):
        torch.testing.assert_close(p, q, rtol=5e-4, atol=1e-5)
