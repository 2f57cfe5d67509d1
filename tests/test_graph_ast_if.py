"""Graph mode: plain Python ``if`` / ``elif`` / ``else`` on tensor values in ``construct`` and in ``@ms.jit``
functions are rewritten from the source into Switch sub-graphs, so one compiled graph serves every outcome and
differentiates through the branch that ran."""
import warnings

import pytest
import torch

import mindspore_b200 as ms
from mindspore_b200 import nn, ops
from mindspore_b200.graph import ast_transform


class Branchy(nn.Cell):
    def __init__(self):
        super().__init__()
        self.w = ms.Parameter(ms.Tensor(torch.tensor([2.0, 3.0])), name="w")

    def construct(self, x, flag=True):
        s = (x * self.w).sum()
        if flag:                      # a Python value: stays a Python branch
            s = s + 0.0
        if s > 0:
            y = x * 2
            z = s
        elif s < -10:
            y = x * 0
            z = s * 0
        else:
            y = x - 1
            z = -s
        return y + z


def _ref(x):
    s = (x * torch.tensor([2.0, 3.0])).sum()
    if s > 0:
        return x * 2 + s
    if s < -10:
        return x * 0 + s * 0
    return x - 1 - s


@pytest.fixture
def graph_mode():
    ms.set_context(mode=ms.GRAPH_MODE, device_target="CPU")
    yield
    ms.set_context(mode=ms.PYNATIVE_MODE)


def test_if_elif_else_on_tensors_compiles_to_one_graph(graph_mode):
    net = Branchy()
    xs = [torch.tensor([1.0, 1.0]), torch.tensor([-1.0, -0.5]), torch.tensor([-4.0, -3.0])]
    for x in xs:
        torch.testing.assert_close(net(ms.Tensor(x)).as_subclass(torch.Tensor), _ref(x))
    assert len(net._compiled) == 1
    (cg,) = net._compiled.values()
    names = [getattr(n.target, "__name__", getattr(n.target, "name", "")) for n in cg.fg.graph.nodes
             if n.op == "call_function"]
    assert names.count("Switch") == 1                      # the elif lives inside the false sub-graph
    grad = ops.GradOperation(get_by_list=True)(net, ms.ParameterTuple([net.w]))
    for x in xs:
        w = torch.tensor([2.0, 3.0], requires_grad=True)
        s = (x * w).sum()
        ref = (x * 2 + s) if s > 0 else ((x * 0 + s * 0) if s < -10 else (x - 1 - s))
        ref.sum().backward()
        (g,) = grad(ms.Tensor(x))
        torch.testing.assert_close(g.as_subclass(torch.Tensor), w.grad)


def test_jit_function_with_augmented_assignment_in_a_branch(graph_mode):
    @ms.jit
    def step(x, limit):
        total = x.sum()
        scale = x * 0 + 1.0
        if total > limit:
            scale = scale * 0.5
            total -= limit
        return x * scale, total

    for vals in ([1.0, 2.0], [10.0, 20.0]):
        x = torch.tensor(vals)
        y, t = step(ms.Tensor(x), ms.Tensor(torch.tensor(5.0)))
        big = x.sum() > 5
        torch.testing.assert_close(y.as_subclass(torch.Tensor), x * (0.5 if big else 1.0))
        assert float(t) == pytest.approx(float(x.sum() - 5 if big else x.sum()))
    assert len(step.__jit_cache__) == 1


def test_unconvertible_branches_are_left_alone():
    def early(x):
        if x.sum() > 0:
            return x
        return -x

    def attr(self, x):
        if x.sum() > 0:
            self.seen = x
        return x

    assert ast_transform.convert_function(early) is early          # a return inside the branch
    assert ast_transform.convert_function(attr) is attr            # assignment to an attribute
    # eager calls of a rewritten function behave like the original
    f = ast_transform.convert_function(Branchy.construct)
    assert f is not Branchy.construct
    net = Branchy()
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        for x in (torch.tensor([1.0, 1.0]), torch.tensor([-1.0, -0.5])):
            torch.testing.assert_close(f(net, ms.Tensor(x)).as_subclass(torch.Tensor), _ref(x))


def test_zero_argument_super_still_works_after_the_rewrite(graph_mode):
    class Base(nn.Cell):
        def construct(self, x):
            return x + 1

    class Child(Base):
        def construct(self, x):
            y = super().construct(x)
            if y.sum() > 0:
                y = y * 3
            return y

    net = Child()
    assert net(ms.Tensor(torch.tensor([1.0]))).tolist() == [6.0]
    assert net(ms.Tensor(torch.tensor([-5.0]))).tolist() == [-4.0]
    assert len(net._compiled) == 1


def test_while_on_a_tensor_condition_is_one_node_with_a_dynamic_trip_count(graph_mode):
    class Halve(nn.Cell):
        def __init__(self):
            super().__init__()
            self.w = ms.Parameter(ms.Tensor(torch.tensor(1.5)), name="w")

        def construct(self, x, limit):
            n = x * 0
            y = x * self.w
            while y.sum() > limit:
                y = y * 0.5
                n = n + 1
            return y, n

    net = Halve()
    lim = ms.Tensor(torch.tensor(1.0))
    for vals, trips in (([8.0, 8.0], 5), ([0.25, 0.25], 0), ([1.0, 1.0], 2)):
        y, n = net(ms.Tensor(torch.tensor(vals)), lim)
        assert n.tolist() == [float(trips)] * 2, (vals, n.tolist())
        torch.testing.assert_close(y.as_subclass(torch.Tensor), torch.tensor(vals) * 1.5 * 0.5 ** trips)
    assert len(net._compiled) == 1
    (cg,) = net._compiled.values()
    names = [getattr(n.target, "__name__", "") for n in cg.fg.graph.nodes if n.op == "call_function"]
    assert names.count("While") == 1
    # reverse mode goes through the iterations that ran: d(sum y)/dw = sum(x) * 0.5^trips
    grad = ops.GradOperation(get_by_list=True)(lambda x, l: net(x, l)[0], ms.ParameterTuple([net.w]))
    (g,) = grad(ms.Tensor(torch.tensor([8.0, 8.0])), lim)
    assert float(g) == pytest.approx(16.0 * 0.5 ** 5)


def test_loop_functions():
    ms.set_context(mode=ms.PYNATIVE_MODE, device_target="CPU")
    s = ops.while_loop(lambda i, acc: i < 5, lambda i, acc: (i + 1, acc + i), (ms.Tensor(torch.tensor(0)),
                                                                                ms.Tensor(torch.tensor(0))))
    assert [int(v) for v in s] == [5, 10]
    assert float(ops.fori_loop(0, 4, lambda i, v: v * 2, ms.Tensor(torch.tensor(1.0)))) == 16.0
    out = ops.fori_loop(ms.Tensor(torch.tensor(2)), ms.Tensor(torch.tensor(5)), lambda i, v: v + i,
                        ms.Tensor(torch.tensor(0)))
    assert int(out) == 2 + 3 + 4
    carry, ys = ops.scan(lambda c, x: (c + x, c * x), ms.Tensor(torch.tensor(0.0)), ms.Tensor(torch.arange(4.0)))
    assert float(carry) == 6.0 and ys.tolist() == [0.0, 0.0, 2.0, 9.0]
