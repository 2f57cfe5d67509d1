"""rewrite.SymbolTree: parse a construct into nodes, edit, regenerate an equivalent / modified network."""
import numpy as np
import torch

import mindspore_b200 as ms
from mindspore_b200 import nn, ops
from mindspore_b200.rewrite import Node, NodeType, ScopedValue, SymbolTree


class Net(nn.Cell):
    def __init__(self):
        super().__init__()
        self.fc1 = nn.Dense(4, 8)
        self.act = nn.ReLU()
        self.fc2 = nn.Dense(8, 2)
        self.scale = 2.0

    def construct(self, x):
        h = self.fc1(x)
        h = self.act(h)
        y = self.fc2(h)
        y = y * self.scale
        return y


class Nested(nn.Cell):
    def __init__(self):
        super().__init__()
        self.a = nn.Dense(3, 3)
        self.b = nn.Tanh()

    def construct(self, x, y):
        return self.b(self.a(x)) + y


def test_round_trip_is_equivalent():
    ms.set_seed(0)
    net = Net()
    st = SymbolTree.create(net)
    kinds = [n.get_node_type() for n in st.nodes()]
    assert kinds == [NodeType.Input, NodeType.CallCell, NodeType.CallCell, NodeType.CallCell, NodeType.MathOps,
                     NodeType.Output]
    new = st.get_network()
    x = ms.Tensor(torch.randn(5, 4))
    np.testing.assert_allclose(new(x).detach().numpy(), net(x).detach().numpy())
    assert {p.name for p in new.trainable_params()} == {p.name for p in net.trainable_params()}
    assert new.fc1.weight is net.fc1.weight


def test_replace_and_insert():
    ms.set_seed(1)
    net = Net()
    st = SymbolTree.create(net)
    relu = st.get_node("act")
    assert relu.get_instance_type() is nn.ReLU and [u.get_name() for u in relu.get_users()] == ["fc2"]
    gelu = Node.create_call_cell(nn.GELU(), targets=relu.get_targets(), args=relu.get_args(), name="gelu")
    st.replace(relu, [gelu])
    drop = Node.create_call_cell(nn.Dropout(p=0.0), targets=["h"], args=["h"], name="drop")
    st.insert(st.after(gelu), drop)
    new = st.get_network()
    assert "self.gelu(h)" in st.get_code() and "self.drop(h)" in st.get_code() and "self.act" not in st.get_code()
    x = ms.Tensor(torch.randn(3, 4))
    ref = net.fc2(nn.GELU()(net.fc1(x))) * 2.0
    np.testing.assert_allclose(new(x).detach().numpy(), ref.detach().numpy(), rtol=1e-5, atol=1e-6)
    assert isinstance(new.gelu, nn.GELU)


def test_nested_calls_are_flattened_and_erase_checks_users():
    net = Nested()
    st = SymbolTree.create(net)
    names = [n.get_name() for n in st.nodes()]
    assert names[:2] == ["x", "y"] and "a" in names and "b" in names
    a = st.get_node("a")
    try:
        st.erase(a)
        raise AssertionError("erase of a used node must fail")
    except RuntimeError:
        pass
    x, y = ms.Tensor(torch.randn(2, 3)), ms.Tensor(torch.randn(2, 3))
    np.testing.assert_allclose(st.get_network()(x, y).detach().numpy(), net(x, y).detach().numpy(), rtol=1e-6)
    # route around `b`: the output add reads a's result directly
    b = st.get_node("b")
    for user in b.get_users():
        pass
    out = [n for n in st.nodes() if n.get_node_type() is NodeType.Output][0]
    assert out.get_args()[0].type.name == "NamingValue"


def test_set_arg_rewires_a_node():
    net = Net()
    st = SymbolTree.create(net)
    fc2 = st.get_node("fc2")
    fc2.set_arg_by_node(0, st.get_node("fc1"))           # skip the activation
    st.erase(st.get_node("act"))
    x = ms.Tensor(torch.randn(2, 4))
    ref = net.fc2(net.fc1(x)) * 2.0
    np.testing.assert_allclose(st.get_network()(x).detach().numpy(), ref.detach().numpy(), rtol=1e-6)
    assert ScopedValue.create_naming_value("h").code() == "h"


def test_pattern_engine_replaces_a_chain():
    from mindspore_b200.rewrite import PatternEngine, PatternNode, Replacement, VarNode

    class DenseRelu(nn.Cell):
        def __init__(self, dense):
            super().__init__()
            self.dense = dense

        def construct(self, x):
            return ops.relu(self.dense(x))

    class Fuse(Replacement):
        def build(self, pattern, is_chain_pattern, matched):
            assert is_chain_pattern
            dense, relu = matched["pattern_0"], matched["pattern_1"]
            return [Node.create_call_cell(DenseRelu(dense.get_instance()), targets=relu.get_targets(),
                                          args=dense.get_args(), name="dense_relu")]

    ms.set_seed(3)
    net = Net()
    st = SymbolTree.create(net)
    assert PatternEngine([nn.Dense, nn.ReLU], Fuse()).apply(st)
    names = [n.get_name() for n in st.nodes()]
    assert "dense_relu" in names and "fc1" not in names and "act" not in names and "fc2" in names
    new = st.get_network()
    x = ms.Tensor(torch.randn(5, 4))
    np.testing.assert_allclose(new(x).detach().numpy(), net(x).detach().numpy(), rtol=1e-6)
    # a pattern that is not there changes nothing; a tree pattern with a wildcard input matches the first Dense
    assert not PatternEngine([nn.Tanh, nn.Dense], Fuse()).apply(SymbolTree.create(net))
    pat = PatternNode("d", nn.Dense, [VarNode()])
    m = {}
    assert PatternEngine(pat)._match(pat, SymbolTree.create(net).get_node("fc1"), m) and list(m) == ["d"]
