"""Shape / dtype inference on abstract values: symbolic dimensions, constraints, signatures, graph annotation."""
import numpy as np
import pytest
import torch

import mindspore_b200 as ms
from mindspore_b200 import Symbol, Tensor, nn, ops
from mindspore_b200.graph import abstract as A
from mindspore_b200.ops.primitive import PrimitiveWithInfer

f32 = torch.float32
T = A.AbstractTensor


def test_symbolic_dimensions_flow_through_primitives():
    out, cons = A.infer_with_constraints(ops.MatMul(), T((None, 8), f32), T((8, None), f32))
    assert repr(out) == "Tensor[float32](s0, s1)" and cons == [] and out.shape_list == [-1, -1]
    out, cons = A.infer_with_constraints(ops.Add(), T((None, 8), f32), T((None, 8), f32))
    assert repr(out) == "Tensor[float32](s0, 8)" and cons == [("s0", "s1")]
    # two independent pairs of equal dimensions come apart
    out, cons = A.infer_with_constraints(lambda a, b, c, d: (a + b, c * d), T((None, 8), f32), T((None, 8), f32),
                                         T((None,), f32), T((None,), f32))
    assert cons == [("s0", "s1"), ("s2", "s3")] and repr(out) == "(Tensor[float32](s0, 8), Tensor[float32](s2))"
    assert repr(A.infer(lambda x: ops.Concat(0)((x, x)), T((None, 3), f32))) == "Tensor[float32](2*s0, 3)"
    shape = A.infer(lambda x: x.shape, T((None, 3), f32))
    assert repr(shape) == "(int(s0), int(3))"
    # a floor division is not affine: the dimension is reported unknown
    conv = A.infer(ops.Conv2D(8, 3, stride=2), T((None, 3, None, None), f32), T((8, 3, 3, 3), f32))
    assert conv.shape_list == [-1, 8, -1, -1] and conv.shape[2] is None and repr(conv.shape[0]) == "s0"
    assert A.infer(ops.Cast(), T((4, None), f32), torch.int32).dtype == torch.int32
    with pytest.raises(A.InferenceError):
        A.infer(ops.MatMul(), T((None, 8), f32), T((7, None), f32))


def test_symbol_ranges_and_divisors_carry_over():
    s = Symbol(divisor=8, min=8, max=64)
    out = A.infer(lambda x: ops.Reshape()(x, (x.shape[0] // 2, -1)), T((s, 6), f32))
    assert repr(out) == "Tensor[float32](s0/2, 12)"
    sym = out.shape[0].to_symbol()
    assert (sym.min, sym.max, sym.divisor, sym.remainder) == (4, 32, 4, 0)
    assert out.shape[0].evaluate({next(iter(out.shape[0].coeffs)): 16}) == 8
    odd = A.infer(lambda x: ops.Concat(0)((x, x, x[:1])), T((Symbol(divisor=4, remainder=1),), f32))
    assert repr(odd.shape[0]) == "2*s0+1" and odd.shape[0].divisor_remainder() == (8, 3)
    # one unique symbol used twice is one dimension; two plain None dimensions are two
    u = Symbol(unique=True)
    out, cons = A.infer_with_constraints(ops.Add(), T((u, 4), f32), T((u, 4), f32))
    assert cons == [] and repr(out) == "Tensor[float32](s0, 4)"


def test_dynamic_rank_and_joins():
    assert A.infer(ops.ReLU(), T(None, f32)).shape_list == [-2]
    assert A.infer(ops.ReduceSum(), T(None, f32)).shape_list == []
    a, b = T((2, 3), f32), T((2, 5), f32)
    assert a.join(b).shape_list == [2, -1] and a.join(T((2, 3, 1), f32)).shape is None
    with pytest.raises(A.InferenceError):
        a.join(T((2, 3), torch.int32))
    one, two = A.AbstractScalar(int, 1), A.AbstractScalar(int, 2)
    assert one.join(one).value == 1 and one.join(two).value is None
    seq = A.to_abstract((1, Tensor(np.zeros((2, 2), np.float32)), None))
    assert repr(seq) == "(int(1), Tensor[float32](2, 2), None)" and seq.broaden()[0].value is None


def test_placeholder_tensors_and_signature_check():
    spec = Tensor(shape=[None, 8], dtype=ms.float32)
    assert spec.symbolic_shape == (None, 8) and spec.device.type == "meta"
    assert A.to_abstract(spec).shape_list == [-1, 8]
    assert A.to_abstract(Tensor(shape=None, dtype=ms.float32)).shape_list == [-2]
    good = Tensor(np.zeros((5, 8), np.float32))
    A.check_signature([spec], [good])
    with pytest.raises(ValueError, match="dimension 1 must be 8"):
        A.check_signature([spec], [Tensor(np.zeros((5, 7), np.float32))])
    with pytest.raises(TypeError, match="dtype"):
        A.check_signature([spec], [Tensor(np.zeros((5, 8), np.int32))])
    with pytest.raises(ValueError, match="rank"):
        A.check_signature([spec], [Tensor(np.zeros((5,), np.float32))])
    s = Symbol(divisor=4, unique=True)
    sig = [Tensor(shape=[s, 2], dtype=ms.float32), Tensor(shape=[s], dtype=ms.float32)]
    A.check_signature(sig, [Tensor(np.zeros((8, 2), np.float32)), Tensor(np.zeros((8,), np.float32))])
    with pytest.raises(ValueError, match="does not admit"):
        A.check_signature(sig, [Tensor(np.zeros((6, 2), np.float32)), Tensor(np.zeros((6,), np.float32))])
    with pytest.raises(ValueError, match="same unique Symbol"):
        A.check_signature(sig, [Tensor(np.zeros((8, 2), np.float32)), Tensor(np.zeros((4,), np.float32))])


def test_jit_signature_and_cell_set_inputs():
    sig = Tensor(shape=[None, 4], dtype=ms.float32)

    @ms.jit(input_signature=[sig])
    def double(x):
        return ops.Concat(0)((x, x)) * 2.0

    y = double(Tensor(np.ones((3, 4), np.float32)))
    assert tuple(y.shape) == (6, 4) and float(y.sum()) == 48.0
    assert tuple(double(Tensor(np.ones((5, 4), np.float32))).shape) == (10, 4)
    with pytest.raises(ValueError):
        double(Tensor(np.ones((3, 5), np.float32)))
    assert repr(double.infer()) == "Tensor[float32](2*s0, 4)"

    net = nn.Dense(4, 3)
    net.set_inputs(sig)
    assert repr(net.infer_outputs()) == "Tensor[float32](s0, 3)"
    ms.set_context(mode=ms.GRAPH_MODE)
    try:
        assert tuple(net(Tensor(np.ones((2, 4), np.float32))).shape) == (2, 3)
        with pytest.raises(ValueError, match="set_inputs"):
            net(Tensor(np.ones((2, 5), np.float32)))
    finally:
        ms.set_context(mode=ms.PYNATIVE_MODE)


def test_primitive_infer_hooks():
    relu = ops.ReLU()
    assert repr(relu.infer(T((None, 3), torch.float16))) == "Tensor[float16](s0, 3)"

    class Twice(PrimitiveWithInfer):
        def __init__(self):
            super().__init__("Twice")

        def _run(self, x):
            return torch.cat([x, x], 0)

    tw = Twice()
    assert tw.infer_shape([3, 5]) == [6, 5] and tw.infer_shape([-1, 5]) == [-1, 5]
    assert tw.infer_dtype(torch.float16) == torch.float16
    assert tw.__infer__({"shape": [2, 2], "dtype": torch.int32}) == {"shape": [4, 2], "dtype": torch.int32,
                                                                     "value": None}

    class Declared(PrimitiveWithInfer):
        def __init__(self):
            super().__init__("Declared")

        def infer_shape(self, x):
            return [x[0], 1]

        def infer_dtype(self, x):
            return torch.float32

    assert Declared().__infer__({"shape": [7, 9], "dtype": torch.int8})["shape"] == [7, 1]


def test_graph_annotation(tmp_path):
    from mindspore_b200.graph.jit import trace_cell
    net = nn.SequentialCell([nn.Dense(4, 6), nn.ReLU(), nn.Dense(6, 2)])
    x = Tensor(np.ones((5, 4), np.float32))
    fg = trace_cell(net, (x,))
    assert A.annotate_graph(fg, (x,)) >= 4
    calls = [n for n in fg.graph.nodes if n.op == "call_function"]
    assert all("abstract" in n.meta for n in calls)
    assert calls[-1].meta["abstract"] == T((5, 2), f32)
    assert ": Tensor[float32](5, 2)" in fg.to_text()
