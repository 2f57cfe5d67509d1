"""Graph files: export a network, load it back, run it through nn.GraphCell and get the same numbers."""
import numpy as np
import pytest
import torch

import mindspore_b200 as ms
from mindspore_b200 import nn, ops
from mindspore_b200.models.lenet import LeNet5


class Small(nn.Cell):
    def __init__(self):
        super().__init__()
        self.fc = nn.Dense(6, 4)
        self.norm = nn.LayerNorm((4,))
        self.softmax = ops.Softmax(-1)
        self.topk = ops.TopK()

    def construct(self, x):
        h = self.norm(self.fc(x))
        p = self.softmax(h[:, 1:])
        v, i = self.topk(p, 2)
        return v * 2.0, i


def test_export_load_round_trip(tmp_path):
    ms.set_seed(0)
    net = Small()
    x = ms.Tensor(torch.randn(5, 6))
    path = ms.export(net, x, file_name=str(tmp_path / "small"), file_format="MINDIR")
    assert path.endswith(".mindir")
    graph = ms.load(path)
    cell = nn.GraphCell(graph)
    v0, i0 = net(x)
    v1, i1 = cell(x)
    np.testing.assert_allclose(v1.numpy(), v0.detach().numpy(), rtol=1e-6)
    assert i1.tolist() == i0.tolist()
    y = ms.Tensor(torch.randn(5, 6))                       # the loaded graph is not tied to the example input
    np.testing.assert_allclose(cell(y)[0].numpy(), net(y)[0].detach().numpy(), rtol=1e-6)
    assert set(graph.params) == {"fc.weight", "fc.bias", "norm.gamma", "norm.beta"}
    graph.set_param("fc.bias", np.zeros(4, np.float32))
    assert not np.allclose(cell(x)[0].numpy(), v0.detach().numpy())


def test_lenet_export_and_encrypted_file(tmp_path):
    ms.set_seed(1)
    net = LeNet5()
    x = ms.Tensor(torch.randn(2, 1, 32, 32))
    key = b"0123456789abcdef"
    path = ms.export(net, x, file_name=str(tmp_path / "lenet.mindir"), file_format="MINDIR", enc_key=key)
    with pytest.raises(Exception):
        ms.load(path)
    cell = nn.GraphCell(ms.load(path, dec_key=key))
    np.testing.assert_allclose(cell(x).numpy(), net(x).detach().numpy(), rtol=1e-5, atol=1e-6)


def test_bad_files_are_rejected(tmp_path):
    from mindspore_b200.graph.mindir import MindIRError
    p = tmp_path / "junk.mindir"
    p.write_bytes(b"not a graph")
    with pytest.raises(MindIRError):
        ms.load(str(p))
    with pytest.raises(ValueError):
        ms.export(Small(), ms.Tensor(torch.randn(1, 6)), file_name=str(tmp_path / "x"), file_format="TFLITE")


def test_export_uses_the_reference_protobuf_layout(tmp_path):
    """LeNet exports as a ModelProto (mind_ir.proto field numbers): weights in graph.parameter, every call a
    REF::<Prim>:<id> node with its primitive record, and loads back to the same numbers."""
    from mindspore_b200.graph import mindir_proto as MP
    ms.set_seed(3)
    net = LeNet5()
    x = ms.Tensor(torch.randn(2, 1, 32, 32))
    path = ms.export(net, x, file_name=str(tmp_path / "lenet_pb"), file_format="MINDIR", container="proto")
    raw = open(path, "rb").read()
    model = MP.messages()["ModelProto"]()
    model.ParseFromString(raw)
    assert model.producer_name == "MindSpore" and model.ir_version
    assert {t.name for t in model.graph.parameter} == {p.name for p in net.get_parameters()}
    conv = next(p for p in model.primitives if p.op_type == "Conv2D")
    attrs = {a.name: a for a in conv.attribute}
    assert attrs["out_channel"].type == MP.A_INT64 and attrs["out_channel"].i == 6
    assert attrs["kernel_size"].type == MP.A_TUPLE and [list(v.ints) for v in attrs["kernel_size"].values] == [[5], [5]]
    assert attrs["pad_mode"].type == MP.A_STRING and attrs["pad_mode"].s == b"valid"
    assert all(n.op_type.startswith("REF::") or n.op_type == "Constant" for n in model.graph.node)
    w = next(t for t in model.graph.parameter if t.name == "conv1.weight")
    assert list(w.dims) == [6, 1, 5, 5] and w.data_type == 1 and len(w.raw_data) == 6 * 25 * 4
    cell = nn.GraphCell(ms.load(path))
    np.testing.assert_allclose(cell(x).numpy(), net(x).detach().numpy(), rtol=1e-5, atol=1e-6)


def test_load_a_file_laid_out_by_an_older_writer(tmp_path):
    """Plain op_type nodes with attributes on the node, weights repeated among the inputs, side-effect plumbing
    (Load / UpdateState / Depend with monads), a Return node: y = relu(x @ w^T + b) * 2 read from such a file."""
    from mindspore_b200.graph import mindir_proto as MP
    M = MP.messages()
    model = M["ModelProto"]()
    model.ir_version = "0.1.0"
    model.producer_name = "MindSpore"
    g = model.graph
    g.name = "net"
    w = torch.randn(4, 6)
    b = torch.randn(4)
    for name, t in (("fc.weight", w), ("fc.bias", b)):
        tp = g.parameter.add()
        tp.name, tp.data_type = name, 1
        tp.dims.extend(t.shape)
        tp.raw_data = t.numpy().tobytes()
    vi = g.input.add()
    vi.name = "x"
    tin = vi.tensor.add()
    tin.dims.extend([3, 6])
    tin.data_type = 1
    g.input.add().name = "fc.weight"                     # older writers list parameters as inputs too

    def node(op, ins, out, **attrs):
        n = g.node.add()
        n.op_type, n.name = op, out
        n.output.append(out)
        n.input.extend(ins)
        for k, v in attrs.items():
            a = n.attribute.add()
            a.name = k
            MP._fill_attr(a, v)
        return n

    u = g.node.add()
    u.op_type, u.name = "Constant", "net:u"
    u.output.append("net:u")
    ua = u.attribute.add()
    ua.name, ua.type = "value", MP.A_UMONAD
    node("Load", ["fc.weight", "net:u"], "net:1")
    node("MatMul", ["x", "net:1"], "net:2", transpose_a=False, transpose_b=True)
    node("BiasAdd", ["net:2", "fc.bias"], "net:3", format="NCHW")
    node("ReLU", ["net:3"], "net:4")
    two = g.node.add()
    two.op_type, two.name = "Constant", "net:5"
    two.output.append("net:5")
    ta = two.attribute.add()
    ta.name = "value"
    MP._fill_attr(ta, torch.tensor(2.0))
    node("Mul", ["net:4", "net:5"], "net:6")
    node("UpdateState", ["net:u", "net:6"], "net:7")
    node("Depend", ["net:6", "net:7"], "net:8")
    node("Return", ["net:8"], "net:9")
    g.output.add().name = "net:9"
    p = tmp_path / "old.mindir"
    p.write_bytes(model.SerializeToString())
    graph = ms.load(str(p))
    x = torch.randn(3, 6)
    out = nn.GraphCell(graph)(ms.Tensor(x))
    np.testing.assert_allclose(out.numpy(), (torch.relu(x @ w.t() + b) * 2).numpy(), rtol=1e-6, atol=1e-6)
    assert set(graph.params) == {"fc.weight", "fc.bias"}
    # an operator this build does not know is named in the error
    node("NoSuchOperator", ["x"], "net:10")
    del g.output[:]
    g.output.add().name = "net:10"
    p.write_bytes(model.SerializeToString())
    from mindspore_b200.graph.mindir import MindIRError
    with pytest.raises(MindIRError, match="NoSuchOperator"):
        ms.load(str(p))


def test_attribute_values_round_trip():
    from mindspore_b200.graph import mindir_proto as MP
    A = MP.messages()["AttributeProto"]
    for v in (3, -7, True, False, 0.5, 1e-7, 3.141592653589793, "same", None, (1, 2, 3), [1.5, "a", (2, False)],
              {"k": 1, "z": (2, 3)}, torch.float16):
        a = A()
        MP._fill_attr(a, v)
        b = A()
        b.ParseFromString(a.SerializeToString())
        got = MP._read_attr(b)
        if isinstance(v, float):
            assert got == pytest.approx(v, rel=1e-7)
        else:
            assert got == v, (v, got)
    t = torch.arange(6, dtype=torch.bfloat16).reshape(2, 3)
    a = A()
    MP._fill_attr(a, t)
    assert torch.equal(MP._read_attr(a), t)


# Two MindIR files as the reference's exporter wrote them (an Add of two inputs, a ReLU), base64: reading them shows
# that the protobuf layout, the primitive references and the attribute encoding agree with the reference's writer.
_REFERENCE_ADD_MINDIR = (
    "CgUwLjEuMBIJTWluZFNwb3JlKgUxLjEuMDqiAwqRAgoaNl80X2NvbnN0cnVjdF93cmFwcGVyLjQ6eF8KGjZfNF9jb25zdHJ1Y3Rf"
    "d3JhcHBlci40OnlfEhs2XzRfY29uc3RydWN0X3dyYXBwZXIuNDo2OjIaGzZfNF9jb25zdHJ1Y3Rfd3JhcHBlci40OjU6MSIDQWRk"
    "Kh9iDggCCAIQAToGc2hhcGUxeg1zaGFwZTpzaGFwZTEsKjQKC2lucHV0X25hbWVzWgF4WgF5ehxzY2FsYXI6TGlzdFt2YWx1ZTEs"
    "dmFsdWUyLF0sgAEIKjAKDG91dHB1dF9uYW1lc1oGb3V0cHV0ehVzY2FsYXI6TGlzdFt2YWx1ZTEsXSyAAQg6D0RlZmF1bHQvQWRk"
    "LW9wNRIXNl80X2NvbnN0cnVjdF93cmFwcGVyLjQqJAoaNl80X2NvbnN0cnVjdF93cmFwcGVyLjQ6eF8SBggCCAIQASokCho2XzRf"
    "Y29uc3RydWN0X3dyYXBwZXIuNDp5XxIGCAIIAhABMiUKGzZfNF9jb25zdHJ1Y3Rfd3JhcHBlci40OjY6MhIGCAIIAhABOgA=")
_REFERENCE_RELU_MINDIR = (
    "CgUwLjEuMBIJTWluZFNwb3JlKggxLjUuMHJjMTqYAwqSAgofMzk0XzM5MV9jb25zdHJ1Y3Rfd3JhcHBlci4xMDI6eBIjMzk0XzM5"
    "MV9jb25zdHJ1Y3Rfd3JhcHBlci4xMDI6MTAzOjEaIzM5NF8zOTFfY29uc3RydWN0X3dyYXBwZXIuMTAyOjEwMzoxIgRSZUxVKiNi"
    "EggBCAEIAggCEAE6BnNoYXBlMXoNc2hhcGU6c2hhcGUxLCoqCgtpbnB1dF9uYW1lc1oBeHoVc2NhbGFyOkxpc3RbdmFsdWUxLF0s"
    "gAEIKjAKDG91dHB1dF9uYW1lc1oGb3V0cHV0ehVzY2FsYXI6TGlzdFt2YWx1ZTEsXSyAAQg6HERlZmF1bHQvcmVsdS1SZUxVL1Jl"
    "TFUtb3AxODgSHTM5NF8zOTFfY29uc3RydWN0X3dyYXBwZXIuMTAyKi0KHzM5NF8zOTFfY29uc3RydWN0X3dyYXBwZXIuMTAyOngS"
    "CggBCAEIAggCEAEyMQojMzk0XzM5MV9jb25zdHJ1Y3Rfd3JhcHBlci4xMDI6MTAzOjESCggBCAEIAggCEAE6AA==")


def test_files_written_by_the_reference_exporter_load_and_run(tmp_path):
    import base64
    for name, blob in (("add", _REFERENCE_ADD_MINDIR), ("relu", _REFERENCE_RELU_MINDIR)):
        (tmp_path / (name + ".mindir")).write_bytes(base64.b64decode(blob))
    add = nn.GraphCell(ms.load(str(tmp_path / "add.mindir")))
    np.testing.assert_allclose(add(ms.Tensor([1.0, -2.0]), ms.Tensor([2.0, 0.5])).numpy(), [3.0, -1.5])
    relu = nn.GraphCell(ms.load(str(tmp_path / "relu.mindir")))
    x = np.array([[-1.0, 2.0], [0.5, -3.0]], np.float32)
    np.testing.assert_allclose(relu(ms.Tensor(x)).numpy(), np.maximum(x, 0))


def test_tuple_attribute_elements_use_the_repeated_fields():
    """Scalars inside a tuple attribute are written as one entry of ints / floats / strings (how the reference's
    exporter stores e.g. kernel_size), top-level scalars as i / f / s; both forms are read."""
    from mindspore_b200.graph import mindir_proto as MP
    ap = MP.messages()["AttributeProto"]()
    MP._fill_attr(ap, (5, 2.5, "same", True))
    assert [list(v.ints) for v in ap.values] == [[5], [], [], [1]] and list(ap.values[1].floats) == [2.5]
    assert list(ap.values[2].strings) == [b"same"] and not ap.values[0].HasField("i")
    assert MP._read_attr(ap) == (5, 2.5, "same", True)
    top = MP.messages()["AttributeProto"]()
    MP._fill_attr(top, 16)
    assert top.i == 16 and not list(top.ints) and MP._read_attr(top) == 16
    legacy = MP.messages()["AttributeProto"]()
    legacy.type = MP.A_TUPLE
    v = legacy.values.add()
    v.type, v.i = MP.A_INT64, 7                              # the single-value field inside a tuple is accepted too
    assert MP._read_attr(legacy) == (7,)


class _Branchy(nn.Cell):
    """A tensor-valued ``if`` and a ``while`` whose trip count depends on the data."""

    def __init__(self):
        super().__init__()
        self.fc = nn.Dense(4, 4)

    def construct(self, x, n):
        from mindspore_b200.graph.control_flow import cond, while_loop
        h = self.fc(x)
        h = cond(h.sum() > 0, lambda v: ops.ReLU()(v) + 1.0, lambda v: v * 2.0, h)
        i0 = ops.ZerosLike()(n)
        _, out = while_loop(lambda i, v: i < n, lambda i, v: (i + 1, v + self.fc(v)), (i0, h))
        return out


def test_control_flow_exports_as_functions_and_runs_from_the_file(tmp_path):
    from mindspore_b200.graph.mindir_proto import messages
    net = _Branchy()
    x = ms.Tensor(np.random.RandomState(0).randn(3, 4).astype(np.float32))
    n = ms.Tensor(np.array(3, np.int64))
    path = str(tmp_path / "branchy")
    ms.export(net, x, n, file_name=path, file_format="MINDIR", container="proto")
    model = messages()["ModelProto"]()
    model.ParseFromString(open(path + ".mindir", "rb").read())
    names = [f.name for f in model.functions]
    assert any("cond_true" in f for f in names) and any("cond_false" in f for f in names)
    assert any("while_header" in f for f in names) and any("while_step" in f for f in names)
    kinds = {p.op_type for p in model.primitives}
    assert {"Switch", "Partial"} <= kinds
    graph = ms.load(path + ".mindir")
    cell = nn.GraphCell(graph)
    for xv, nv in ((x, 3), (-x, 0), (x * 0.1, 5)):                 # both branches, several trip counts
        nt = ms.Tensor(np.array(nv, np.int64))
        want = net(xv, nt)
        got = cell(xv, nt)
        assert np.allclose(got.detach().numpy(), want.detach().numpy(), atol=1e-5)
    assert sorted(p.name for p in cell.get_parameters()) == sorted(p.name for p in net.get_parameters())
    # long loops run in constant stack depth
    long_n = ms.Tensor(np.array(3000, np.int64))
    small = ms.Tensor(np.zeros((3, 4), np.float32))
    assert cell(small, long_n).shape == (3, 4)


def test_a_model_with_closures_in_the_reference_conventions(tmp_path):
    """Built field by field the way the reference's exporter names things: a function reads a node of the main graph
    (a free variable), is called by name (``REF::<function>``) and through a Switch of two function values."""
    from mindspore_b200.graph.mindir_proto import _fill_attr, load_model_proto, messages
    M = messages()
    model = M["ModelProto"]()
    model.ir_version, model.producer_name, model.mind_ir_version = "0.1.1", "MindSpore", 2

    def prim(op):
        pp = model.primitives.add()
        pp.name, pp.op_type, pp.prim_type = "%s:%d" % (op, len(model.primitives)), op, 1
        return "REF::" + pp.name

    def node(gp, name, op_type, inputs):
        nd = gp.node.add()
        nd.name = name
        nd.output.append(name)
        nd.op_type = op_type
        nd.input.extend(inputs)
        return name

    def const(gp, name, value):
        nd = gp.node.add()
        nd.name = name
        nd.output.append(name)
        nd.op_type = "Constant"
        ap = nd.attribute.add()
        ap.name = "value"
        _fill_attr(ap, value)
        return name

    g = model.graph
    g.name = "main_1"
    for nm in ("x", "y"):
        vi = g.input.add()
        vi.name = nm
        tp = vi.tensor.add()
        tp.dims.extend([2])
        tp.data_type = 1
    s = node(g, "main_1:s:1", prim("Add"), ["x", "y"])                      # free variable of both functions
    zero = const(g, "main_1:c:2", 0.0)
    total = node(g, "main_1:t:3", prim("ReduceSum"), ["x"])
    c = node(g, "main_1:c:4", prim("Greater"), [total, zero])
    sw = node(g, "main_1:sw:5", prim("Switch"), [c, "then_2", "else_3"])
    picked = node(g, "main_1:call:6", "REF::" + sw, [])
    direct = node(g, "main_1:call:7", "REF::scale_4", [picked])
    g.output.add().name = direct
    f = model.functions.add()
    f.name = "then_2"
    f.output.add().name = node(f, "then_2:m:1", prim("Mul"), [s, "x"])
    f = model.functions.add()
    f.name = "else_3"
    f.output.add().name = node(f, "else_3:m:1", prim("Sub"), [s, "x"])
    f = model.functions.add()
    f.name = "scale_4"
    f.input.add().name = "scale_4:v"
    two = const(f, "scale_4:c:1", 2.0)
    f.output.add().name = node(f, "scale_4:m:2", prim("Mul"), ["scale_4:v", two])

    cell = nn.GraphCell(load_model_proto(model.SerializeToString()))
    x = ms.Tensor(np.array([1.0, 2.0], np.float32))
    y = ms.Tensor(np.array([0.5, 0.5], np.float32))
    assert np.allclose(cell(x, y).numpy(), ((x + y) * x * 2).numpy())
    assert np.allclose(cell(-x, y).numpy(), (((-x) + y) - (-x)) .numpy() * 2)
