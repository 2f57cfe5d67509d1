"""ONNX export: the file parses field by field as ONNX, and an independent evaluator of its nodes reproduces the net."""
import numpy as np
import pytest
import torch
import torch.nn.functional as F

import mindspore_b200 as ms
from mindspore_b200 import nn, ops
from mindspore_b200.graph import onnx_proto
from mindspore_b200.models.lenet import LeNet5


def _attrs(node):
    out = {}
    for a in node.attribute:
        if a.type == onnx_proto.AT_INT:
            out[a.name] = int(a.i)
        elif a.type == onnx_proto.AT_FLOAT:
            out[a.name] = float(a.f)
        elif a.type == onnx_proto.AT_STRING:
            out[a.name] = a.s.decode()
        elif a.type == onnx_proto.AT_INTS:
            out[a.name] = [int(i) for i in a.ints]
        elif a.type == onnx_proto.AT_FLOATS:
            out[a.name] = [float(i) for i in a.floats]
        elif a.type == onnx_proto.AT_TENSOR:
            out[a.name] = onnx_proto.read_tensor(a.t)
    return out


def _pads(a, rank=2):
    if a.get("auto_pad") in (None, "NOTSET"):
        p = a.get("pads", [0] * (2 * rank))
        assert p[:rank] == p[rank:], "the evaluator takes symmetric pads"
        return p[:rank]
    assert a["auto_pad"] == "VALID"
    return [0] * rank


def run_onnx(model, feeds):
    """Evaluates the graph with the operator definitions of the ONNX specification (the subset the exporter emits)."""
    env = {t.name: onnx_proto.read_tensor(t) for t in model.graph.initializer}
    env.update({k: torch.as_tensor(np.asarray(v)) for k, v in feeds.items()})
    for nd in model.graph.node:
        a = _attrs(nd)
        x = [env[i] for i in nd.input]
        op = nd.op_type
        if op == "Conv":
            y = F.conv2d(x[0], x[1], x[2] if len(x) > 2 else None, a.get("strides", [1, 1]), _pads(a),
                         a.get("dilations", [1, 1]), a.get("group", 1))
        elif op == "MaxPool":
            y = F.max_pool2d(x[0], a["kernel_shape"], a.get("strides"), _pads(a))
        elif op == "AveragePool":
            y = F.avg_pool2d(x[0], a["kernel_shape"], a.get("strides"), _pads(a))
        elif op == "Gemm":
            A = x[0].t() if a.get("transA") else x[0]
            B = x[1].t() if a.get("transB") else x[1]
            y = a.get("alpha", 1.0) * (A @ B) + (a.get("beta", 1.0) * x[2] if len(x) > 2 else 0)
        elif op == "Flatten":
            y = x[0].reshape(int(np.prod(x[0].shape[:a.get("axis", 1)])), -1)
        elif op in ("Add", "Sub", "Mul", "Div", "Pow"):
            y = {"Add": torch.add, "Sub": torch.sub, "Mul": torch.mul, "Div": torch.div, "Pow": torch.pow}[op](*x)
        elif op in ("Relu", "Sigmoid", "Tanh", "Erf", "Exp", "Sqrt", "Neg"):
            y = getattr(torch, {"Relu": "relu", "Neg": "neg"}.get(op, op.lower()))(x[0])
        elif op == "MatMul":
            y = x[0] @ x[1]
        elif op == "Reshape":
            y = x[0].reshape([int(d) for d in x[1]])
        elif op == "Transpose":
            y = x[0].permute(a["perm"])
        elif op in ("Softmax", "LogSoftmax"):
            y = (torch.softmax if op == "Softmax" else torch.log_softmax)(x[0], a.get("axis", -1))
        elif op == "LayerNormalization":
            y = F.layer_norm(x[0], x[0].shape[a["axis"]:], x[1], x[2], a.get("epsilon", 1e-5))
        elif op == "BatchNormalization":
            y = F.batch_norm(x[0], x[3], x[4], x[1], x[2], False, 0.0, a.get("epsilon", 1e-5))
        elif op == "ReduceMean":
            y = x[0].mean(a["axes"], keepdim=bool(a.get("keepdims", 1))) if "axes" in a else x[0].mean()
        elif op == "ReduceSum":
            y = x[0].sum([int(d) for d in x[1]], keepdim=bool(a.get("keepdims", 1))) if len(x) > 1 else x[0].sum()
        elif op == "Concat":
            y = torch.cat(x, a["axis"])
        elif op == "Identity":
            y = x[0]
        elif op == "Gather":
            y = torch.index_select(x[0], a.get("axis", 0), x[1].reshape(-1)).reshape(
                x[0].shape[:a.get("axis", 0)] + x[1].shape + x[0].shape[a.get("axis", 0) + 1:])
        elif op == "Slice":
            idx = [slice(None)] * x[0].dim()
            for b, e_, ax, st in zip(x[1].tolist(), x[2].tolist(), x[3].tolist(), x[4].tolist()):
                idx[ax] = slice(b, e_, st)
            y = x[0][tuple(idx)]
        elif op == "Squeeze":
            y = x[0]
            for ax in sorted(x[1].tolist(), reverse=True):
                y = y.squeeze(ax)
        elif op == "Cast":
            y = x[0].to(onnx_proto.DT_REV[a["to"]])
        else:
            raise AssertionError("the evaluator has no %s" % op)
        env[nd.output[0]] = y
    return [env[o.name] for o in model.graph.output]


def _load(path):
    model = onnx_proto.messages()["ModelProto"]()
    model.ParseFromString(open(path, "rb").read())
    return model


def _varint(buf, pos):
    val = shift = 0
    while True:
        b = buf[pos]
        pos += 1
        val |= (b & 0x7F) << shift
        if b < 0x80:
            return val, pos
        shift += 7


def test_lenet_file_is_onnx_on_the_wire_and_evaluates(tmp_path):
    ms.set_seed(1)
    net = LeNet5()
    x = ms.Tensor(np.random.RandomState(0).randn(2, 1, 32, 32).astype(np.float32))
    path = ms.export(net, x, file_name=str(tmp_path / "lenet"), file_format="ONNX")
    assert path.endswith(".onnx")
    raw = open(path, "rb").read()
    # top-level fields by number, read without the schema: 1 ir_version (varint), 2 producer_name, 3 producer_version,
    # 7 graph, 8 opset_import
    pos, seen = 0, {}
    while pos < len(raw):
        tag, pos = _varint(raw, pos)
        field, wire = tag >> 3, tag & 7
        if wire == 0:
            val, pos = _varint(raw, pos)
        else:
            assert wire == 2
            n, pos = _varint(raw, pos)
            val, pos = raw[pos:pos + n], pos + n
        seen[field] = val
    assert seen[1] == 8 and seen[2] == b"MindSpore" and set(seen) == {1, 2, 3, 7, 8}
    assert seen[8] == bytes([0x10, onnx_proto.OPSET])            # OperatorSetIdProto: version (field 2), default domain
    model = _load(path)
    assert [n.op_type for n in model.graph.node].count("Conv") == 2
    assert [i.name for i in model.graph.input] == ["x"] or len(model.graph.input) == 1
    dims = [d.dim_value for d in model.graph.input[0].type.tensor_type.shape.dim]
    assert dims == [2, 1, 32, 32] and model.graph.input[0].type.tensor_type.elem_type == 1
    assert {t.name for t in model.graph.initializer} >= {p.name for p in net.get_parameters()}
    got = run_onnx(model, {model.graph.input[0].name: x.numpy()})[0]
    np.testing.assert_allclose(got.numpy(), net(x).detach().numpy(), rtol=1e-4, atol=1e-5)


class _Block(nn.Cell):
    """Attention-shaped arithmetic: dense layers, layer norm, GELU, reshapes / transposes, batched matmul, softmax."""

    def __init__(self):
        super().__init__()
        self.qkv = nn.Dense(16, 48)
        self.out = nn.Dense(16, 16)
        self.norm = nn.LayerNorm((16,))
        self.gelu = nn.GELU(approximate=False)

    def construct(self, x):
        b, s, _ = x.shape
        h = self.norm(x)
        qkv = self.qkv(h).reshape(b, s, 3, 4, 4).permute(2, 0, 3, 1, 4)
        q, k, v = qkv[0], qkv[1], qkv[2]
        att = ops.Softmax(-1)(ops.BatchMatMul()(q, k.permute(0, 1, 3, 2)) * 0.5)
        y = ops.BatchMatMul()(att, v).permute(0, 2, 1, 3).reshape(b, s, 16)
        return x + self.gelu(self.out(y)), y.mean(-1)


def test_attention_block_and_conv_bn(tmp_path):
    ms.set_seed(2)
    net = _Block()
    x = ms.Tensor(np.random.RandomState(1).randn(2, 5, 16).astype(np.float32))
    try:
        path = ms.export(net, x, file_name=str(tmp_path / "block"), file_format="ONNX")
    except Exception as e:                                                                  # noqa: BLE001
        pytest.fail("export failed: %s" % e)
    model = _load(path)
    kinds = {n.op_type for n in model.graph.node}
    assert {"LayerNormalization", "Softmax", "Erf", "Transpose", "MatMul"} <= kinds
    got = run_onnx(model, {model.graph.input[0].name: x.numpy()})
    want = net(x)
    assert len(got) == 2
    for g, w in zip(got, want):
        np.testing.assert_allclose(g.numpy(), w.detach().numpy(), rtol=1e-4, atol=1e-5)

    conv = nn.SequentialCell([nn.Conv2d(3, 4, 3, pad_mode="pad", padding=1, has_bias=True), nn.BatchNorm2d(4),
                              nn.ReLU(), nn.AvgPool2d(2, 2)])
    conv.set_train(False)
    img = ms.Tensor(np.random.RandomState(2).randn(2, 3, 8, 8).astype(np.float32))
    model = _load(ms.export(conv, img, file_name=str(tmp_path / "conv"), file_format="ONNX"))
    assert [n.op_type for n in model.graph.node if n.op_type in ("Conv", "BatchNormalization", "AveragePool")] == \
        ["Conv", "BatchNormalization", "AveragePool"]
    got = run_onnx(model, {model.graph.input[0].name: img.numpy()})[0]
    np.testing.assert_allclose(got.numpy(), conv(img).detach().numpy(), rtol=1e-4, atol=1e-5)


def test_what_onnx_cannot_carry_is_reported(tmp_path):
    from mindspore_b200.graph.control_flow import cond
    from mindspore_b200.graph.mindir import MindIRError

    class Branch(nn.Cell):
        def construct(self, x):
            return cond(x.sum() > 0, lambda v: v + 1.0, lambda v: v - 1.0, x)

    with pytest.raises(MindIRError, match="control flow"):
        ms.export(Branch(), ms.Tensor(np.ones((2, 2), np.float32)), file_name=str(tmp_path / "b"), file_format="ONNX")
    with pytest.raises(NotImplementedError):
        ms.export(Branch(), ms.Tensor(np.ones((2, 2), np.float32)), file_name=str(tmp_path / "b"), file_format="AIR")
