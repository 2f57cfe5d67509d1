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
