"""Summary event files, tensor dump, hal / mint / numpy namespaces."""
import json
import os

import numpy as np
import torch

import mindspore_b200 as ms
from mindspore_b200 import nn
from mindspore_b200.train import summary as S
from mindspore_b200.utils import dump as D


def test_summary_record_event_file(tmp_path):
    with S.SummaryRecord(str(tmp_path)) as rec:
        rec.add_value("scalar", "loss", ms.Tensor(torch.tensor(0.25)))
        rec.add_value("histogram", "w", ms.Tensor(torch.randn(100)))
        rec.add_value("tensor", "act", ms.Tensor(torch.ones(2, 3)))
        rec.record(7)
        rec.add_value("scalar", "loss", ms.Tensor(torch.tensor(0.125)))
        rec.record(8)
        rec.flush()
        name = rec.file_name
    assert os.path.basename(name).startswith("events.out.events.summary.") and name.endswith("_MS")
    events = [S.parse_event(p) for p in S.read_frames(name)]
    assert events[0]["version"] == "MindSpore.Event:1"
    assert events[1]["step"] == 7 and events[1]["values"]["loss[:scalar]"] == 0.25
    assert events[1]["values"]["act[:tensor]"]["tensor_dims"] == [2, 3]
    assert events[2]["values"]["loss[:scalar]"] == 0.125
    blob = bytearray(open(name, "rb").read())
    blob[40] ^= 0xFF
    bad = tmp_path / "bad_MS"
    bad.write_bytes(bytes(blob))
    try:
        S.read_frames(str(bad))
        raise AssertionError("corruption not detected")
    except ValueError:
        pass


def test_set_dump_writes_cell_outputs(tmp_path, monkeypatch):
    cfg = tmp_path / "dump.json"
    cfg.write_text(json.dumps({"common_dump_settings": {"path": str(tmp_path / "out"), "net_name": "Net",
                                                        "iteration": "0|2"}}))
    monkeypatch.setenv("MINDSPORE_DUMP_CONFIG", str(cfg))
    D.reset()
    ms.set_context(device_target="CPU")
    net = nn.Dense(4, 2)
    ms.set_dump(net)
    for _ in range(3):
        net(ms.Tensor(torch.ones(1, 4)))
        D.next_iteration()
    base = tmp_path / "out" / "rank_0" / "Net" / "0"
    assert sorted(os.listdir(base)) == ["0", "2"]
    arr = np.load(base / "2" / "Dense.output.0.npy")
    assert arr.shape == (1, 2)
    ms.set_dump(net, enabled=False)


def test_namespaces():
    from mindspore_b200 import hal, mint
    import mindspore_b200.numpy as mnp
    assert hal.device_count("CPU") == 1 and isinstance(hal.memory_stats(), dict)
    s = hal.Stream()
    s.synchronize()
    x = mint.arange(6).reshape(2, 3)
    assert isinstance(x, ms.Tensor) and mint.sum(x).item() == 15
    assert mint.nn.Linear is nn.Dense and hasattr(mint.nn.functional, "softmax")
    a = mnp.linspace(0, 1, 5)
    assert isinstance(a, ms.Tensor) and float(mnp.sum(a)) == 2.5
    assert mnp.concatenate([mnp.ones((2, 2)), mnp.zeros((1, 2))]).shape == (3, 2)
    assert mnp.argmax(mnp.array([1, 5, 2])).item() == 1
