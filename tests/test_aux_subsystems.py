"""Summary event files, tensor dump, hal / mint / numpy namespaces."""
import json
import os

import numpy as np
import pytest
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
    assert issubclass(mint.nn.Linear, nn.Dense) and hasattr(mint.nn.functional, "softmax")
    a = mnp.linspace(0, 1, 5)
    assert isinstance(a, ms.Tensor) and float(mnp.sum(a)) == 2.5
    assert mnp.concatenate([mnp.ones((2, 2)), mnp.zeros((1, 2))]).shape == (3, 2)
    assert mnp.argmax(mnp.array([1, 5, 2])).item() == 1


def test_summary_collector_writes_event_file_and_landscape(tmp_path):
    import json
    import numpy as np
    import mindspore_b200 as ms
    import mindspore_b200.dataset as ds
    from mindspore_b200 import nn
    from mindspore_b200.train import Model
    from mindspore_b200.train.callback import SummaryCollector, SummaryLandscape
    ms.set_seed(0)
    rng = np.random.default_rng(0)
    x = rng.normal(size=(32, 4)).astype(np.float32)
    y = x.sum(1, keepdims=True).astype(np.float32)
    data = ds.NumpySlicesDataset((x, y), ["x", "y"], shuffle=False).batch(8)
    net = nn.Dense(4, 1)
    model = Model(net, nn.MSELoss(), nn.SGD(net.trainable_params(), 0.05))
    model.train(2, data, callbacks=[SummaryCollector(str(tmp_path), collect_freq=2)], dataset_sink_mode=False)
    events = [f for f in os.listdir(tmp_path) if f.startswith("events") and not f.endswith(".jsonl")]
    assert events and os.path.getsize(os.path.join(tmp_path, events[0])) > 40
    lines = [json.loads(l) for f in os.listdir(tmp_path) if f.endswith(".jsonl") for l in open(os.path.join(tmp_path, f))]
    assert [l["step"] for l in lines] == [2, 4, 6, 8]
    loss_net = nn.WithLossCell(net, nn.MSELoss())
    path = SummaryLandscape(str(tmp_path)).gen_landscapes_with_multi_process(
        lambda: (model, loss_net, data, None), {"landscape_size": 5, "span": 1.0})
    grid = np.array(json.load(open(path))["loss"])
    assert grid.shape == (5, 5) and grid[2, 2] < grid.mean() and np.isfinite(grid).all()


def test_step_trace_splits_phases_exposed_communication_and_gaps():
    """Synthetic timeline: two steps; forward, backward (by name and by GEMM operand layout), optimizer, a
    collective half hidden behind a GEMM, and an idle gap."""
    import types
    import torch
    from mindspore_b200.profiler import Profiler

    def ev(name, start, end, cuda=True):
        return types.SimpleNamespace(name=name, time_range=types.SimpleNamespace(start=start, end=end),
                                     device_type=torch.autograd.DeviceType.CUDA if cuda else torch.autograd.DeviceType.CPU)

    def step(t):
        return [ev("msb::step", t, t + 50, cuda=False),
                ev("msb::rmsnorm_fwd_kernel<2>", t + 100, t + 200),
                ev("void msb::gemm_bf16_kernel<256, false, false, 0>(...)", t + 200, t + 500),
                ev("ncclDevKernel_AllGather_RING_LL", t + 400, t + 700),        # 100 us hidden, 200 us exposed
                ev("void msb::gemm_bf16_kernel<256, false, true, 0>(...)", t + 800, t + 1000),    # dgrad
                ev("msb::fa_bwd_dq_kernel", t + 1000, t + 1100),
                ev("void msb::adamw_kernel<float>(...)", t + 1100, t + 1300)]

    prof = Profiler.__new__(Profiler)
    prof._events = lambda: step(0) + step(10000)
    rows = prof.step_trace()
    assert len(rows) == 2
    for r in rows:
        assert r["fp_ms"] == 0.4 and r["bp_ms"] == 0.3 and r["optimizer_ms"] == 0.2 and r["comm_ms"] == 0.3
        assert r["comm_exposed_ms"] == 0.2 and r["gap_ms"] == 0.1 and r["total_ms"] == 1.2 and r["kernels"] == 6


def test_timed_synchronize_polls_and_gives_up():
    """hal.wait_event (the core of synchronize(timeout=...)): returns once the query holds, raises after the limit;
    driven by a fake clock, no device involved."""
    from mindspore_b200 import hal
    now = [0.0]
    polls = []

    def sleep(dt):
        polls.append(dt)
        now[0] += dt
    state = {"n": 0}

    def done_after_three():
        state["n"] += 1
        return state["n"] > 3
    hal.wait_event(done_after_three, 5.0, clock=lambda: now[0], sleep=sleep)
    assert state["n"] == 4 and len(polls) == 3 and polls[1] > polls[0]
    with pytest.raises(hal.StreamSyncTimeout, match="did not finish within 2.0 s"):
        hal.wait_event(lambda: False, 2.0, what="device 0", clock=lambda: now[0], sleep=sleep)
    hal.synchronize(timeout=1.0)          # no GPU here: returns at once


def test_offline_debugger_reads_dumps_and_checks_watchpoints(tmp_path, monkeypatch):
    import json

    from mindspore_b200 import nn
    from mindspore_b200.offline_debug import dbg_services as D
    from mindspore_b200.utils import dump
    cfg = tmp_path / "dump.json"
    cfg.write_text(json.dumps({"common_dump_settings": {"path": str(tmp_path / "out"), "net_name": "Net",
                                                        "iteration": "all"}}))
    monkeypatch.setenv("MINDSPORE_DUMP_CONFIG", str(cfg))
    dump.reset()

    class Net(nn.Cell):
        def __init__(self):
            super().__init__()
            self.fc = nn.Dense(3, 2)
            self.act = nn.ReLU()

        def construct(self, x):
            return self.act(self.fc(x))

    net = Net()
    dump.set_dump(net.fc)
    dump.set_dump(net.act)
    x = ms.Tensor(np.array([[1.0, -2.0, 3.0]], np.float32))
    net(x)                                            # iteration 0
    dump.next_iteration()
    net(x)                                            # iteration 1: the same values
    dump.next_iteration()
    net(x * float("inf"))                             # iteration 2: overflow
    dump.set_dump(net.fc, False)
    dump.set_dump(net.act, False)
    dump.reset()

    dbg = D.DbgServices(str(tmp_path / "out"))
    with pytest.raises(RuntimeError):
        dbg.check_watchpoints(0)
    dbg.initialize("Net")
    info = D.TensorInfo("Dense", 0, 0, 0, 0)
    (data,) = dbg.read_tensors([info])
    want = net.fc(x).detach().numpy()
    assert data.shape == [1, 2] and np.allclose(np.frombuffer(data.data_ptr, np.float32).reshape(1, 2), want)
    (base,) = dbg.read_tensor_base([info])
    (stat,) = dbg.read_tensor_stats([info])
    assert base.data_size == 8 and stat.count == 2 and abs(stat.max_value - want.max()) < 1e-6
    assert "nan_count = 0" in str(stat)
    (missing,) = dbg.read_tensor_base([D.TensorInfo("Nothing", 0, 0, 0, 0)])
    assert missing.data_size == 0

    everywhere = {"*": {"rank_id": [0], "root_graph_id": [0], "is_output": True}}
    dbg.add_watchpoint(1, D.GENERAL_OVERFLOW, everywhere, [])
    dbg.add_watchpoint(2, D.MIN_LT, {"ReLU": {"is_output": True}}, [D.Parameter("param", False, 0.5)])
    dbg.add_watchpoint(3, D.NOT_CHANGED, {"Dense": {}}, [D.Parameter("rtol", False, 1e-6)])
    dbg.add_watchpoint(4, D.ALL_ZERO, everywhere, [D.Parameter("zero_percentage_ge", False, 100.0)])
    hits0 = dbg.check_watchpoints(0)
    relu = net(x).detach().numpy()
    expect_min = relu.min() < 0.5
    assert [h.watchpoint_id for h in hits0 if h.name == "ReLU" and h.watchpoint_id == 2] == ([2] if expect_min else [])
    if expect_min:
        hit = next(h for h in hits0 if h.watchpoint_id == 2)
        assert hit.parameters[0].hit and abs(hit.parameters[0].actual_value - relu.min()) < 1e-6
    assert not any(h.watchpoint_id in (1, 3) for h in hits0)
    assert any(h.watchpoint_id == 4 for h in hits0) == bool((relu == 0).all())
    hits1 = dbg.check_watchpoints(1)
    assert [h.name for h in hits1 if h.watchpoint_id == 3] == ["Dense"]
    hits2 = dbg.check_watchpoints(2)
    assert {h.name for h in hits2 if h.watchpoint_id == 1} >= {"Dense"}
    dbg.remove_watchpoint(1)
    assert not any(h.watchpoint_id == 1 for h in dbg.check_watchpoints(2))
    with pytest.raises(ValueError):
        dbg.add_watchpoint(9, 99, everywhere, [])
    with pytest.raises(ValueError):
        dbg.remove_watchpoint(1)
