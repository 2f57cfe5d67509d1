"""Flight recorder: ring semantics, snapshot, dump on an uncaught exception in a child process, and the hooks in the
train step / collectives."""
import os
import subprocess
import sys
import textwrap

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_ring_keeps_the_latest_events(tmp_path):
    from mindspore_b200.utils import recorder
    recorder.enable(str(tmp_path), mode=1, capacity=32)
    for i in range(100):
        recorder.record("kernel", "launch %d" % i, a=i, b=2 * i, step=i // 10)
    snap = recorder.snapshot()
    assert len(snap) == 32
    assert [e["a"] for e in snap] == list(range(68, 100))
    assert snap[-1]["text"] == "launch 99" and snap[-1]["category"] == "kernel" and snap[-1]["step"] == 9
    assert all(snap[i]["t_ns"] <= snap[i + 1]["t_ns"] for i in range(31))
    path = recorder.dump()
    lines = open(path).read().splitlines()
    assert lines[0].startswith("#") and len(lines) == 33 and lines[-1].endswith("launch 99")
    recorder.disable()


def test_step_and_collective_hooks(tmp_path):
    import mindspore_b200 as ms
    from mindspore_b200 import nn
    from mindspore_b200.utils import recorder
    recorder.enable(str(tmp_path), capacity=64)
    net = nn.WithLossCell(nn.Dense(4, 2), nn.MSELoss())
    step = nn.TrainOneStepCell(net, nn.SGD(net.trainable_params(), 0.1))
    x = ms.Tensor(np.ones((3, 4), np.float32))
    y = ms.Tensor(np.zeros((3, 2), np.float32))
    step(x, y)
    step(x, y)
    ev = [e for e in recorder.snapshot() if e["category"] == "step"]
    assert [e["step"] for e in ev] == [1, 2] and ev[0]["text"].startswith("begin")
    recorder.disable()


def test_dump_on_uncaught_exception(tmp_path):
    code = textwrap.dedent("""
        import sys
        sys.path.insert(0, %r)
        from mindspore_b200.utils import recorder
        assert recorder.enable_from_env()
        recorder.record("checkpoint", "saving step 7", a=7)
        raise RuntimeError("boom")
    """ % ROOT)
    env = dict(os.environ, MS_RDR_ENABLE="1", MS_RDR_PATH=str(tmp_path), RANK="3")
    p = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True, timeout=300)
    assert p.returncode != 0 and "boom" in p.stderr
    text = open(os.path.join(str(tmp_path), "rank_3", "rdr.txt")).read()
    assert "saving step 7" in text and "uncaught RuntimeError: boom" in text
