import csv
import os

import torch

import mindspore_b200 as ms
from mindspore_b200 import nn


def test_profiler_writes_tables(tmp_path):
    ms.set_context(device_target="CPU")
    net = nn.Dense(8, 4)
    prof = ms.Profiler(output_path=str(tmp_path), profile_memory=True)
    for _ in range(3):
        net(ms.Tensor(torch.randn(2, 8)))
    prof.stop()
    prof.analyse()
    out = tmp_path / "profiler"
    names = set(os.listdir(out))
    assert {"kernel_time_0.csv", "op_type_0.csv", "timeline_0.json", "memory_0.csv"} <= names
    rows = list(csv.reader(open(out / "op_type_0.csv")))
    assert rows[0] == ["op_type", "calls", "host_total_us"] and len(rows) > 1
    assert isinstance(prof.op_analyse(), list)


def test_env_profiler(monkeypatch, tmp_path):
    monkeypatch.delenv("MS_PROFILER_OPTIONS", raising=False)
    assert ms.EnvProfiler.from_env() is None
    monkeypatch.setenv("MS_PROFILER_OPTIONS", '{"start": true, "output_path": "%s"}' % tmp_path)
    p = ms.EnvProfiler.from_env()
    assert p is not None
    p.stop()
