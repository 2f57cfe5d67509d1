"""Strategy files (protobuf + JSON) and checkpoint transformation between shard strategies."""
import os

import numpy as np
import pytest
import torch

import mindspore_b200 as ms
from mindspore_b200.parallel import checkpoint_transform as CT
from mindspore_b200.parallel import strategy_ckpt as SC
from mindspore_b200.parallel.layout import TensorLayout, slice_for_rank


def _entry(dev, tmap, shard_size=0, stage=0):
    return SC.ParamLayoutEntry(dev, tmap, (), (), 0, 0, shard_size, stage)


@pytest.mark.parametrize("ext", [".ckpt", ".json"])
def test_strategy_file_roundtrip(tmp_path, ext):
    sf = SC.StrategyFile(1)
    sf.layouts["w"] = _entry([2, 4], [0, -1], shard_size=2, stage=1)
    sf.layouts["b"] = _entry([8], [-1], stage=1)
    sf.strategies["Default/MatMul-op1"] = (1, [(2, 1), (1, 4)])
    path = str(tmp_path / ("strategy" + ext))
    sf.save(path)
    back = SC.StrategyFile.load(path)
    assert back.current_stage == 1
    assert back.layouts["w"] == sf.layouts["w"] and back.layouts["b"] == sf.layouts["b"]
    assert back.strategies == sf.strategies
    assert SC.build_searched_strategy(path)["w"] == [[2, 4], [0, -1], [], [], 0, 0, 2]


def test_group_info_roundtrip(tmp_path):
    path = str(tmp_path / "group_info.pb")
    SC.save_group_info(path, {"g0": [0, 1], "g1": [2, 3]}, [0, 2])
    assert SC.restore_group_info_list(path) == [0, 2]


def _save_sharded(dirname, full, layouts, world, prefix="net"):
    for r in range(world):
        items = []
        for name, t in full.items():
            lay = layouts.get(name)
            sl = t if lay is None else slice_for_rank(t, lay, r).contiguous()
            items.append({"name": name, "data": ms.Tensor(sl.clone())})
        d = os.path.join(dirname, "rank_%d" % r)
        os.makedirs(d, exist_ok=True)
        ms.save_checkpoint(items, os.path.join(d, "%s%d.ckpt" % (prefix, r)))


def _strategy(path, layouts, stage=0):
    sf = SC.StrategyFile(stage)
    for n, lay in layouts.items():
        sf.layouts[n] = SC.ParamLayoutEntry.from_layout(lay, stage)
    sf.save(path)


def test_transform_between_strategies(tmp_path):
    torch.manual_seed(0)
    full = {"w1": torch.randn(16, 8), "w2": torch.randn(8, 16), "bias": torch.randn(16), "step": torch.tensor([3.0])}
    src_lay = {"w1": TensorLayout((2, 2), (0, -1), (16, 8)),            # rows over mp, replicated over dp
               "w2": TensorLayout((2, 2), (-1, 0), (8, 16), opt_shard_size=2),   # cols over mp + optimizer shard
               "bias": TensorLayout((4,), (0,), (16,))}
    dst_lay = {"w1": TensorLayout((8,), (-1, 0), (16, 8)),
               "w2": TensorLayout((2, 4), (1, 0), (8, 16)),
               "bias": TensorLayout((8,), (-1,), (16,))}
    src_dir, dst_dir = str(tmp_path / "src"), str(tmp_path / "dst")
    _save_sharded(src_dir, full, src_lay, 4)
    s_file, d_file = str(tmp_path / "src_strategy.ckpt"), str(tmp_path / "dst_strategy.json")
    _strategy(s_file, src_lay)
    _strategy(d_file, dst_lay)
    need = CT.rank_list_for_transform(0, s_file, d_file)
    assert need and set(need) <= {0, 1, 2, 3}
    CT.transform_checkpoints(src_dir, dst_dir, "new", s_file, d_file)
    for r in range(8):
        got = ms.load_checkpoint(os.path.join(dst_dir, "rank_%d" % r, "new%d.ckpt" % r))
        for name, t in full.items():
            lay = dst_lay.get(name)
            exp = t if lay is None else slice_for_rank(t, lay, r)
            torch.testing.assert_close(got[name].as_subclass(torch.Tensor), exp)
    # back to a single full checkpoint
    CT.transform_checkpoint_by_rank(0, {r: os.path.join(dst_dir, "rank_%d" % r, "new%d.ckpt" % r) for r in range(8)},
                                    str(tmp_path / "full.ckpt"), d_file, None)
    merged = ms.load_checkpoint(str(tmp_path / "full.ckpt"))
    for name, t in full.items():
        torch.testing.assert_close(merged[name].as_subclass(torch.Tensor), t)


def test_missing_source_rank_is_reported(tmp_path):
    full = {"w": torch.arange(32.0).reshape(8, 4)}
    lay = {"w": TensorLayout((4,), (0, -1), (8, 4))}
    src_dir = str(tmp_path / "src")
    _save_sharded(src_dir, full, lay, 4)
    os.remove(os.path.join(src_dir, "rank_2", "net2.ckpt"))
    s_file = str(tmp_path / "s.ckpt")
    _strategy(s_file, lay)
    with pytest.raises(ValueError, match="needs checkpoints of source ranks"):
        CT.transform_checkpoints(src_dir, str(tmp_path / "dst"), "x", s_file, None)


def test_merge_pipeline_strategies_and_sliced_parameter(tmp_path):
    d = tmp_path / "strategies"
    d.mkdir()
    _strategy(str(d / "stage0.ckpt"), {"a": TensorLayout((2,), (0,), (4,))}, stage=0)
    _strategy(str(d / "stage1.ckpt"), {"b": TensorLayout((2,), (-1,), (4,))}, stage=1)
    merged = CT.merge_pipeline_strategys(str(d), str(tmp_path / "merged.ckpt"))
    assert merged.layouts["a"].stage == 0 and merged.layouts["b"].stage == 1
    full = torch.arange(24.0).reshape(6, 4)
    lay = TensorLayout((2, 3), (0, -1), (6, 4))
    parts = [ms.Parameter(slice_for_rank(full, lay, r).clone(), name="p") for r in range(6)]
    strat = {"p": SC.ParamLayoutEntry.from_layout(lay).as_list()}
    out = CT.merge_sliced_parameter(parts, strat)
    torch.testing.assert_close(out.as_subclass(torch.Tensor), full)


def test_get_ckpt_path_with_strategy_finds_a_replica(tmp_path):
    """dev matrix (dp=2, mp=2), weight split over mp only: ranks 0 / 2 and 1 / 3 hold the same slices."""
    from mindspore_b200 import nn, train
    sf = SC.StrategyFile(0)
    sf.layouts["w"] = _entry([2, 2], [0, -1])
    spath = str(tmp_path / "strategy.ckpt")
    sf.save(spath)
    for r in (1, 2, 3):
        d = tmp_path / ("rank_%d" % r)
        d.mkdir()
        ms.save_checkpoint(nn.Dense(2, 2), str(d / "net.ckpt"))
    (tmp_path / "rank_0").mkdir()
    (tmp_path / "rank_0" / "net.ckpt").write_bytes(b"damaged")
    found = train.get_ckpt_path_with_strategy(str(tmp_path / "rank_0" / "net.ckpt"), spath)
    assert found == str(tmp_path / "rank_2" / "net.ckpt")
    ok = train.get_ckpt_path_with_strategy(str(tmp_path / "rank_1" / "net.ckpt"), spath)
    assert ok == str(tmp_path / "rank_1" / "net.ckpt")
    os.remove(str(tmp_path / "rank_2" / "net.ckpt"))
    assert train.get_ckpt_path_with_strategy(str(tmp_path / "rank_0" / "net.ckpt"), spath) is None
