"""yaml operator definitions -> generated primitives and functional wrappers."""
import importlib.util
import os

import pytest
import torch

import mindspore_b200 as ms
from mindspore_b200 import ops_generate as og


def _load(tmp_path, src):
    path = tmp_path / "gen_ops_def.py"
    path.write_text(src)
    spec = importlib.util.spec_from_file_location("gen_ops_def", str(path))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_generated_module_runs(tmp_path):
    defs = og.load_definitions([os.path.join(os.path.dirname(og.__file__), "ops_def")])
    assert {"logaddexp", "roll_ext", "leaky_relu_ext"} <= set(defs)
    mod = _load(tmp_path, og.generate(defs))
    a, b = ms.Tensor(torch.tensor([0.0, 1.0])), ms.Tensor(torch.tensor([1.0, 1.0]))
    torch.testing.assert_close(torch.as_tensor(mod.logaddexp(a, b).numpy()), torch.logaddexp(a, b).as_subclass(torch.Tensor))
    r = mod.RollExt((1,), (0,))
    assert r.shifts == (1,) and r(ms.Tensor(torch.arange(4))).tolist() == [3, 0, 1, 2]
    assert mod.roll_ext(ms.Tensor(torch.arange(4)), (1,), (0,)).tolist() == [3, 0, 1, 2]
    assert mod.leaky_relu_ext(ms.Tensor(torch.tensor([-1.0, 2.0]))).tolist() == pytest.approx([-0.01, 2.0])
    assert mod.normal_float_float(0.0, 1.0, (2, 3)).shape == (2, 3)
    with pytest.raises(TypeError):
        mod.logaddexp(a, 3)
    with pytest.raises(TypeError):
        mod.RollExt("x")


def test_bad_definitions_are_rejected(tmp_path):
    bad = tmp_path / "bad.yaml"
    bad.write_text("foo:\n  args:\n    x: {dtype: quaternion}\n  impl: x\n")
    with pytest.raises(og.gen_ops.OpDefError):
        og.load_definitions([str(bad)])
    bad.write_text("foo:\n  args:\n    x: {dtype: tensor, default: null}\n    y: {dtype: tensor}\n  impl: x\n")
    with pytest.raises(og.gen_ops.OpDefError):
        og.load_definitions([str(bad)])
    bad.write_text("foo:\n  returns: {}\n")
    with pytest.raises(og.gen_ops.OpDefError):
        og.load_definitions([str(bad)])
