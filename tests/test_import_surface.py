"""The reference's import paths and top-level names, FLOPs collection of a compiled graph, checkpoint weight
obfuscation, QuantDtype, save_mindir / convert_model."""
import importlib
import os

import numpy as np
import pytest
import torch

import mindspore_b200 as ms
from mindspore_b200 import nn, ops


@pytest.mark.parametrize("path,attr", [
    ("amp", "DynamicLossScaler"), ("log", "get_log_config"), ("mindrecord", "FileWriter"),
    ("nn.learning_rate_schedule", "CosineDecayLR"), ("nn.dynamic_lr", "piecewise_constant_lr"),
    ("nn.transformer", "TransformerOpParallelConfig"), ("parallel._transformer.moe", "MoE"),
    ("parallel.cluster.run", "main"), ("ops.operations.comm_ops", "AllReduce"), ("ops.function", "relu"),
    ("common.api", "jit"), ("common.lazy_inline", "lazy_inline"), ("common.mutable", "mutable"),
    ("common.dump", "set_dump"), ("train.summary.summary_record", "SummaryRecord"),
    ("nn.wrap.loss_scale", "DynamicLossScaleUpdateCell"), ("nn.wrap.cell_wrapper", "PipelineCell"),
    ("parallel.algo_parameter_config", "set_algo_parameters"), ("parallel._cost_model_context", "set_cost_model_context"),
    ("communication.comm_func", "all_reduce"), ("profiler.profiling", "Profiler"), ("safeguard", "obfuscate_ckpt"),
    ("dataset.engine.datasets", "GeneratorDataset"), ("train.callback", "ModelCheckpoint"),
])
def test_reference_import_paths_resolve(path, attr):
    mod = importlib.import_module("mindspore_b200." + path)
    assert hasattr(mod, attr), (path, attr)


def test_top_level_names_and_aliases_are_the_real_modules():
    for n in ["QuantDtype", "ms_class", "JitConfig", "flops_collection", "save_mindir", "FileWriter", "MindPage",
              "DatasetHelper", "connect_network_with_dataset", "build_train_network", "FixedLossScaleManager",
              "check_checkpoint", "export_split_mindir", "parse_print", "convert_model", "load_checkpoint_async",
              "get_log_config", "reshard", "SymbolTree", "obfuscate_ckpt", "load_obf_params_into_net",
              "SummaryCollector", "EarlyStopping", "ckpt_to_safetensors", "get_ckpt_path_with_strategy"]:
        assert hasattr(ms, n), n
    import mindspore_b200.amp as amp
    import mindspore_b200.train.amp as real
    assert amp is real and ms.amp is real and real.__spec__.name == "mindspore_b200.train.amp"
    with pytest.raises(AttributeError):
        ms.no_such_name
    with pytest.raises(ImportError):
        importlib.import_module("mindspore_b200.no_such_module")
    q = ms.QuantDtype
    assert q.INT8.value == 7 and q.UINT8.value == 107 and q.UINT4.num_bits == 4 and str(q.INT4) == "INT4"
    assert q.switch_signed(q.INT8) is q.UINT8 and q.INT4.value_range() == (-8, 7) and not q.is_signed(q.UINT2)


class _Mlp(nn.Cell):
    def __init__(self):
        super().__init__()
        self.fc1 = nn.Dense(32, 64)
        self.fc2 = nn.Dense(64, 8)

    def construct(self, x):
        return self.fc2(ops.relu(self.fc1(x)))


def test_flops_collection_counts_the_compiled_training_graph():
    from mindspore_b200.graph.flops import graph_flops
    from mindspore_b200.graph.jit import trace_cell
    ms.set_seed(0)
    net = _Mlp()
    x = ms.Tensor(torch.randn(16, 32))
    fwd = graph_flops(trace_cell(net, (x,)))
    mm = 2 * 16 * 32 * 64 + 2 * 16 * 64 * 8
    assert mm <= fwd["model"] <= mm + 16 * (64 * 3 + 8 * 2)           # contractions + a few element-wise passes
    ms.set_context(mode=ms.GRAPH_MODE)
    try:
        loss_net = nn.WithLossCell(net, nn.MSELoss())
        step = nn.TrainOneStepCell(loss_net, nn.SGD(net.trainable_params(), learning_rate=0.1))
        step.set_train()
        step(x, ms.Tensor(torch.randn(16, 8)))
        full, hw, shard, shard_hw, dynamic = ms.flops_collection("train")
        assert 3 * mm <= full <= 3 * mm + 40 * 16 * 64 and hw == full and shard == full and dynamic is False
    finally:
        ms.set_context(mode=ms.PYNATIVE_MODE)
    with pytest.raises(RuntimeError):
        from mindspore_b200.graph import flops
        flops._last.clear()
        ms.flops_collection("train")


def test_obfuscated_checkpoint_needs_the_ratios(tmp_path):
    ms.set_seed(1)
    net = _Mlp()
    x = ms.Tensor(torch.randn(4, 32))
    want = net(x).detach().numpy()
    src, dst = tmp_path / "plain", tmp_path / "obf"
    src.mkdir()
    dst.mkdir()
    ms.save_checkpoint(net, str(src / "net.ckpt"))
    ratios = ms.obfuscate_ckpt(net, str(src), target_modules=["", "fc1|fc2"], saved_path=str(dst), obfuscate_scale=50)
    assert len(ratios) == 2 and all(1 / 50 <= r <= 50 for r in ratios)
    assert os.listdir(dst) == ["net_obf.ckpt"]
    scaled = ms.load_checkpoint(str(dst / "net_obf.ckpt"))
    np.testing.assert_allclose(scaled["fc1.weight"].detach().numpy(),
                               net.fc1.weight.detach().numpy() * ratios[0], rtol=1e-5)
    np.testing.assert_allclose(scaled["fc1.bias"].detach().numpy(), net.fc1.bias.detach().numpy())
    ms.set_seed(2)
    other = _Mlp()
    ms.load_param_into_net(other, scaled)
    assert not np.allclose(other(x).detach().numpy(), want, atol=1e-3)        # scaled weights alone are wrong
    ms.load_obf_params_into_net(other, ["", "fc1|fc2"], ratios)
    np.testing.assert_allclose(other(x).detach().numpy(), want, rtol=1e-4, atol=1e-5)
    with pytest.raises(ValueError):
        ms.obfuscate_ckpt(net, str(src), target_modules=["", "nope"], saved_path=str(dst))
    with pytest.raises(ValueError):
        ms.obfuscate_ckpt(net, str(src), target_modules=["a b", "fc1"], saved_path=str(dst))
    with pytest.raises(ValueError):
        ms.load_obf_params_into_net(_Mlp(), ["", "fc1|fc2"], [1.0])
    with pytest.raises(NotImplementedError):
        ms.obfuscate_model({})


def test_save_mindir_and_convert_model(tmp_path):
    ms.set_seed(3)
    net = _Mlp()
    x = ms.Tensor(torch.randn(2, 32))
    ms.export(net, x, file_name=str(tmp_path / "m"), file_format="MINDIR")
    ms.convert_model(str(tmp_path / "m.mindir"), str(tmp_path / "copy.mindir"), "MINDIR")
    g = ms.load(str(tmp_path / "copy.mindir"))
    np.testing.assert_allclose(nn.GraphCell(g)(x).detach().numpy(), net(x).detach().numpy(), rtol=1e-5, atol=1e-6)
    with pytest.raises(NotImplementedError):
        ms.convert_model(str(tmp_path / "m.mindir"), str(tmp_path / "m.onnx"), "ONNX")
    with pytest.raises(ValueError):
        ms.convert_model(str(tmp_path / "m.mindir"), str(tmp_path / "m.x"), "AIR")
    with pytest.raises(TypeError):
        ms.save_mindir(object(), str(tmp_path / "bad"))


def test_remaining_nn_names():
    x = ms.Tensor(torch.randn(2, 3, 8, 8))
    y = nn.Conv2dBnAct(3, 4, 3, has_bn=True, activation="relu")(x)
    assert y.shape == (2, 4, 8, 8) and float(y.min()) >= 0
    assert nn.DenseBnAct(5, 2, has_bn=True, activation="leakyrelu")(ms.Tensor(torch.randn(4, 5))).shape == (4, 2)
    d = nn.DenseThor(4, 3)
    assert sorted(p.name for p in d.get_parameters()) == ["bias", "matrix_a", "matrix_g", "weight"]
    assert [p.name for p in d.trainable_params()] == ["weight", "bias"] or \
        sorted(p.name for p in d.trainable_params()) == ["bias", "weight"]
    assert nn.Conv2dThor(3, 4, 3).matrix_a.shape == (27, 27) and nn.EmbeddingThor(10, 4).matrix_g.shape == (4, 4)
    assert nn.EmbeddingLookupThor(10, 4).matrix_a.shape == (10,)
    loss = nn.TripletMarginWithDistanceLoss(margin=1.0)(ms.Tensor(torch.zeros(2, 3)), ms.Tensor(torch.zeros(2, 3)),
                                                        ms.Tensor(torch.full((2, 3), 0.1)))
    assert abs(float(loss) - (1 - 0.1 * 3 ** 0.5)) < 1e-3
    pooled, idx = torch.nn.functional.max_pool1d(torch.arange(8.).reshape(1, 1, 8), 2, return_indices=True)
    assert nn.MaxUnpool1d(2)(ms.Tensor(pooled), ms.Tensor(idx)).shape == (1, 1, 8)
    assert nn.FractionalMaxPool3d(2, output_size=(2, 2, 2))(ms.Tensor(torch.randn(1, 1, 5, 5, 5))).shape == (1, 1, 2, 2, 2)
    drop = nn.DropoutExt(0.25)
    assert drop.p == 0.25

    class Opt:
        @nn.opt_init_args_register
        def __init__(self, params, learning_rate=0.1, beta=ms.Tensor([0.9])):
            self.lr = learning_rate

    assert Opt([1, 2], learning_rate=0.5).init_args == {"learning_rate": 0.5}


def test_numpy_and_scipy_fft_names():
    import scipy.fft as sfft

    import mindspore_b200.numpy as mnp
    from mindspore_b200.scipy import fft as F
    x = np.random.RandomState(0).randn(3, 8).astype(np.float32)
    for kind in (1, 2, 3, 4):
        for norm in (None, "ortho"):
            if kind == 1 and norm:
                continue
            np.testing.assert_allclose(F.dct(ms.Tensor(x), kind, norm=norm).numpy(), sfft.dct(x, kind, norm=norm),
                                       rtol=1e-4, atol=1e-4)
            np.testing.assert_allclose(F.idct(ms.Tensor(x), kind, norm=norm).numpy(), sfft.idct(x, kind, norm=norm),
                                       rtol=1e-4, atol=1e-4)
    assert mnp.append(ms.Tensor([1, 2]), [3]).tolist() == [1, 2, 3]
    assert mnp.intersect1d([1, 3, 4, 3], [3, 1, 1]).tolist() == [1, 3]
    assert mnp.setdiff1d([1, 2, 3, 2, 4], [3, 4, 5]).tolist() == [1, 2]
    assert mnp.isin([1, 2], [2]).tolist() == [False, True] and mnp.in1d([[1, 2]], [1]).tolist() == [True, False]
    assert mnp.mgrid[0:3, 0:2].shape == (2, 3, 2) and [a.shape for a in mnp.ogrid[0:3, 0:2]] == [(3, 1), (1, 2)]
    assert mnp.mgrid[0:1:5j].tolist() == [0, 0.25, 0.5, 0.75, 1.0]
    p = np.array([0, 0.5, 6.5, 7.0], np.float32)
    np.testing.assert_allclose(mnp.unwrap(ms.Tensor(p)).numpy(), np.unwrap(p), rtol=1e-5)
    assert mnp.promote_types(ms.int32, ms.float32) == torch.float32
    q, r = mnp.divmod_(ms.Tensor([7, -7]), 2)
    assert q.tolist() == [3, -4] and r.tolist() == [1, 1]
    assert mnp.fft.fft(ms.Tensor([1., 0., 0., 0.])).shape == (4,) and mnp.size(ms.Tensor([[1, 2]]), 1) == 2
    assert mnp.matrix_power(ms.Tensor([[1., 1.], [0., 1.]]), 3).tolist() == [[1, 3], [0, 1]]
    rows, cols = mnp.tril_indices_from(ms.Tensor(np.zeros((3, 3))))
    assert rows.tolist() == [0, 1, 1, 2, 2, 2] and cols.tolist() == [0, 0, 1, 0, 1, 2]


def test_small_methods_of_core_classes(tmp_path):
    import threading

    import mindspore_b200.dataset as ds
    net = _Mlp()
    assert net.create_time == net.create_time and net.pipeline_segment == -1
    net.pipeline_segment = 2
    assert net.pipeline_segment == 2
    with pytest.raises(ValueError):
        net.pipeline_segment = -3
    net.check_names_and_refresh_name()
    net.set_param_fl(push_to_server=True)
    assert net.fc1.weight.push_weight_to_server is True and net.fc1.weight.requires_aggr is True
    p = net.fc1.weight
    assert p.key == p.key and p.cache_shape == ()
    p.cache_shape = [4, 2]
    assert p.cache_shape == (4, 2)
    opt = nn.SGD(net.trainable_params(), learning_rate=0.25)
    assert float(opt.get_lr_parameter(p)) == 0.25 and opt.target == "CPU"
    with pytest.raises(ValueError):
        opt.target = "TPU"
    data = ds.NumpySlicesDataset({"x": np.arange(6)}, shuffle=False)
    assert not data.is_shuffled() and data.shuffle(4).is_shuffled() and data.shard(2, 0).is_sharded()
    assert data.batch(2).to_json()["op_type"] == "Batch"
    data.set_init_step(3)
    assert data.get_init_step() == 3
    gated = data.sync_wait("go", num_batch=2)
    assert gated.is_sync() and list(gated.get_sync_notifiers()) == ["go"]
    seen = []
    t = threading.Thread(target=lambda: seen.extend(int(r["x"]) for r in gated.create_dict_iterator(output_numpy=True)))
    ds.config.set_callback_timeout(5)
    t.start()
    for _ in range(2):
        gated.sync_update("go")
    t.join(10)
    ds.config.set_callback_timeout(60)
    assert seen == [0, 1, 2, 3, 4, 5]
    with pytest.raises(RuntimeError):
        data.sync_update("nope")
    out = tmp_path / "prof"
    out.mkdir()
    (out / "kernel_time_0.csv").write_text("name,calls,total_us,mean_us,share\nk,2,10.0,5.0,1.0\n")
    rows = ms.Profiler.offline_analyse(str(out))
    assert rows[0][0]["name"] == "k" and rows[0][0]["calls"] == "2"
