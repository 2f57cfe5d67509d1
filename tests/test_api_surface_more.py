"""Smaller public pieces: Bayesian layers, time-distributed / parameter-update wrappers, TensorArray, THOR conversion,
dataset debug hooks and helpers, the shard layer of mindrecord, and the import paths that lead to them."""
import importlib
import os

import numpy as np
import pytest
import torch

import mindspore_b200 as ms
from mindspore_b200 import nn, ops


def test_bayesian_layers_kl_and_training_loss():
    from torch.distributions import Normal, kl_divergence
    from mindspore_b200.nn.probability import bnn_layers as B
    ms.set_seed(0)
    dense = B.DenseReparam(3, 2)
    want = kl_divergence(Normal(dense.weight_posterior.mean.detach(), dense.weight_posterior.sd_value().detach()),
                         Normal(0.0, 0.1)).sum() + \
        kl_divergence(Normal(dense.bias_posterior.mean.detach(), dense.bias_posterior.sd_value().detach()),
                      Normal(0.0, 0.1)).sum()
    assert abs(float(dense.compute_kl_loss()) - float(want)) < 1e-3 * float(want)

    class Net(nn.Cell):
        def __init__(self):
            super().__init__()
            self.conv = B.ConvReparam(1, 2, 3, stride=2, has_bias=True)
            self.flat = nn.Flatten()
            self.local = B.DenseLocalReparam(2 * 4 * 4, 3, activation="relu")
            self.head = B.DenseReparam(3, 2)

        def construct(self, x):
            return self.head(self.local(self.flat(self.conv(x))))

    net = Net()
    x = ms.Tensor(np.random.RandomState(0).randn(4, 1, 8, 8).astype(np.float32))
    assert net(x).shape == (4, 2)
    assert not np.allclose(net(x).detach().numpy(), net(x).detach().numpy())       # weights are sampled per call
    label = ms.Tensor(np.array([0, 1, 1, 0]))
    cell = B.WithBNNLossCell(net, nn.SoftmaxCrossEntropyWithLogits(sparse=True, reduction="mean"), 1, 1e-3)
    assert len(cell.kl_loss) == 3 and cell.backbone_network is net
    loss = cell(x, label)
    loss.backward()
    grads = [p.grad for p in net.trainable_params()]
    assert len(grads) == 12 and all(g is not None and torch.isfinite(g).all() for g in grads)
    # the local reparameterisation has the mean of the plain one
    big = ms.Tensor(np.ones((4000, 3), np.float32))
    local = B.DenseLocalReparam(3, 2, has_bias=False)
    mean = (big[:1] @ local.weight_posterior.mean.t()).detach()
    assert torch.allclose(local(big).detach().mean(0), mean[0], atol=2e-3)
    with pytest.raises(TypeError):
        B.NormalPosterior("w", [2, 2], loc_std=-1)
    with pytest.raises(ValueError):
        B.WithBNNLossCell(net, None, dnn_factor=-1)


def test_time_distributed_parameter_update_tensor_array():
    x = ms.Tensor(np.random.RandomState(1).randn(2, 3, 4).astype(np.float32))
    dense = nn.Dense(4, 5)
    folded = nn.TimeDistributed(dense, time_axis=1, reshape_with_axis=0)(x)
    looped = nn.TimeDistributed(dense, time_axis=1)(x)
    assert folded.shape == (2, 3, 5) and np.allclose(folded.detach().numpy(), looped.detach().numpy(), atol=1e-6)
    with pytest.raises(ValueError):
        nn.TimeDistributed(dense, 1)(ms.Tensor(np.ones((2, 4), np.float32)))
    lr = ms.Parameter(ms.Tensor(np.zeros(2, np.float32)), name="lr")
    nn.ParameterUpdate(lr)(ms.Tensor(np.array([0.5, 0.25], np.float32)))
    assert lr.tolist() == [0.5, 0.25]
    with pytest.raises(TypeError):
        nn.ParameterUpdate(ms.Tensor(np.zeros(2, np.float32)))

    ta = nn.TensorArray(ms.float32, (2,), dynamic_size=True)
    ta.write(0, torch.tensor([1.0, 2.0]))
    ta.write(2, torch.tensor([5.0, 6.0]))
    assert ta.size() == 3 and ta.read(1).tolist() == [0.0, 0.0] and ta.stack().shape == (3, 2)
    with pytest.raises(TypeError):
        ta.write(1, torch.tensor([1, 2]))
    ta.clear()
    assert ta.size() == 0
    fixed = nn.TensorArray(ms.int64, (), dynamic_size=False, size=2)
    fixed.write(1, torch.tensor(7))
    with pytest.raises(ValueError):
        fixed.write(2, torch.tensor(7))
    fixed.close()
    with pytest.raises(RuntimeError):
        fixed.size()
    lin = nn.Linear(4, 3, bias=False)
    assert lin.bias is None and lin(ms.Tensor(np.ones((2, 4), np.float32))).shape == (2, 3)


def test_thor_conversion_shares_the_weights():
    from mindspore_b200.models.lenet import LeNet5
    from mindspore_b200.train import ConvertModelUtils, ConvertNetUtils, Model, ModelThor
    net = LeNet5()
    x = ms.Tensor(np.random.RandomState(2).randn(2, 1, 32, 32).astype(np.float32))
    before, weight = net(x).detach().numpy(), net.fc1.weight
    ConvertNetUtils().convert_to_thor_net(net)
    assert type(net.fc1).__name__ == "DenseThor" and type(net.conv1).__name__ == "Conv2dThor"
    assert net.fc1.weight is weight and np.allclose(net(x).detach().numpy(), before)
    names = [p.name for p in net.get_parameters()]
    assert "fc1.weight" in names and "fc1.matrix_a" in names and "conv2.matrix_g" in names
    seq = nn.SequentialCell([nn.Dense(4, 4), nn.ReLU(), nn.Dense(4, 2)])
    ConvertNetUtils().convert_to_thor_net(seq)
    assert [type(c).__name__ for c in seq.cell_list] == ["DenseThor", "ReLU", "DenseThor"]
    loss = nn.SoftmaxCrossEntropyWithLogits(sparse=True, reduction="mean")
    sgd = nn.Momentum(net.trainable_params(), 0.1, 0.9)
    model = Model(net, loss, sgd)
    assert ConvertModelUtils.convert_to_thor_model(model, net, loss, sgd) is model
    thor = nn.thor(net, 0.01, 0.03, 0.9)
    assert isinstance(ConvertModelUtils.convert_to_thor_model(model, net, loss, thor), ModelThor)


def test_dataset_debug_hooks_and_helpers(tmp_path, capsys):
    import mindspore_b200.dataset as ds
    from mindspore_b200.dataset import debug
    from mindspore_b200.dataset.utils import LineReader, imshow_det_bbox

    class Count(debug.DebugHook):
        calls = []

        def compute(self, *args):
            Count.calls.append((self.prev_op_name, self.is_first_op, [np.asarray(c).tolist() for c in args[0]]))

    data = ds.NumpySlicesDataset({"x": np.arange(4, dtype=np.float32).reshape(2, 2)}, shuffle=False)
    ds.config.set_debug_mode(True, [Count(), debug.PrintMetaDataHook()])
    try:
        def plus_one(x):
            return x + 1
        rows = [r["x"].tolist() for r in data.map([plus_one, lambda x: x * 2], ["x"], num_parallel_workers=4)
                .create_dict_iterator(output_numpy=True)]
    finally:
        ds.config.set_debug_mode(False)
    assert rows == [[2.0, 4.0], [6.0, 8.0]]
    assert Count.calls[0] == ("plus_one", True, [[0.0, 1.0]]) and Count.calls[1] == ("plus_one", False, [[1.0, 2.0]])
    assert len(Count.calls) == 6
    out = capsys.readouterr().out
    assert "[Dataset debugger] Print the [INPUT] of the operation [plus_one]." in out
    assert "The dtype is [float32]. The shape is [(2,)]." in out
    with pytest.raises(TypeError):
        ds.config.set_debug_mode(True, [object()])
    assert ds.config.get_debug_mode() is False

    text = tmp_path / "lines.txt"
    text.write_bytes("first\nsecond line\n\nlast without end".encode())
    reader = LineReader(str(text))
    assert len(reader) == 4 and reader[2] == "second line" and reader.readline(3) == "" and reader[4].startswith("last")
    with pytest.raises(ValueError):
        reader.readline(5)
    reader.close()

    pic = imshow_det_bbox(np.zeros((3, 32, 32), np.uint8), np.array([[2, 2, 10, 10, 0.9], [20, 20, 4, 4, 0.1]]),
                          np.array([1, 0]), class_names=["cat", "dog"], score_threshold=0.5,
                          segm=np.ones((2, 32, 32), bool), out_file=str(tmp_path / "boxes.png"))
    assert pic.shape == (32, 32, 3) and tuple(pic[2, 5]) == (0, 255, 0) and tuple(pic[20, 22]) != (0, 255, 0)
    assert os.path.getsize(tmp_path / "boxes.png") > 0
    with pytest.raises(ValueError):
        imshow_det_bbox(np.zeros((32, 32), np.uint8), np.zeros((1, 4)), np.zeros(1))


def test_shard_layer_and_index_rebuild(tmp_path):
    from mindspore_b200.dataset import mindrecord as MR
    from mindspore_b200.dataset import mindrecord_format as F
    path = str(tmp_path / "t.mindrecord")
    head = MR.ShardHeader()
    head.add_schema(MR.ShardHeader.build_schema({"label": {"type": "int32"}, "name": {"type": "string"},
                                                 "img": {"type": "bytes"}, "v": {"type": "int64", "shape": [-1]}}, "d"))
    head.add_index_fields(["label", "name"])
    assert head.blob_fields == ["img", "v"]
    w = MR.ShardWriter()
    w.open([path])
    w.set_page_size(1 << 15)
    w.set_shard_header(head)
    w.write_raw_data([{"label": i, "name": "n%d" % i, "img": bytes([i]) * 9000, "v": np.arange(i + 1)}
                      for i in range(10)])
    w.commit()
    before = F.read_index(path + ".db")
    assert len({r[5] for r in before}) > 1                   # several blob pages: the rows span row groups
    os.remove(path + ".db")
    gen = MR.ShardIndexGenerator(path)
    gen.build()
    gen.write_to_db()
    assert F.read_index(path + ".db") == before
    r = MR.ShardReader()
    r.open(path)
    r.launch()
    first = r.get_next()
    assert r.len() == 10 and int(first["label"]) == 0 and r.get_blob_fields() == ["img", "v"]
    assert r.get_header().index_fields == ["label", "name"]
    r.close()
    seg = MR.ShardSegment()
    seg.open(path)
    seg.set_category_field("label")
    assert '"key": "label"' in seg.read_category_info()


def test_reference_import_paths_resolve():
    for path, names in (
            ("nn.layer.basic", ["Dense", "Dropout"]), ("nn.layer.activation", ["ReLU", "get_activation"]),
            ("nn.layer.normalization", ["LayerNorm"]), ("nn.layer.timedistributed", ["TimeDistributed"]),
            ("nn.metrics", ["Accuracy", "get_metric_fn"]), ("nn.extend", ["Linear"]),
            ("nn.extend.layer.normalization", ["LayerNorm"]), ("nn.reinforcement", ["TensorArray"]),
            ("nn.probability.bnn_layers.dense_variational", ["DenseReparam"]),
            ("nn.optim.optimizer", ["Optimizer"]), ("ops.extend.nn_func", ["leaky_relu_ext"]),
            ("mindrecord.shardwriter", ["ShardWriter"]), ("mindrecord.tools.cifar10", ["Cifar10"]),
            ("mindrecord.config", ["set_enc_key"]), ("boost.grad_freeze", ["FreezeOpt"]),
            ("train.train_thor", ["ConvertNetUtils", "ConvertModelUtils"]),
            ("train.train_thor.model_thor", ["ModelThor"]), ("common.sparse_tensor", ["RowTensor", "COOTensor"]),
            ("dataset.core.config", ["set_seed", "get_num_parallel_workers", "ErrorSamplesMode"]),
            ("dataset.debug", ["PrintDataHook"]), ("dataset.utils", ["LineReader"]),
            ("dataset.callback", ["DSCallback", "WaitedDSCallback"]),
            ("dataset.engine", ["MnistDataset", "CocoDataset", "DistributedSampler"]),
            ("parallel.checkpoint_transform", ["load_segmented_checkpoints"]),
            ("ops.composite", ["tail", "hyper_add", "zeros_like", "matmul", "_Grad", "ms_next"]),
            ("experimental.optim.optimizer", ["Optimizer"]), ("context", ["STRICT", "COMPATIBLE", "LAX"])):
        mod = importlib.import_module("mindspore_b200." + path)
        for n in names:
            assert hasattr(mod, n), (path, n)
    from mindspore_b200.ops import composite as C
    assert C.tail((1, 2, 3)) == (2, 3) and C.hyper_add((1, (2, 3)), (10, (20, 30))) == (11, (22, 33))
    assert C.ms_next((4, 5)) == (4, (5,)) and C.ms_hasnext(()) is False and C.iter_converter({"a": 1}) == ("a",)

    @C.add_flags(core=True)
    def f():
        return 1
    assert f._func_graph_flags == {"core": True}
    assert float(ops.leaky_relu_ext(ms.Tensor(np.array([-2.0], np.float32)), 0.5)[0]) == -1.0
    with ms.common._no_grad():
        y = ms.Parameter(ms.Tensor(np.ones(2, np.float32)), name="p") * 2
    assert not y.requires_grad and repr(ms.common._null) == "null" and not ms.common._null


def test_sampler_replacement_sparse_add_and_append(tmp_path):
    import mindspore_b200.dataset as ds
    from mindspore_b200.common import initializer as init
    from mindspore_b200.dataset import mindrecord as MR
    data = ds.NumpySlicesDataset({"x": np.arange(10)}, shuffle=False)
    data.use_sampler(ds.SequentialSampler(2, 3))
    assert [int(r["x"]) for r in data.create_dict_iterator(output_numpy=True)] == [2, 3, 4]
    data.add_sampler(ds.SubsetSampler([2, 0]))                   # draws from what the sequential sampler yields
    assert [int(r["x"]) for r in data.create_dict_iterator(output_numpy=True)] == [4, 2]
    data.use_sampler(None)
    assert len([1 for _ in data.create_dict_iterator(output_numpy=True)]) == 10

    a = ms.CSRTensor(ms.Tensor(np.array([0, 1, 2]), ms.int64), ms.Tensor(np.array([0, 1]), ms.int64),
                     ms.Tensor(np.array([1.0, 2.0], np.float32)), (2, 2))
    b = ms.CSRTensor(ms.Tensor(np.array([0, 1, 1]), ms.int64), ms.Tensor(np.array([1]), ms.int64),
                     ms.Tensor(np.array([5.0], np.float32)), (2, 2))
    out = a.add(b, 2.0, 1.0)
    assert out.to_dense().tolist() == [[2.0, 5.0], [0.0, 4.0]] and a.itemsize == 4
    assert init.initializer(init.Normal(0.1), (2, 3)).shape == (2, 3) and callable(ms.initializer)

    path = str(tmp_path / "a.mindrecord")
    w = MR.FileWriter(path)
    w.add_schema({"id": {"type": "int64"}})
    w.write_raw_data([{"id": 0}, {"id": 1}])
    w.commit()
    again = MR.FileWriter(str(tmp_path / "unused.mindrecord"))
    again.init_append(path)
    again.write_raw_data([{"id": 2}])
    again.commit()
    assert [int(r["id"]) for r in MR.FileReader(path).get_next()] == [0, 1, 2]
