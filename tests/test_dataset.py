import numpy as np
import pytest
import torch

import mindspore_b200 as ms
import mindspore_b200.dataset as ds
from mindspore_b200 import nn


def test_pipeline_ops_and_sizes():
    data = {"x": np.arange(20, dtype=np.float32).reshape(10, 2), "y": np.arange(10, dtype=np.int32)}
    d = ds.NumpySlicesDataset(data, shuffle=False)
    assert d.get_col_names() == ["x", "y"] and d.get_dataset_size() == 10
    d2 = d.map(lambda x: x * 2, input_columns="x", num_parallel_workers=2).batch(4, drop_remainder=False)
    assert d2.get_dataset_size() == 3
    rows = list(d2.create_dict_iterator(output_numpy=True))
    assert rows[0]["x"].shape == (4, 2) and rows[-1]["x"].shape == (2, 2)
    np.testing.assert_array_equal(np.concatenate([r["y"] for r in rows]), np.arange(10))
    np.testing.assert_array_equal(rows[0]["x"][1], [4, 6])
    assert d.shard(3, 1).get_dataset_size() == 3
    assert [int(r[1]) for r in d.shard(3, 1).create_tuple_iterator(output_numpy=True)] == [1, 4, 7]
    assert d.take(3).repeat(2).get_dataset_size() == 6
    assert len(list(d.skip(8))) == 2
    sh = sorted(int(r[1]) for r in d.shuffle(4).create_tuple_iterator(output_numpy=True))
    assert sh == list(range(10))
    z = ds.zip((d.project("x"), d.project("y").rename("y", "label")))
    assert z.get_col_names() == ["x", "label"]
    assert len(list(z.prefetch(2))) == 10


def test_generator_sources_and_sharding():
    def gen():
        for i in range(7):
            yield np.array([i], np.int32), np.array(i * i, np.int64)
    g = ds.GeneratorDataset(gen, ["a", "b"], num_shards=2, shard_id=1)
    assert [int(r[0][0]) for r in g.create_tuple_iterator(output_numpy=True)] == [1, 3, 5]
    with pytest.raises(ValueError):
        ds.GeneratorDataset(gen, None)


def test_record_file_roundtrip(tmp_path):
    path = str(tmp_path / "train.mindrecord")
    w = ds.FileWriter(path)
    w.add_schema({"image": {"type": "bytes"}, "label": {"type": "int32"}, "feat": {"type": "float32", "shape": [-1]}})
    rows = [{"image": bytes([i] * (i + 1)), "label": i, "feat": np.arange(i + 2, dtype=np.float32)} for i in range(5)]
    w.write_raw_data(rows)
    w.commit()
    r = ds.FileReader(path)
    assert len(r) == 5
    row = r.read(3)
    assert bytes(row["image"]) == bytes([3] * 4) and int(row["label"]) == 3
    np.testing.assert_array_equal(row["feat"], np.arange(5, dtype=np.float32))
    md = ds.MindDataset(path, columns_list=["label", "feat"], shuffle=False)
    assert [int(x[0]) for x in md.create_tuple_iterator(output_numpy=True)] == [0, 1, 2, 3, 4]


def test_model_train_consumes_dataset():
    ms.set_context(device_target="CPU")
    torch.manual_seed(0)
    ms.set_seed(0)
    rng = np.random.default_rng(0)
    x = rng.standard_normal((64, 8)).astype(np.float32)
    w = rng.standard_normal((8, 1)).astype(np.float32)
    y = x @ w
    data = ds.NumpySlicesDataset({"x": x, "y": y}, shuffle=True).batch(16)
    net = nn.Dense(8, 1)
    model = ms.Model(net, nn.MSELoss(), nn.Adam(net.trainable_params(), 0.05))
    model.train(60, data, dataset_sink_mode=False)
    pred = net(ms.Tensor(x)).detach().numpy()
    assert float(((pred - y) ** 2).mean()) < 0.1
