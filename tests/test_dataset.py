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


def _write_idx(path, arr):
    import struct
    with open(path, "wb") as f:
        f.write(struct.pack(">HBB", 0, 8, arr.ndim) + struct.pack(">" + "I" * arr.ndim, *arr.shape) + arr.tobytes())


def test_source_datasets_and_samplers(tmp_path):
    import numpy as np
    import mindspore_b200.dataset as ds
    rng = np.random.default_rng(0)
    imgs = rng.integers(0, 256, (20, 28, 28), dtype=np.uint8)
    labs = (np.arange(20) % 4).astype(np.uint8)
    _write_idx(str(tmp_path / "train-images-idx3-ubyte"), imgs)
    _write_idx(str(tmp_path / "train-labels-idx1-ubyte"), labs)
    mn = ds.MnistDataset(str(tmp_path), usage="train", shuffle=False)
    rows = list(mn.create_dict_iterator(output_numpy=True, num_epochs=1))
    assert len(rows) == 20 and rows[3]["image"].shape == (28, 28, 1) and int(rows[3]["label"]) == 3
    assert np.array_equal(rows[5]["image"][..., 0], imgs[5])
    # samplers
    sub = ds.MnistDataset(str(tmp_path), usage="train", sampler=ds.SubsetSampler([4, 2, 9]))
    assert [int(r["label"]) for r in sub.create_dict_iterator(output_numpy=True, num_epochs=1)] == [0, 2, 1]
    parts = []
    for sid in range(3):
        d = ds.MnistDataset(str(tmp_path), usage="train", sampler=ds.DistributedSampler(3, sid, shuffle=False))
        parts.append([int(np.where((imgs == r["image"][..., 0]).all((1, 2)))[0][0])
                      for r in d.create_dict_iterator(output_numpy=True, num_epochs=1)])
    assert all(len(p) == 7 for p in parts) and set(sum(parts, [])) == set(range(20))
    pk = ds.MnistDataset(str(tmp_path), usage="train", sampler=ds.PKSampler(2))
    assert sorted(int(r["label"]) for r in pk.create_dict_iterator(output_numpy=True, num_epochs=1)) == [0, 0, 1, 1, 2, 2, 3, 3]
    w = ds.WeightedRandomSampler([0, 0, 1.0] + [0] * 17, num_samples=5).bind(20)
    assert list(w) == [2] * 5
    rs = ds.RandomSampler(num_samples=6).bind(20)
    assert len(set(rs)) == 6
    # cifar-10 binary
    cdir = tmp_path / "cifar"
    cdir.mkdir()
    rec = np.zeros((5, 3073), np.uint8)
    rec[:, 0] = [1, 2, 3, 4, 5]
    rec[:, 1:] = rng.integers(0, 256, (5, 3072), dtype=np.uint8)
    rec.tofile(str(cdir / "data_batch_1.bin"))
    c = list(ds.Cifar10Dataset(str(cdir), usage="train", shuffle=False).create_dict_iterator(output_numpy=True, num_epochs=1))
    assert len(c) == 5 and c[0]["image"].shape == (32, 32, 3) and int(c[4]["label"]) == 5
    assert np.array_equal(c[0]["image"][:, :, 0].reshape(-1), rec[0, 1:1025])
    # image folder (decoded with PIL)
    from PIL import Image
    for cls in ("cat", "dog"):
        (tmp_path / "img" / cls).mkdir(parents=True)
        for k in range(2):
            Image.fromarray(rng.integers(0, 256, (6, 5, 3), dtype=np.uint8)).save(str(tmp_path / "img" / cls / ("%d.png" % k)))
    f = ds.ImageFolderDataset(str(tmp_path / "img"), decode=True, shuffle=False)
    fr = list(f.create_dict_iterator(output_numpy=True, num_epochs=1))
    assert [int(r["label"]) for r in fr] == [0, 0, 1, 1] and fr[0]["image"].shape == (6, 5, 3)
    assert f.get_class_indexing() == {"cat": 0, "dog": 1}
    # text and csv
    (tmp_path / "a.txt").write_text("hello world\n\nsecond line\n")
    t = [str(r["text"]) for r in ds.TextFileDataset(str(tmp_path / "a.txt")).create_dict_iterator(output_numpy=True, num_epochs=1)]
    assert t == ["hello world", "second line"]
    (tmp_path / "a.csv").write_text("x,y,name\n1,2.5,a\n3,,b\n")
    rows = list(ds.CSVDataset(str(tmp_path / "a.csv"), column_defaults=[0, 0.5, ""]).create_dict_iterator(output_numpy=True, num_epochs=1))
    assert int(rows[1]["x"]) == 3 and float(rows[1]["y"]) == 0.5 and str(rows[0]["name"]) == "a"


def test_vision_and_general_transforms():
    import io
    import numpy as np
    from PIL import Image
    import mindspore_b200.dataset.transforms as T
    import mindspore_b200.dataset.vision as V
    img = np.random.default_rng(0).integers(0, 256, (20, 30, 3), dtype=np.uint8)
    buf = io.BytesIO()
    Image.fromarray(img).save(buf, format="PNG")
    assert np.array_equal(V.Decode()(np.frombuffer(buf.getvalue(), np.uint8)), img)
    assert V.RandomResizedCrop(8)(img).shape == (8, 8, 3) and V.RandomCropDecodeResize(6)(
        np.frombuffer(buf.getvalue(), np.uint8)).shape == (6, 6, 3)
    t = V.ToTensor()(img)
    assert t.shape == (3, 20, 30) and t.dtype == np.float32 and t.max() <= 1.0
    assert V.Pad((1, 2))(img).shape == (24, 32, 3) and V.Pad(2, padding_mode=V.Border.REFLECT)(img)[0, 0, 0] == img[2, 2, 0]
    assert V.Rotate(90, expand=True)(img).shape == (30, 20, 3)
    assert np.array_equal(V.HorizontalFlip()(img), img[:, ::-1]) and np.array_equal(V.VerticalFlip()(img), img[::-1])
    assert np.array_equal(V.Crop((2, 3), (4, 5))(img), img[2:6, 3:8]) and np.array_equal(V.Invert()(img), 255 - img)
    g = V.Grayscale(3)(img)
    assert g.shape == (20, 30, 3) and np.array_equal(g[..., 0], g[..., 2])
    assert np.array_equal(V.AdjustBrightness(1.0)(img), img) and V.AdjustBrightness(0.0)(img).max() == 0
    assert V.AdjustHue(0.2)(img).shape == img.shape and V.RandomColorAdjust(0.2, 0.2, 0.2, 0.1)(img).shape == img.shape
    flat = np.full((9, 9, 1), 7, np.uint8)
    assert np.array_equal(V.GaussianBlur(3)(flat), flat)
    e = V.RandomErasing(prob=1.0, value=-1.0)(t)
    assert (e == -1.0).any() and e.shape == t.shape
    x, y = V.MixUpBatch()(np.stack([img] * 4), np.eye(4))
    assert x.shape == (4, 20, 30, 3) and np.allclose(y.sum(1), 1)
    x, y = V.CutMixBatch("NCHW")(np.zeros((4, 3, 8, 8)), np.eye(4))
    assert x.shape == (4, 3, 8, 8) and np.allclose(y.sum(1), 1)
    assert T.Mask("gt", 2)(np.array([1, 2, 3, 4])).tolist() == [False, False, True, True]
    assert T.PadEnd([5], -1)(np.array([1, 2])).tolist() == [1, 2, -1, -1, -1]
    u, idx, cnt = T.Unique()(np.array([3, 1, 3, 2]))
    assert u.tolist() == [3, 1, 2] and idx.tolist() == [0, 1, 0, 2] and cnt.tolist() == [2, 1, 1]
    assert T.Concatenate(0, prepend=[0], append=[9])(np.array([1, 2])).tolist() == [0, 1, 2, 9]
    assert T.Slice(slice(1, 3))(np.arange(5)).tolist() == [1, 2] and T.Fill(3)(np.zeros(2)).tolist() == [3, 3]
    assert T.RandomApply([lambda v: v + 1], prob=1.0)(np.array([1])).tolist() == [2]
    assert T.RandomChoice([lambda v: v * 2])(np.array([2])).tolist() == [4]


def test_concat_filter_flat_map_padded_and_bucket_batches(tmp_path):
    import numpy as np
    import mindspore_b200.dataset as ds
    a = ds.NumpySlicesDataset(np.arange(5), ["x"], shuffle=False)
    b = ds.NumpySlicesDataset(np.arange(10, 13), ["x"], shuffle=False)
    both = a + b
    vals = lambda d: [int(r["x"]) for r in d.create_dict_iterator(output_numpy=True, num_epochs=1)]
    assert both.get_dataset_size() == 8 and vals(both) == [0, 1, 2, 3, 4, 10, 11, 12]
    assert vals(a.concat([b, b]))[-3:] == [10, 11, 12]
    assert vals(both.filter(lambda x: x % 2 == 0)) == [0, 2, 4, 10, 12]
    fm = a.flat_map(lambda x: ds.NumpySlicesDataset(np.array([x, x]), ["x"], shuffle=False))
    assert vals(fm) == [0, 0, 1, 1, 2, 2, 3, 3, 4, 4]
    assert vals(a.apply(lambda d: d.take(2))) == [0, 1]
    tr, te = a.split([3, 2], randomize=False)
    assert vals(tr) == [0, 1, 2] and vals(te) == [3, 4]
    p1, p2 = both.split([0.5, 0.5])
    assert sorted(vals(p1) + vals(p2)) == sorted(vals(both))
    seqs = [np.arange(n, dtype=np.int32) for n in (2, 5, 3, 1, 4, 6)]
    g = ds.GeneratorDataset([(s,) for s in seqs], ["tok"], shuffle=False)
    pb = list(g.padded_batch(3, pad_info={"tok": ([None], -1)}).create_dict_iterator(output_numpy=True, num_epochs=1))
    assert pb[0]["tok"].shape == (3, 5) and pb[0]["tok"][0].tolist() == [0, 1, -1, -1, -1] and pb[1]["tok"].shape == (3, 6)
    bb = list(g.bucket_batch_by_length(["tok"], [3, 5], [2, 2, 2], pad_to_bucket_boundary=True)
              .create_dict_iterator(output_numpy=True, num_epochs=1))
    shapes = sorted(tuple(x["tok"].shape) for x in bb)
    assert shapes == [(2, 2), (2, 4), (2, 6)]
    path = str(tmp_path / "saved.mindrecord")
    ds.NumpySlicesDataset({"x": np.arange(4, dtype=np.int32), "y": np.arange(4, dtype=np.float32) * 0.5},
                          shuffle=False).save(path)
    back = ds.MindDataset(path, shuffle=False)
    rows = list(back.create_dict_iterator(output_numpy=True, num_epochs=1))
    assert [int(r["x"]) for r in rows] == [0, 1, 2, 3] and float(rows[3]["y"]) == 1.5


def test_config_settings_iterators_and_sampler_selection(tmp_path):
    import json
    cfg = ds.config
    cfg.set_enable_shared_mem(False)
    assert cfg.get_enable_shared_mem() is False and cfg.get_callback_timeout() == 60
    with pytest.raises(TypeError):
        cfg.set_numa_enable(1)
    with pytest.raises(ValueError):
        cfg.set_monitor_sampling_interval(0)
    cfg.set_error_samples_mode(cfg.ErrorSamplesMode.SKIP)
    assert cfg.get_error_samples_mode() == 2
    (tmp_path / "c.json").write_text(json.dumps({"numParallelWorkers": 3, "seed": 11, "prefetchSize": 5}))
    old = (cfg.get_num_parallel_workers(), cfg.get_seed(), cfg.get_prefetch_size())
    cfg.load(str(tmp_path / "c.json"))
    assert (cfg.get_num_parallel_workers(), cfg.get_seed(), cfg.get_prefetch_size()) == (3, 11, 5)
    cfg.set_num_parallel_workers(old[0]), cfg.set_seed(old[1]), cfg.set_prefetch_size(old[2])
    cfg.set_enable_shared_mem(True)
    data = ds.NumpySlicesDataset({"x": np.arange(4)}, shuffle=False)
    it = data.create_dict_iterator(num_epochs=2, output_numpy=True)
    assert isinstance(it, ds.DictIterator) and it.get_col_names() == ["x"]
    assert [int(r["x"]) for r in it] == [0, 1, 2, 3] and [int(r["x"]) for r in it] == [0, 1, 2, 3]
    with pytest.raises(RuntimeError):
        list(it)                                               # a third epoch was not asked for
    tup = data.create_tuple_iterator(output_numpy=True)
    assert int(next(tup)[0]) == 0 and isinstance(tup, ds.TupleIterator)
    dummy = ds.DummyIterator(data, "dict", output_numpy=True)
    assert int(next(dummy)["x"]) == 0 and int(next(dummy)["x"]) == 0
    from mindspore_b200.dataset import samplers
    assert isinstance(samplers.select_sampler(None, None, None, None, None), samplers.RandomSampler)
    assert isinstance(samplers.select_sampler(None, None, False, None, None), samplers.SequentialSampler)
    assert isinstance(samplers.select_sampler(None, None, None, 2, 0), samplers.DistributedSampler)
    assert samplers.select_sampler(2, [3, 1, 2], None, None, None).bind(4).indices().tolist() == [3, 1]
    with pytest.raises(RuntimeError):
        samplers.select_sampler(None, samplers.SequentialSampler(), True, None, None)
