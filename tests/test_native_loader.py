"""Native batch pipeline (csrc/host/data_pipeline.cpp): ordering, shuffle determinism, sharding, remainder handling
and the image transform against a numpy restatement."""
import numpy as np
import torch

from mindspore_b200.dataset.native_loader import NativeBatchLoader


def _cols(n=103):
    x = np.arange(n * 6, dtype=np.float32).reshape(n, 2, 3)
    y = np.arange(n, dtype=np.int64)
    return {"x": x, "y": y}


def test_sequential_batches_in_order():
    cols = _cols()
    ld = NativeBatchLoader(cols, batch_size=10, shuffle=False, drop_remainder=False, num_parallel_workers=3)
    assert ld.get_dataset_size() == 11
    seen = []
    for b in ld.epoch(0):
        assert b["x"].shape[1:] == (2, 3) and b["x"].dtype == torch.float32
        assert torch.equal(b["x"], torch.from_numpy(cols["x"][b["y"].numpy()]))
        seen += b["y"].tolist()
    assert seen == list(range(103))
    ld.close()


def test_shuffle_is_a_permutation_and_reproducible():
    cols = _cols(64)
    a = NativeBatchLoader(cols, batch_size=8, shuffle=True, seed=5, num_parallel_workers=4)
    b = NativeBatchLoader(cols, batch_size=8, shuffle=True, seed=5, num_parallel_workers=1)
    e0 = [v for bt in a.epoch(0) for v in bt["y"].tolist()]
    e1 = [v for bt in a.epoch(1) for v in bt["y"].tolist()]
    f0 = [v for bt in b.epoch(0) for v in bt["y"].tolist()]
    assert sorted(e0) == list(range(64)) and sorted(e1) == list(range(64))
    assert e0 != list(range(64)) and e0 != e1 and e0 == f0
    a.close(); b.close()


def test_shards_partition_the_rows():
    cols = _cols(50)
    got = []
    for sid in range(3):
        ld = NativeBatchLoader(cols, batch_size=4, shuffle=True, seed=1, num_shards=3, shard_id=sid,
                               drop_remainder=False)
        got.append([v for bt in ld.epoch(2) for v in bt["y"].tolist()])
        ld.close()
    assert sorted(sum(got, [])) == list(range(50))
    assert all(len(set(g)) == len(g) for g in got)


def test_restart_epoch_midway():
    ld = NativeBatchLoader(_cols(40), batch_size=4, prefetch=2, num_parallel_workers=2)
    it = ld.epoch(0)
    next(it); next(it)
    again = [v for bt in ld.epoch(0) for v in bt["y"].tolist()]
    assert again == list(range(40))
    ld.close()


def test_image_transform_matches_numpy():
    rng = np.random.default_rng(0)
    img = rng.integers(0, 256, size=(12, 10, 9, 3), dtype=np.uint8)
    lab = np.arange(12, dtype=np.int32)
    mean, std = [10.0, 20.0, 30.0], [2.0, 4.0, 8.0]
    ld = NativeBatchLoader({"image": img, "label": lab}, batch_size=4, num_parallel_workers=2)
    ld.set_image_transform("image", out_size=(10, 9), flip=False, mean=mean, std=std)      # no crop, no flip
    for b in ld.epoch(0):
        ref = (img[b["label"].numpy()].astype(np.float32) - np.array(mean, np.float32)) / np.array(std, np.float32)
        ref = ref.transpose(0, 3, 1, 2)
        assert b["image"].shape == (4, 3, 10, 9)
        np.testing.assert_allclose(b["image"].numpy(), ref, rtol=1e-6, atol=1e-6)
    ld.close()
    # crop + flip: every output is some crop of the source, possibly mirrored
    ld = NativeBatchLoader({"image": img, "label": lab}, batch_size=3, seed=3)
    ld.set_image_transform("image", out_size=(6, 5), flip=True)
    flips = 0
    for b in ld.epoch(0):
        for im, lb in zip(b["image"].numpy(), b["label"].tolist()):
            src = img[lb].astype(np.float32).transpose(2, 0, 1)
            found = None
            for y0 in range(10 - 6 + 1):
                for x0 in range(9 - 5 + 1):
                    win = src[:, y0:y0 + 6, x0:x0 + 5]
                    if np.array_equal(win, im):
                        found = "plain"
                    elif np.array_equal(win[:, :, ::-1], im):
                        found = "flip"
            assert found is not None
            flips += found == "flip"
    assert 0 < flips < 12
    ld.close()
