"""Source datasets on tiny synthetic copies of their on-disk layouts."""
import json
import os
import struct
import wave

import numpy as np
import pytest

import mindspore_b200.dataset as ds


def _rows(d, cols=None):
    return list(d.create_dict_iterator(output_numpy=True, num_epochs=1))


def _idx(path, arr):
    arr = np.asarray(arr, dtype=np.uint8)
    with open(path, "wb") as f:
        f.write(struct.pack(">HBB", 0, 8, arr.ndim) + struct.pack(">" + "I" * arr.ndim, *arr.shape) + arr.tobytes())


def _wav(path, samples, rate=8000):
    with wave.open(str(path), "wb") as w:
        w.setnchannels(1)
        w.setsampwidth(2)
        w.setframerate(rate)
        w.writeframes((np.asarray(samples) * 32767).astype("<i2").tobytes())


def test_idx_and_binary_vision(tmp_path):
    rng = np.random.default_rng(0)
    for prefix, n in (("train", 5), ("t10k", 3)):
        _idx(tmp_path / (prefix + "-images-idx3-ubyte"), rng.integers(0, 255, (n, 28, 28)))
        _idx(tmp_path / (prefix + "-labels-idx1-ubyte"), np.arange(n))
    d = ds.FashionMnistDataset(str(tmp_path), usage="all", shuffle=False)
    rows = _rows(d)
    assert len(rows) == 8 and rows[0]["image"].shape == (28, 28, 1) and [int(r["label"]) for r in rows[:5]] == [0, 1, 2, 3, 4]
    assert ds.KMnistDataset(str(tmp_path), usage="test").get_dataset_size() == 3
    _idx(tmp_path / "emnist-letters-train-images-idx3-ubyte", rng.integers(0, 255, (2, 28, 28)))
    _idx(tmp_path / "emnist-letters-train-labels-idx1-ubyte", [7, 9])
    assert [int(r["label"]) for r in _rows(ds.EMnistDataset(str(tmp_path), "letters", "train", shuffle=False))] == [7, 9]
    with pytest.raises(ValueError):
        ds.EMnistDataset(str(tmp_path), "nope")
    c100 = tmp_path / "c100"
    c100.mkdir()
    rec = np.concatenate([np.array([[3, 42]], np.uint8).repeat(4, 0), rng.integers(0, 255, (4, 3072), dtype=np.uint8)], 1)
    rec.tofile(c100 / "train.bin")
    r = _rows(ds.Cifar100Dataset(str(c100), usage="train", shuffle=False))
    assert len(r) == 4 and int(r[0]["coarse_label"]) == 3 and int(r[0]["fine_label"]) == 42 and r[0]["image"].shape == (32, 32, 3)
    fake = _rows(ds.FakeImageDataset(6, (8, 8, 3), 4, base_seed=1, shuffle=False))
    again = _rows(ds.FakeImageDataset(6, (8, 8, 3), 4, base_seed=1, shuffle=True))
    assert len(fake) == 6 and sorted(int(r["label"]) for r in fake) == sorted(int(r["label"]) for r in again)
    sem = tmp_path / "sem"
    sem.mkdir()
    line = np.concatenate([np.ones(256), np.eye(10)[4]])
    np.savetxt(sem / "semeion.data", np.stack([line, line]))
    assert [int(r["label"]) for r in _rows(ds.SemeionDataset(str(sem), shuffle=False))] == [4, 4]
    usps = tmp_path / "usps"
    usps.mkdir()
    (usps / "usps").write_text("3 1:1.0 256:-1.0\n10 2:0.5\n")
    r = _rows(ds.USPSDataset(str(usps), usage="train", shuffle=False))
    assert [int(x["label"]) for x in r] == [2, 9] and r[0]["image"][0, 0, 0] == 255 and r[0]["image"][15, 15, 0] == 0


def test_folder_json_and_xml_vision(tmp_path):
    root = tmp_path / "cal" / "101_ObjectCategories"
    for c in ("ant", "bee", "BACKGROUND_Google"):
        (root / c).mkdir(parents=True)
        (root / c / "1.jpg").write_bytes(b"\xff\xd8" + c.encode())
    d = ds.Caltech101Dataset(str(tmp_path / "cal"), shuffle=False)
    assert d.get_class_indexing() == {"ant": 0, "bee": 1} and [int(r["label"]) for r in _rows(d)] == [0, 1]
    coco = tmp_path / "coco"
    coco.mkdir()
    (coco / "a.jpg").write_bytes(b"img-a")
    ann = {"images": [{"id": 1, "file_name": "a.jpg"}, {"id": 2, "file_name": "b.jpg"}],
           "annotations": [{"image_id": 1, "bbox": [1, 2, 3, 4], "category_id": 5, "iscrowd": 0},
                           {"image_id": 1, "bbox": [5, 6, 7, 8], "category_id": 6, "iscrowd": 1}],
           "categories": [{"id": 5, "name": "cat"}, {"id": 6, "name": "dog"}]}
    (coco / "ann.json").write_text(json.dumps(ann))
    r = _rows(ds.CocoDataset(str(coco), str(coco / "ann.json"), task="Detection", extra_metadata=True))
    assert len(r) == 1 and r[0]["bbox"].tolist() == [[1, 2, 3, 4], [5, 6, 7, 8]] and r[0]["category_id"].tolist() == [[5], [6]]
    assert str(r[0]["_meta-filename"]) == "a.jpg"
    voc = tmp_path / "voc"
    for sub in ("ImageSets/Main", "Annotations", "JPEGImages"):
        (voc / sub).mkdir(parents=True)
    (voc / "ImageSets/Main/train.txt").write_text("0001\n")
    (voc / "JPEGImages/0001.jpg").write_bytes(b"jpg")
    (voc / "Annotations/0001.xml").write_text(
        "<annotation><object><name>car</name><difficult>1</difficult><truncated>0</truncated><bndbox><xmin>10</xmin>"
        "<ymin>20</ymin><xmax>50</xmax><ymax>80</ymax></bndbox></object></annotation>")
    v = ds.VOCDataset(str(voc), task="Detection", usage="train")
    r = _rows(v)
    assert v.get_class_indexing() == {"car": 0} and r[0]["bbox"].tolist() == [[10, 20, 40, 60]] and r[0]["difficult"].tolist() == [[1]]
    man = tmp_path / "m.manifest"
    (tmp_path / "x.jpg").write_bytes(b"x")
    man.write_text(json.dumps({"source": str(tmp_path / "x.jpg"), "usage": "TRAIN", "annotation": [{"name": "dog"}]}) + "\n"
                   + json.dumps({"source": str(tmp_path / "x.jpg"), "usage": "EVAL", "annotation": [{"name": "cat"}]}) + "\n")
    m = ds.ManifestDataset(str(man), usage="train")
    assert m.get_dataset_size() == 1 and m.get_class_indexing() == {"dog": 0}
    cel = tmp_path / "celeba"
    cel.mkdir()
    (cel / "list_attr_celeba.txt").write_text("2\n" + " ".join("a%d" % i for i in range(40)) + "\n"
                                              "1.jpg " + " ".join(["1", "-1"] * 20) + "\n2.jpg " + " ".join(["-1"] * 40) + "\n")
    (cel / "list_eval_partition.txt").write_text("1.jpg 0\n2.jpg 2\n")
    for n in ("1.jpg", "2.jpg"):
        (cel / n).write_bytes(b"j")
    r = _rows(ds.CelebADataset(str(cel), usage="train"))
    assert len(r) == 1 and r[0]["attr"].tolist() == [1, 0] * 20


def test_text_datasets(tmp_path):
    (tmp_path / "train.csv").write_text('"3","Title one","Body one"\n"1","T2","B2"\n')
    r = _rows(ds.AGNewsDataset(str(tmp_path), usage="train", shuffle=False))
    assert [str(x["index"]) for x in r] == ["3", "1"] and str(r[0]["title"]) == "Title one"
    for part in ("train", "test"):
        for sub in ("pos", "neg"):
            (tmp_path / "imdb" / part / sub).mkdir(parents=True)
            (tmp_path / "imdb" / part / sub / "0_1.txt").write_text("%s %s review" % (part, sub))
    r = _rows(ds.IMDBDataset(str(tmp_path / "imdb"), usage="train", shuffle=False))
    assert [(str(x["text"]), int(x["label"])) for x in r] == [("train pos review", 1), ("train neg review", 0)]
    (tmp_path / "train.txt").write_text("He PRP B-NP\nruns VBZ B-VP\n\nStop VB B-VP\n")
    r = _rows(ds.CoNLL2000Dataset(str(tmp_path), usage="train", shuffle=False))
    assert len(r) == 2 and r[0]["word"].tolist() == ["He", "runs"] and r[0]["chunk_tag"].tolist() == ["B-NP", "B-VP"]
    (tmp_path / "ptb.train.txt").write_text(" the cat \n\n sat \n")
    assert [str(x["text"]) for x in _rows(ds.PennTreebankDataset(str(tmp_path), usage="train", shuffle=False))] == [" the cat ", " sat "]
    (tmp_path / "train-v1.1.json").write_text(json.dumps({"data": [{"paragraphs": [{"context": "C", "qas": [
        {"question": "Q", "answers": [{"text": "A", "answer_start": 3}]}]}]}]}))
    r = _rows(ds.SQuADDataset(str(tmp_path), usage="train"))
    assert str(r[0]["context"]) == "C" and r[0]["text"].tolist() == ["A"] and r[0]["answer_start"].tolist() == [3]
    (tmp_path / "afqmc.json").write_text('{"sentence1": "a", "sentence2": "b", "label": "1"}\n')
    r = _rows(ds.CLUEDataset(str(tmp_path / "afqmc.json"), task="AFQMC", usage="train"))
    assert str(r[0]["label"]) == "1" and str(r[0]["sentence2"]) == "b"
    (tmp_path / "train.de").write_text("eins\nzwei\n")
    (tmp_path / "train.en").write_text("one\ntwo\n")
    r = _rows(ds.Multi30kDataset(str(tmp_path), usage="train", shuffle=False))
    assert [(str(x["text"]), str(x["translation"])) for x in r] == [("eins", "one"), ("zwei", "two")]
    (tmp_path / "train.tsv").write_text("sentence\tlabel\nfine film\t1\n")
    assert str(_rows(ds.SST2Dataset(str(tmp_path), usage="train"))[0]["sentence"]) == "fine film"


def test_audio_datasets(tmp_path):
    yes = tmp_path / "yesno"
    yes.mkdir()
    _wav(yes / "0_1_0_1_1_1_0_0.wav", np.linspace(-0.5, 0.5, 100))
    r = _rows(ds.YesNoDataset(str(yes)))
    assert r[0]["waveform"].shape == (1, 100) and int(r[0]["sample_rate"]) == 8000 and r[0]["labels"].tolist() == [0, 1, 0, 1, 1, 1, 0, 0]
    assert abs(float(r[0]["waveform"][0, -1]) - 0.5) < 1e-3
    sc = tmp_path / "sc"
    (sc / "yes").mkdir(parents=True)
    (sc / "no").mkdir()
    _wav(sc / "yes" / "abc_nohash_0.wav", np.zeros(10))
    _wav(sc / "no" / "abc_nohash_1.wav", np.zeros(10))
    (sc / "testing_list.txt").write_text("no/abc_nohash_1.wav\n")
    r = _rows(ds.SpeechCommandsDataset(str(sc), usage="test"))
    assert len(r) == 1 and str(r[0]["label"]) == "no" and int(r[0]["utterance_number"]) == 1
    assert ds.SpeechCommandsDataset(str(sc), usage="train").get_dataset_size() == 1
    lj = tmp_path / "lj"
    (lj / "wavs").mkdir(parents=True)
    _wav(lj / "wavs" / "LJ001-0001.wav", np.zeros(20))
    (lj / "metadata.csv").write_text("LJ001-0001|Dr. Smith|Doctor Smith\n")
    r = _rows(ds.LJSpeechDataset(str(lj)))
    assert str(r[0]["normalized_transcript"]) == "Doctor Smith" and r[0]["waveform"].shape == (1, 20)


def test_schema_tfrecord_padded_cache_and_tools(tmp_path):
    s = ds.Schema()
    s.add_column("image", "uint8", [2, 2])
    s.add_column("label", "int64")
    back = ds.Schema()
    back.from_json(json.loads(s.to_json()))
    assert [c["name"] for c in back.columns] == ["image", "label"] and back.columns[0]["shape"] == [2, 2]
    with pytest.raises(RuntimeError):
        back.parse_columns([{"name": "x"}])
    pad = ds.PaddedDataset([{"image": np.zeros(2, np.uint8), "label": np.int32(9)}] * 3)
    assert pad.get_dataset_size() == 3 and int(_rows(pad)[0]["label"]) == 9
    with pytest.raises(TypeError):
        ds.PaddedDataset([])

    def varint(n):
        out = bytearray()
        while True:
            b = n & 0x7F
            n >>= 7
            out.append(b | (0x80 if n else 0))
            if not n:
                return bytes(out)
    ld = lambda num, payload: varint(num << 3 | 2) + varint(len(payload)) + payload
    ex = ld(1, ld(1, ld(1, b"label") + ld(2, ld(3, ld(1, varint(7))))) + ld(1, ld(1, b"img") + ld(2, ld(1, ld(1, b"\x01\x02")))))
    with open(tmp_path / "d.tfrecord", "wb") as f:
        f.write(struct.pack("<Q", len(ex)) + b"\0" * 4 + ex + b"\0" * 4)
    r = _rows(ds.TFRecordDataset(str(tmp_path / "d.tfrecord"), columns_list=["label", "img"]))
    assert r[0]["label"].tolist() == [7] and r[0]["img"].tolist() == [1, 2]
    cache = ds.DatasetCache(session_id=1, size=1)
    cache.put(0, (np.zeros(600_000, np.uint8),))
    cache.put(1, (np.zeros(600_000, np.uint8),))
    assert cache.get(0) is None and cache.get(1) is not None and cache.get_stat()["num_rows"] == 1
    a = ds.NumpySlicesDataset({"x": np.arange(6)}, shuffle=False).batch(2)
    b = ds.NumpySlicesDataset({"x": np.arange(6)}, shuffle=False).batch(3)
    tree = ds.serialize(a, str(tmp_path / "p.json"))
    assert tree["op_type"] == "Batch" and tree["children"][0]["columns"] == ["x"]
    assert ds.deserialize(json_filepath=str(tmp_path / "p.json")) == tree
    assert ds.compare(a, a) and not ds.compare(a, b)
    ds.sync_wait_for_dataset(0, 1, 1)
    cb = ds.DSCallback(step_size=2)
    assert cb.step_size == 2
    with pytest.raises(ValueError):
        ds.DSCallback(0)
