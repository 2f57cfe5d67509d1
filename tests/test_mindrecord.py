"""Record files: shards, append, index + MindPage, encryption and integrity settings, and the converters
(CSV, MNIST idx, CIFAR pickles, ImageNet folders, TFRecord)."""
import gzip
import json
import os
import pickle
import struct

import numpy as np
import pytest

from mindspore_b200 import mindrecord as MR
from mindspore_b200.dataset import MindDataset


def _rows(n, start=0):
    return [{"id": start + i, "label": (start + i) % 3, "name": "row%d" % (start + i),
             "vec": np.arange(4, dtype=np.float32) + start + i, "blob": bytes([i % 256] * (i % 5 + 1))}
            for i in range(n)]


SCHEMA = {"id": {"type": "int64"}, "label": {"type": "int32"}, "name": {"type": "string"},
          "vec": {"type": "float32", "shape": [4]}, "blob": {"type": "bytes"}}


def test_sharded_write_read_append_and_dataset(tmp_path):
    path = str(tmp_path / "data.mr")
    w = MR.FileWriter(path, shard_num=3)
    assert w.add_schema(SCHEMA, "demo") == MR.SUCCESS
    w.add_index(["label", "name"])
    w.write_raw_data(_rows(10))
    assert w.commit() == MR.SUCCESS
    assert sorted(os.listdir(tmp_path)) == ["data.mr0", "data.mr0.db", "data.mr1", "data.mr1.db", "data.mr2",
                                            "data.mr2.db"]
    r = MR.FileReader(path + "1")                       # any shard opens them all
    assert len(r) == 10 and r.schema() == SCHEMA
    ids = sorted(int(row["id"]) for row in r.get_next())
    assert ids == list(range(10))
    row = next(x for x in r.get_next() if int(x["id"]) == 7)
    assert str(row["name"]) == "row7" and row["vec"].tolist() == [7, 8, 9, 10] and bytes(row["blob"]) == bytes([7] * 3)
    r.close()
    with pytest.raises(RuntimeError):
        MR.FileWriter(path, shard_num=3)                # exists
    with pytest.raises(ValueError):
        w2 = MR.FileWriter(str(tmp_path / "bad.mr"))
        w2.add_schema({"vec": {"type": "float32", "shape": [4]}})
        w2.write_raw_data([{"vec": np.zeros(5, np.float32)}])
    a = MR.FileWriter.open_for_append(path + "0")
    a.write_raw_data(_rows(5, start=10))
    a.commit()
    assert len(MR.FileReader(path + "0")) == 15
    ds = MindDataset(path + "0", columns_list=["id", "vec"], shuffle=False)
    got = sorted(int(r[0]) for r in ds.create_tuple_iterator(output_numpy=True))
    assert got == list(range(15))
    cols = MR.FileReader(path + "0", columns=["name"])
    assert list(next(cols.get_next())) == ["name"]
    with pytest.raises(ValueError):
        MR.FileReader(path + "0", columns=["nope"])


def test_mindpage_categories(tmp_path):
    path = str(tmp_path / "page.mr")
    w = MR.FileWriter(path)
    w.add_schema(SCHEMA)
    w.add_index(["label", "name"])
    w.write_raw_data(_rows(11))
    w.commit()
    page = MR.MindPage(path)
    assert page.candidate_fields == ["label", "name"] and page.category_field == "label"
    info = json.loads(page.read_category_info())
    assert info["key"] == "label"
    assert [(c["name"], c["count"]) for c in info["categories"]] == [("0", 4), ("1", 4), ("2", 3)]
    rows = page.read_at_page_by_id(1, 1, 3)             # second page of three rows of label 1: ids 10 only
    assert [int(r["id"]) for r in rows] == [10]
    rows = page.read_at_page_by_name("2", 0, 2)
    assert [int(r["id"]) for r in rows] == [2, 5]
    page.set_category_field("name")
    assert len(json.loads(page.read_category_info())["categories"]) == 11
    with pytest.raises(ValueError):
        page.set_category_field("vec")
    with pytest.raises(IndexError):
        page.read_at_page_by_id(99, 0, 1)


def test_encryption_and_hash_settings(tmp_path):
    path = str(tmp_path / "enc.mr")
    try:
        MR.set_enc_key("0123456789abcdef")
        MR.set_enc_mode("AES-CBC")
        MR.set_hash_mode("sha256")
        w = MR.FileWriter(path)
        w.add_schema(SCHEMA)
        w.write_raw_data(_rows(4))
        w.commit()
        raw = open(path, "rb").read()
        assert b"row1" not in raw and raw.startswith(b"MSB200RECENC")
        assert [int(r["id"]) for r in MR.FileReader(path).get_next()] == [0, 1, 2, 3]
        MR.set_enc_key(None)
        with pytest.raises(RuntimeError, match="encrypted"):
            MR.FileReader(path)
        MR.set_enc_key("fedcba9876543210")
        with pytest.raises(Exception):
            MR.FileReader(path)
        with pytest.raises(ValueError):
            MR.set_enc_key("short")
        with pytest.raises(ValueError):
            MR.set_hash_mode("md5")
        # plain file with a digest: a flipped payload byte is noticed
        MR.set_enc_key(None)
        p2 = str(tmp_path / "hash.mr")
        w = MR.FileWriter(p2)
        w.add_schema(SCHEMA)
        w.write_raw_data(_rows(4))
        w.commit()
        blob = bytearray(open(p2, "rb").read())
        blob[blob.index(b"row2") + 3] ^= 1
        open(p2, "wb").write(bytes(blob))
        with pytest.raises(RuntimeError, match="integrity"):
            MR.FileReader(p2)
    finally:
        MR.set_enc_key(None)
        MR.set_enc_mode("AES-GCM")
        MR.set_dec_mode(None)
        MR.set_hash_mode(None)


def test_csv_mnist_cifar_imagenet_converters(tmp_path):
    csv = tmp_path / "t.csv"
    csv.write_text("a,b,c\n1,0.5,x\n2,1.5,y\n3,2.5,z\n")
    MR.CsvToMR(str(csv), str(tmp_path / "csv.mr"), columns_list=["a", "c"]).transform()
    rows = list(MR.FileReader(str(tmp_path / "csv.mr")).get_next())
    assert [int(r["a"]) for r in rows] == [1, 2, 3] and [str(r["c"]) for r in rows] == ["x", "y", "z"]
    with pytest.raises(ValueError):
        MR.CsvToMR(str(csv), str(tmp_path / "csv2.mr"), columns_list=["nope"])

    mn = tmp_path / "mnist"
    mn.mkdir()
    rng = np.random.default_rng(0)
    for stem, n in (("train", 6), ("t10k", 3)):
        imgs = rng.integers(0, 255, (n, 28, 28), dtype=np.uint8)
        labs = np.arange(n, dtype=np.uint8)
        with gzip.open(mn / ("%s-images-idx3-ubyte.gz" % stem), "wb") as f:
            f.write(struct.pack(">IIII", 0x803, n, 28, 28) + imgs.tobytes())
        with open(mn / ("%s-labels-idx1-ubyte" % stem), "wb") as f:
            f.write(struct.pack(">II", 0x801, n) + labs.tobytes())
        if stem == "train":
            first = imgs[0].copy()
    MR.MnistToMR(str(mn), str(tmp_path / "mnist")).transform()
    tr = list(MR.FileReader(str(tmp_path / "mnist_train.mindrecord")).get_next())
    assert len(tr) == 6 and len(MR.FileReader(str(tmp_path / "mnist_test.mindrecord"))) == 3
    assert int(tr[0]["label"]) == 0 and np.array_equal(tr[0]["data"].reshape(28, 28), first)

    cf = tmp_path / "cifar"
    cf.mkdir()
    for name in ["data_batch_%d" % i for i in range(1, 6)] + ["test_batch"]:
        with open(cf / name, "wb") as f:
            pickle.dump({b"data": rng.integers(0, 255, (2, 3072), dtype=np.uint8), b"labels": [1, 7]}, f)
    MR.Cifar10ToMR(str(cf), str(tmp_path / "c10.mr")).transform()
    assert len(MR.FileReader(str(tmp_path / "c10.mr"))) == 10 and len(MR.FileReader(str(tmp_path / "c10.mr_test"))) == 2
    r0 = MR.FileReader(str(tmp_path / "c10.mr")).read(1)
    assert int(r0["label"]) == 7 and r0["data"].size == 3072
    c100 = tmp_path / "cifar100"
    c100.mkdir()
    for name in ("train", "test"):
        with open(c100 / name, "wb") as f:
            pickle.dump({b"data": rng.integers(0, 255, (3, 3072), dtype=np.uint8), b"fine_labels": [5, 6, 7],
                         b"coarse_labels": [0, 1, 2]}, f)
    MR.Cifar100ToMR(str(c100), str(tmp_path / "c100.mr")).transform()
    r = MR.FileReader(str(tmp_path / "c100.mr")).read(2)
    assert int(r["fine_label"]) == 7 and int(r["coarse_label"]) == 2

    img = tmp_path / "imgs"
    for cls in ("n01", "n02"):
        (img / cls).mkdir(parents=True)
        for k in range(2):
            (img / cls / ("%d.JPEG" % k)).write_bytes(b"\xff\xd8" + cls.encode() + bytes([k]))
    (tmp_path / "map.txt").write_text("n01 0\nn02 1\n")
    MR.ImageNetToMR(str(tmp_path / "map.txt"), str(img), str(tmp_path / "inet.mr"), partition_number=2).transform()
    rd = MR.FileReader(str(tmp_path / "inet.mr0"))
    assert len(rd) == 4 and sorted(int(x["label"]) for x in rd.get_next()) == [0, 0, 1, 1]


def _varint(n):
    out = bytearray()
    while True:
        b = n & 0x7F
        n >>= 7
        out.append(b | (0x80 if n else 0))
        if not n:
            return bytes(out)


def _ld(num, payload):
    return _varint(num << 3 | 2) + _varint(len(payload)) + payload


def test_tfrecord_converter_decodes_examples_without_tensorflow(tmp_path):
    def example(label, vec, name):
        feats = b""
        f_int = _ld(3, _ld(1, _varint(label)))                               # Int64List packed
        f_flt = _ld(2, _ld(1, np.asarray(vec, "<f4").tobytes()))             # FloatList packed
        f_byt = _ld(1, _ld(1, name))                                          # BytesList
        for key, f in (("label", f_int), ("vec", f_flt), ("name", f_byt)):
            feats += _ld(1, _ld(1, key.encode()) + _ld(2, f))
        return _ld(1, feats)
    path = tmp_path / "t.tfrecord"
    with open(path, "wb") as f:
        for i in range(3):
            ex = example(i + 5, [i, i + 0.5], b"n%d" % i)
            f.write(struct.pack("<Q", len(ex)) + b"\0\0\0\0" + ex + b"\0\0\0\0")
    MR.TFRecordToMR(str(path), str(tmp_path / "tf.mr"),
                    {"label": {"type": "int64"}, "vec": {"type": "float32", "shape": [2]}, "name": {"type": "string"}},
                    ).transform()
    rows = list(MR.FileReader(str(tmp_path / "tf.mr")).get_next())
    assert [int(np.asarray(r["label"]).reshape(-1)[0]) for r in rows] == [5, 6, 7]
    assert rows[2]["vec"].tolist() == [2.0, 2.5] and str(rows[1]["name"]) == "n1"


# Shard 0 of a four-shard dataset as the reference's writer produced it (format version 2.0, header 16 KB, pages of
# 32 KB; zlib + base64): four rows with an int32 label and four blob fields.
_REFERENCE_SHARD = (
    "eNrt0kGL00AUwPGue1n07M3DMue4NE2pS/HSxcuCIIgguCxhkpluA2lakqxaS2n2W/gFvPvdBK910kyapvYkqJf/79CZefPmzeu0"
    "16edraWYaKl06mfRFy2G7sC77DsiSpT+7I8jHatMDG+W+wExFLEMdCwckYUTPZV+ZGLd1a0j5vJOb9N1ovx09mm706/iVZad28vc"
    "waUN5Iu5CYir12+u/FejdyOxF69PlgXv0tn93ARsV9XGbDzOdG57yCYyVfWRLJdpvuuku3LarXX3WnNbrQ367cbejt7/zb5uW5d7"
    "vRflw1Svuy0YxLOg+TmETFO58KVpppoFu1m4mylhiiqdhab7JJ77tlpTdrkrY6amu/J73jx3zSn7naMk93pi1Vyyl+c6B5mDfpMZ"
    "lpl2K1jkOmu21H6R3vEi1b+rKWH7WDWvKJVKdZbp6jHC+Hqqgoup+Y+mOpylqls+wm9R92i0dzTqiSO/WB5leRSaO5P7OHbER51m"
    "0SwxDfYuumLVAQAAAAAAAAAAAAAAAAAAAAAAAAAAAIA/8+yktXxZfpShjbE2Y2HGwozrMlBvFtXmxgQ7xfacjWx9rYvVpTdWnVDY"
    "dWHX6zrh8GDRPrixiZ1i128roxzLhTleZXx/+uSD5/04uP4siefnSubSrs9/2oQHOz6u++KNeCPe6J++EQAAAAAAAAAAAAAAAAAA"
    "AAAAAAAAAAAAAAAAAAAAAAAAAAAAAAAAAAAAAAAAAPA/ndnx4VssAx0frk8O1o8O1qe/AHIt4Xw=")


def test_a_file_written_by_the_reference_reads_back(tmp_path):
    import base64
    import zlib

    from mindspore_b200.dataset import mindrecord_format as F
    path = tmp_path / "aclImdb.mindrecord0"
    path.write_bytes(zlib.decompress(base64.b64decode(_REFERENCE_SHARD)))
    assert F.looks_like_mindrecord(str(path))
    assert [os.path.basename(p) for p in F.shard_paths(str(path))] == ["aclImdb.mindrecord%d" % k for k in range(4)]
    reader = MR.FileReader([str(path)])                       # this shard alone
    assert len(reader) == 4 and reader.index_fields == ["label"]
    assert reader.schema()["array_b"] == {"shape": [1, -1], "type": "int64"}
    rows = list(reader.get_next())
    assert [int(r["label"]) for r in rows] == [0, 1, 2, 3]
    r = rows[1]
    assert r["array_a"].dtype == np.int32 and r["array_a"][:6].tolist() == [0, 1, -1, 127, -128, 128]
    assert r["array_b"].shape == (1, 19) and r["array_d"].tolist() == [[-10, -127], [10, 127]]
    assert bytes(r["array_c"]) == b"nlp data"


def test_written_files_follow_the_reference_layout(tmp_path):
    import json
    import sqlite3
    import struct

    import msgpack

    from mindspore_b200.dataset import mindrecord_format as F
    path = str(tmp_path / "lay.mindrecord")
    w = MR.FileWriter(path)
    w.set_header_size(1 << 14)
    w.set_page_size(1 << 15)
    w.add_schema({"label": {"type": "int32"}, "ids": {"type": "int64", "shape": [-1]}, "img": {"type": "bytes"}}, "lay")
    w.add_index(["label"])
    w.write_raw_data([{"label": i, "ids": np.array([i, 300 * i, -70000 * i]), "img": bytes([i]) * 5} for i in range(3)])
    w.commit()
    data = open(path, "rb").read()
    (n,) = struct.unpack("<Q", data[:8])
    head = json.loads(data[8:8 + n])
    assert head["header_size"] == 1 << 14 and head["page_size"] == 1 << 15 and head["version"] == "3.0"
    assert head["schema"][0]["blob_fields"] == ["ids", "img"] and head["shard_addresses"] == ["lay.mindrecord"]
    kinds = [p["page_type"] for p in head["page"]]
    assert kinds == ["BLOB_DATA", "RAW_DATA"]
    raw_at = (1 << 14) + (1 << 15)                             # page 1
    (m,) = struct.unpack("<Q", data[raw_at:raw_at + 8])
    assert msgpack.unpackb(data[raw_at + 8:raw_at + 8 + m]) == {"label": 0}
    blob_at = 1 << 14                                          # page 0: u64 length, then per field u64 BE length + bytes
    (b,) = struct.unpack("<Q", data[blob_at:blob_at + 8])
    (ids_len,) = struct.unpack(">Q", data[blob_at + 8:blob_at + 16])
    ids = data[blob_at + 16:blob_at + 16 + ids_len]
    assert struct.unpack(">I", ids[:4])[0] == 3 and F.uncompress_ints(ids, np.int64).tolist() == [0, 0, 0]
    assert len(data) == raw_at + head["page"][1]["page_size"]  # the file ends with the last page's data
    con = sqlite3.connect(path + ".db")
    rows = list(con.execute("SELECT ROW_ID, PAGE_ID_RAW, PAGE_OFFSET_RAW, PAGE_ID_BLOB, label_0 FROM INDEXES"))
    assert rows[0] == (0, 1, 0, 0, 0) and [r[4] for r in rows] == [0, 1, 2]
    assert list(con.execute("SELECT NAME FROM SHARD_NAME")) == [("lay.mindrecord",)]
    back = list(MR.FileReader(path).get_next())
    assert back[2]["ids"].tolist() == [2, 600, -140000] and bytes(back[2]["img"]) == b"\x02" * 5
    a = np.array([0, -1, 127, -128, 128, -32768, 32768, 2 ** 31 - 1, -2 ** 31, 2 ** 31, -2 ** 62], np.int64)
    assert (F.uncompress_ints(F.compress_ints(a), np.int64) == a).all()
    assert len(F.compress_ints(np.zeros(8, np.int64))) == 4 + 2 + 8
    with pytest.raises(ValueError):
        w2 = MR.FileWriter(str(tmp_path / "big.mindrecord"))
        w2.set_page_size(1 << 15)
        w2.add_schema({"img": {"type": "bytes"}})
        w2.write_raw_data([{"img": b"x" * (1 << 16)}])
        w2.commit()
