"""Record files: a schema'd, indexed, optionally sharded and encrypted container of rows (MindRecord).

Files are written in, and read from, the reference's MindRecord layout (``mindrecord_format.py``: JSON header, raw
and blob pages, msgpack rows, SQLite index beside each shard), so datasets written by the reference open here.
With an encryption key or a hash mode set, the writer uses the private container described next instead (the
reference encrypts record files with a tool of its own, which is not reproduced); the reader takes both.

Layout of one shard ``<name>`` (``<name>0 .. <name>N-1`` with ``shard_num = N``): magic ``MSB200RECORD\\0``, u32 header
length, JSON header {schema, row offsets, row count, index fields, per-row index values, shard list}, then the rows;
each row is the concatenation of its fields, a field being u32 meta length + u64 payload length + JSON shape + payload
(raw bytes for ``bytes`` / ``string`` fields, C-order array data for numeric fields).  Random access by row through
the offset table; ``MindPage`` pages through the rows of one category of an indexed field.  With an encryption key
set (``set_enc_key``) the whole file body after the magic is one AES block of ``train.crypto``; ``set_hash_mode``
appends a digest of the plain body that the reader verifies.

Parity (API): python/mindspore/mindrecord/filewriter.py (FileWriter: open_for_append / add_schema / add_index /
write_raw_data / commit), filereader.py (FileReader: get_next / schema / len / close), mindpage.py (MindPage),
config.py (set_enc_key / set_enc_mode / set_dec_mode / set_hash_mode), tools/*.py (CsvToMR, MnistToMR, Cifar10ToMR,
Cifar100ToMR, ImageNetToMR, TFRecordToMR)."""
from __future__ import annotations

import gzip
import hashlib
import json
import os
import pickle
import struct

import numpy as np

SUCCESS, FAILED = 0, -1
_MAGIC = b"MSB200RECORD\0"
_MAGIC_ENC = b"MSB200RECENC\0"
_TYPES = {"int32": np.int32, "int64": np.int64, "float32": np.float32, "float64": np.float64, "uint8": np.uint8,
          "float16": np.float16, "bytes": None, "string": None}

_config = {"enc_key": None, "enc_mode": "AES-GCM", "dec_mode": None, "hash_mode": None}


def set_enc_key(enc_key):
    """Key (str or bytes of length 16 / 24 / 32, or None to switch encryption off) for files written and read from
    now on."""
    if enc_key is None:
        _config["enc_key"] = None
        return
    key = enc_key.encode() if isinstance(enc_key, str) else bytes(enc_key)
    if len(key) not in (16, 24, 32):
        raise ValueError("The length of enc_key must be 16, 24 or 32, but got %d" % len(key))
    _config["enc_key"] = key


def set_enc_mode(enc_mode="AES-GCM"):
    if callable(enc_mode):
        _config["enc_mode"] = enc_mode
        return
    if enc_mode not in ("AES-GCM", "AES-CBC"):
        raise ValueError("enc_mode must be 'AES-GCM', 'AES-CBC' or a callable, but got %r" % (enc_mode,))
    _config["enc_mode"] = enc_mode


def set_dec_mode(dec_mode="AES-GCM"):
    """None means: the same as the encryption mode."""
    if dec_mode is not None and not callable(dec_mode) and dec_mode not in ("AES-GCM", "AES-CBC"):
        raise ValueError("dec_mode must be 'AES-GCM', 'AES-CBC', a callable or None, but got %r" % (dec_mode,))
    _config["dec_mode"] = dec_mode


def set_hash_mode(hash_mode):
    """'sha256' / 'sha384' / 'sha512' / a callable(bytes) -> bytes / None."""
    if hash_mode is not None and not callable(hash_mode) and hash_mode not in ("sha256", "sha384", "sha512"):
        raise ValueError("hash_mode must be None, 'sha256', 'sha384', 'sha512' or a callable, but got %r"
                         % (hash_mode,))
    _config["hash_mode"] = hash_mode


def _digest(body):
    mode = _config["hash_mode"]
    if mode is None:
        return b""
    return bytes(mode(body)) if callable(mode) else hashlib.new(mode, body).digest()


def _seal(body):
    """magic + (encrypted) body + digest, as written to disk."""
    tail = _digest(body)
    body = body + struct.pack("<I", len(tail)) + tail
    key = _config["enc_key"]
    if key is None:
        return _MAGIC + body
    mode = _config["enc_mode"]
    if callable(mode):
        return _MAGIC_ENC + bytes(mode(body, key))
    from ..train import crypto
    return _MAGIC_ENC + crypto.encrypt(body, key, mode)


def _unseal(path):
    with open(path, "rb") as f:
        blob = f.read()
    if blob.startswith(_MAGIC_ENC):
        key = _config["enc_key"]
        if key is None:
            raise RuntimeError("%s is encrypted: call set_enc_key first" % path)
        mode = _config["dec_mode"] or _config["enc_mode"]
        if callable(mode):
            body = bytes(mode(blob[len(_MAGIC_ENC):], key))
        else:
            from ..train import crypto
            body = crypto.decrypt(blob[len(_MAGIC_ENC):], key, mode)
    elif blob.startswith(_MAGIC):
        body = blob[len(_MAGIC):]
    else:
        raise RuntimeError("%s is not a record file" % path)
    # trailer: u32 digest length + digest, found from the header's own length fields
    (hlen,) = struct.unpack("<I", body[:4])
    head = json.loads(body[4:4 + hlen])
    end = 4 + hlen + head["bytes"]
    (tlen,) = struct.unpack("<I", body[end:end + 4])
    tail = body[end + 4:end + 4 + tlen]
    plain = body[:end]
    if tlen and _config["hash_mode"] is not None and _digest(plain) != tail:
        raise RuntimeError("%s: integrity check failed (hash mismatch)" % path)
    return head, plain[4 + hlen:]


def _encode_row(schema, row):
    parts = []
    for name, spec in schema.items():
        if name not in row:
            raise ValueError("row lacks field %s" % name)
        v = row[name]
        if spec["type"] == "bytes":
            payload, meta = bytes(v), None
        elif spec["type"] == "string":
            payload, meta = str(v).encode(), None
        else:
            arr = np.ascontiguousarray(np.asarray(v, dtype=_TYPES[spec["type"]]))
            want = spec.get("shape")
            if want is not None and len(want) == arr.ndim and any(w not in (-1, s) for w, s in zip(want, arr.shape)):
                raise ValueError("field %s: shape %s does not match the schema's %s" % (name, list(arr.shape), want))
            payload, meta = arr.tobytes(), list(arr.shape)
        m = json.dumps(meta).encode()
        parts.append(struct.pack("<IQ", len(m), len(payload)) + m + payload)
    return b"".join(parts)


def _index_value(row, field):
    v = row[field]
    if isinstance(v, np.ndarray):
        v = v.reshape(-1)[0].item() if v.size else None
    elif isinstance(v, (np.integer, np.floating)):
        v = v.item()
    elif isinstance(v, (bytes, bytearray)):
        v = bytes(v).decode(errors="replace")
    return v


def _shard_names(file_name, shard_num):
    if shard_num == 1:
        return [file_name]
    width = len(str(shard_num - 1))
    return ["%s%0*d" % (file_name, width, i) for i in range(shard_num)]


class FileWriter:
    """Writes rows into ``shard_num`` files (rows go round-robin).  ``add_schema`` once, ``add_index`` optional,
    ``write_raw_data`` any number of times, ``commit`` to finish."""

    def __init__(self, file_name, shard_num=1, overwrite=False):
        if not isinstance(shard_num, int) or not 1 <= shard_num <= 1000:
            raise ValueError("shard_num must be an int in [1, 1000], but got %r" % (shard_num,))
        self.file_name, self.shard_num = file_name, shard_num
        self.files = _shard_names(file_name, shard_num)
        for f in self.files:
            if os.path.exists(f) and not overwrite:
                raise RuntimeError("%s already exists (pass overwrite=True)" % f)
        self.schema, self.desc, self.index_fields = None, None, []
        self.rows = [[] for _ in range(shard_num)]
        self.row_dicts = [[] for _ in range(shard_num)]
        self.index_values = [[] for _ in range(shard_num)]
        self._count = 0
        self._committed = False
        self._header_size, self._page_size = None, None

    def set_header_size(self, header_size):
        """Bytes reserved for the header (16 KB .. 128 MB; default 16 MB)."""
        if not isinstance(header_size, int) or not (1 << 14) <= header_size <= (1 << 27):
            raise ValueError("header_size must be an int in [16 KB, 128 MB], but got %r" % (header_size,))
        self._header_size = header_size
        return SUCCESS

    def set_page_size(self, page_size):
        """Bytes per page (32 KB .. 256 MB; default 32 MB): the largest row must fit one page."""
        if not isinstance(page_size, int) or not (1 << 15) <= page_size <= (1 << 28):
            raise ValueError("page_size must be an int in [32 KB, 256 MB], but got %r" % (page_size,))
        self._page_size = page_size
        return SUCCESS

    @classmethod
    def open_for_append(cls, file_name):
        """Re-opens a committed file (any shard of it) so that more rows can be added; ``commit`` rewrites it."""
        from . import mindrecord_format as F
        if F.looks_like_mindrecord(file_name):
            paths = F.shard_paths(file_name)
            first = F.ShardFile(paths[0])
            w = cls.__new__(cls)
            w.file_name, w.shard_num, w.files = file_name, len(paths), paths
            w.schema = first.schema
            w.desc = first.header["schema"][0].get("desc")
            w.index_fields = [f["index_field"] for f in first.header.get("index_fields", [])]
            w.rows, w.row_dicts, w.index_values, w._count, w._committed = [], [], [], 0, False
            w._header_size, w._page_size = first.header["header_size"], first.header["page_size"]
            for path in paths:
                sf = F.ShardFile(path)
                dicts = [sf.read(i) for i in range(len(sf))]
                w.row_dicts.append(dicts)
                w.rows.append([b""] * len(dicts))
                w.index_values.append([[_index_value(d, f) for f in w.index_fields] for d in dicts])
                w._count += len(dicts)
            return w
        head, _ = _unseal(file_name)
        shards = head.get("shards") or [os.path.basename(file_name)]
        folder = os.path.dirname(os.path.abspath(file_name))
        w = cls.__new__(cls)
        w.file_name, w.shard_num = file_name, len(shards)
        w.files = [os.path.join(folder, s) for s in shards]
        w.schema, w.desc, w.index_fields = head["schema"], head.get("desc"), head.get("index_fields", [])
        w.rows, w.row_dicts, w.index_values, w._count, w._committed = [], [], [], 0, False
        w._header_size, w._page_size = None, None
        for f in w.files:
            h, body = _unseal(f)
            offs = h["offsets"] + [len(body)]
            w.row_dicts.append(None)                      # rows of the private container stay encoded
            w.rows.append([bytes(body[offs[i]:offs[i + 1]]) for i in range(h["count"])])
            w.index_values.append(list(h.get("index_values", [])))
            w._count += h["count"]
        return w

    def init_append(self, file_name):
        """Turns this writer into one that appends to the committed dataset ``file_name`` (filewriter.py
        ``_init_append``'s public form)."""
        self.__dict__.update(type(self).open_for_append(file_name).__dict__)
        return SUCCESS

    def add_schema(self, content, desc=None):
        if not isinstance(content, dict) or not content:
            raise ValueError("schema must be a non-empty dict of field -> {'type': ..., 'shape': ...}")
        for name, spec in content.items():
            if spec.get("type") not in _TYPES:
                raise ValueError("field %s: unsupported type %r" % (name, spec.get("type")))
        self.schema, self.desc = content, desc
        return SUCCESS

    def add_index(self, index_fields):
        if self.schema is None:
            raise RuntimeError("add_schema must be called before add_index")
        for f in index_fields:
            if f not in self.schema:
                raise ValueError("index field %s is not in the schema" % f)
            if self.schema[f]["type"] == "bytes":
                raise ValueError("index field %s must be a numeric or string field, not bytes" % f)
        self.index_fields = list(index_fields)
        return SUCCESS

    def write_raw_data(self, raw_data, parallel_writer=False):
        if self.schema is None:
            raise RuntimeError("add_schema must be called before write_raw_data")
        if not isinstance(raw_data, (list, tuple)):
            raise TypeError("raw_data must be a list of dicts")
        for row in raw_data:
            shard = self._count % self.shard_num
            self.rows[shard].append(_encode_row(self.schema, row))
            if self.row_dicts[shard] is not None:
                self.row_dicts[shard].append(dict(row))
            self.index_values[shard].append([_index_value(row, f) for f in self.index_fields])
            self._count += 1
        return SUCCESS

    def _private_container(self):
        return _config["enc_key"] is not None or _config["hash_mode"] is not None or any(
            d is None for d in self.row_dicts)

    def commit(self):
        names = [os.path.basename(f) for f in self.files]
        if not self._private_container():
            from . import mindrecord_format as F
            F.write_dataset(self.files, self.schema, self.desc, self.index_fields, self.row_dicts,
                            self._header_size or F.DEFAULT_HEADER_SIZE, self._page_size or F.DEFAULT_PAGE_SIZE)
            self._committed = True
            return SUCCESS
        for path, rows, idx in zip(self.files, self.rows, self.index_values):
            offsets, pos = [], 0
            for r in rows:
                offsets.append(pos)
                pos += len(r)
            header = json.dumps({"schema": self.schema, "desc": self.desc, "offsets": offsets, "count": len(rows),
                                 "bytes": pos, "index_fields": self.index_fields, "index_values": idx,
                                 "shards": names}).encode()
            with open(path, "wb") as f:
                f.write(_seal(struct.pack("<I", len(header)) + header + b"".join(rows)))
        self._committed = True
        return SUCCESS

    def get_shard_files(self):
        return list(self.files)


class _Shard:
    def __init__(self, path):
        self.head, self.body = _unseal(path)
        self.offsets = self.head["offsets"]
        self.count = self.head["count"]


class _ReferenceShard:
    """A shard in the MindRecord layout, behind the interface the reader uses."""

    def __init__(self, path):
        from . import mindrecord_format as F
        self.file = F.ShardFile(path)
        self.count = len(self.file)
        index = [f["index_field"] for f in self.file.header.get("index_fields", [])]
        self.head = {"schema": self.file.schema, "index_fields": index,
                     "desc": self.file.header["schema"][0].get("desc")}


class FileReader:
    """Reads one or several record files.  Given one shard of a sharded file it opens all of them."""

    def __init__(self, file_name, num_consumer=4, columns=None, operator=None):
        from . import mindrecord_format as F
        paths = [file_name] if isinstance(file_name, str) else list(file_name)
        reference = F.looks_like_mindrecord(paths[0])
        if isinstance(file_name, str) and reference:
            paths = F.shard_paths(paths[0])                 # a list of files is taken as given
        elif isinstance(file_name, str):
            head, _ = _unseal(paths[0])
            shards = head.get("shards")
            if shards and len(shards) > 1:
                folder = os.path.dirname(os.path.abspath(paths[0]))
                paths = [os.path.join(folder, s) for s in shards]
        self.shards = [_ReferenceShard(p) if reference else _Shard(p) for p in paths]
        self._schema = self.shards[0].head["schema"]
        self.index_fields = self.shards[0].head.get("index_fields", [])
        self.count = sum(s.count for s in self.shards)
        self.columns = list(columns) if columns else list(self._schema)
        for c in self.columns:
            if c not in self._schema:
                raise ValueError("column %s is not in the schema %s" % (c, list(self._schema)))
        self._where = [(si, k) for si, s in enumerate(self.shards) for k in range(s.count)]

    def __len__(self):
        return self.count

    def len(self):
        return self.count

    def schema(self):
        return self._schema

    def read(self, i):
        si, k = self._where[i]
        sh = self.shards[si]
        if isinstance(sh, _ReferenceShard):
            return sh.file.read(k, self.columns)
        pos = sh.offsets[k]
        body, row = sh.body, {}
        for name, spec in self._schema.items():
            mlen, plen = struct.unpack_from("<IQ", body, pos)
            pos += 12
            meta = json.loads(body[pos:pos + mlen])
            pos += mlen
            payload = body[pos:pos + plen]
            pos += plen
            if name not in self.columns:
                continue
            if spec["type"] == "bytes":
                row[name] = np.frombuffer(payload, dtype=np.uint8)
            elif spec["type"] == "string":
                row[name] = np.array(bytes(payload).decode())
            else:
                row[name] = np.frombuffer(payload, dtype=_TYPES[spec["type"]]).reshape(meta)
        return row

    def index_value(self, i, field):
        si, k = self._where[i]
        if isinstance(self.shards[si], _ReferenceShard):
            return self.shards[si].file.index_values(k, [field])[0]
        return self.shards[si].head["index_values"][k][self.index_fields.index(field)]

    def get_next(self):
        for i in range(self.count):
            yield self.read(i)

    def show(self):
        for row in self.get_next():
            print(row)

    def close(self):
        self.shards = []


class MindPage:
    """Pages through the rows of one category (= one value of an indexed field)."""

    def __init__(self, file_name, num_consumer=4):
        self.reader = FileReader(file_name, num_consumer)
        self._field = self.reader.index_fields[0] if self.reader.index_fields else None

    @property
    def candidate_fields(self):
        return list(self.reader.index_fields)

    def get_category_fields(self):
        return self.candidate_fields

    @property
    def category_field(self):
        return self._field

    def set_category_field(self, category_field):
        if category_field not in self.reader.index_fields:
            raise ValueError("%s is not an indexed field (candidates: %s)" % (category_field, self.candidate_fields))
        self._field = category_field
        return True

    def _categories(self):
        if self._field is None:
            raise RuntimeError("the file has no index field; add_index when writing it")
        groups = {}
        for i in range(len(self.reader)):
            groups.setdefault(self.reader.index_value(i, self._field), []).append(i)
        return groups

    def read_category_info(self):
        """JSON string {"key": field, "categories": [{"id", "name", "count"}]}, categories in order of appearance."""
        groups = self._categories()
        return json.dumps({"key": self._field, "categories": [
            {"id": i, "name": str(name), "count": len(rows)} for i, (name, rows) in enumerate(groups.items())]})

    def _page(self, rows, page, num_row):
        if page < 0 or num_row <= 0:
            raise ValueError("page must be >= 0 and num_row > 0")
        return [self.reader.read(i) for i in rows[page * num_row:(page + 1) * num_row]]

    def read_at_page_by_id(self, category_id, page, num_row):
        groups = list(self._categories().values())
        if not 0 <= category_id < len(groups):
            raise IndexError("category id %d outside [0, %d)" % (category_id, len(groups)))
        return self._page(groups[category_id], page, num_row)

    def read_at_page_by_name(self, category_name, page, num_row):
        for name, rows in self._categories().items():
            if str(name) == str(category_name):
                return self._page(rows, page, num_row)
        raise KeyError("no category named %r in field %s" % (category_name, self._field))


# ---------------------------------------------------------------------------------------------------- converters
class _Converter:
    def __init__(self, destination, partition_number=1):
        self.destination, self.partition_number = destination, partition_number

    def _rows(self):
        raise NotImplementedError

    def _schema(self):
        raise NotImplementedError

    def _index(self):
        return []

    def run(self):
        w = FileWriter(self.destination, self.partition_number, overwrite=True)
        w.add_schema(self._schema(), type(self).__name__)
        if self._index():
            w.add_index(self._index())
        batch = []
        for row in self._rows():
            batch.append(row)
            if len(batch) >= 256:
                w.write_raw_data(batch)
                batch = []
        if batch:
            w.write_raw_data(batch)
        return w.commit()

    def transform(self):
        return self.run()


class CsvToMR(_Converter):
    """One row per CSV line; integer columns become int64, other numeric ones float64, the rest string."""

    def __init__(self, source, destination, columns_list=None, partition_number=1):
        super().__init__(destination, partition_number)
        import pandas as pd
        if not os.path.exists(source):
            raise IOError("Csv file %s does not exist" % source)
        self.df = pd.read_csv(source)
        if columns_list:
            missing = [c for c in columns_list if c not in self.df.columns]
            if missing:
                raise ValueError("columns %s are not in the csv file" % missing)
            self.df = self.df[list(columns_list)]

    def _kind(self, col):
        k = self.df[col].dtype.kind
        return "int64" if k in "iub" else "float64" if k == "f" else "string"

    def _schema(self):
        return {c: {"type": self._kind(c)} for c in self.df.columns}

    def _rows(self):
        kinds = {c: self._kind(c) for c in self.df.columns}
        for rec in self.df.to_dict("records"):
            yield {c: (str(v) if kinds[c] == "string" else v) for c, v in rec.items()}


def _read_idx(path):
    opener = gzip.open if path.endswith(".gz") else open
    with opener(path, "rb") as f:
        data = f.read()
    magic, = struct.unpack(">I", data[:4])
    ndim = magic & 0xFF
    dims = struct.unpack(">" + "I" * ndim, data[4:4 + 4 * ndim])
    return np.frombuffer(data, dtype=np.uint8, offset=4 + 4 * ndim).reshape(dims)


class MnistToMR(_Converter):
    """``source`` holds the four idx files (plain or .gz); writes ``<destination>_train.mindrecord`` and
    ``<destination>_test.mindrecord`` with fields label (int64) and data (bytes: the 28 x 28 image, raw)."""

    def __init__(self, source, destination, partition_number=1):
        super().__init__(destination, partition_number)
        self.source = source

    def _find(self, stem):
        for name in (stem, stem + ".gz"):
            p = os.path.join(self.source, name)
            if os.path.exists(p):
                return p
        raise IOError("%s not found in %s" % (stem, self.source))

    def run(self):
        for split, img, lab in (("train", "train-images-idx3-ubyte", "train-labels-idx1-ubyte"),
                                ("test", "t10k-images-idx3-ubyte", "t10k-labels-idx1-ubyte")):
            images, labels = _read_idx(self._find(img)), _read_idx(self._find(lab))
            w = FileWriter("%s_%s.mindrecord" % (self.destination, split), self.partition_number, overwrite=True)
            w.add_schema({"label": {"type": "int64"}, "data": {"type": "bytes"}}, "mnist_" + split)
            w.add_index(["label"])
            w.write_raw_data([{"label": int(l), "data": im.tobytes()} for im, l in zip(images, labels)])
            w.commit()
        return SUCCESS


class _CifarToMR(_Converter):
    train_files, test_files, label_keys = (), (), ()

    def __init__(self, source, destination):
        super().__init__(destination, 1)
        self.source = source

    def _load(self, names):
        rows = []
        for n in names:
            with open(os.path.join(self.source, n), "rb") as f:
                d = pickle.load(f, encoding="bytes")
            data = np.asarray(d[b"data"], dtype=np.uint8).reshape(-1, 3, 32, 32).transpose(0, 2, 3, 1)
            labels = [d[k] for k in self.label_keys]
            for i in range(data.shape[0]):
                row = {"id": len(rows), "data": np.ascontiguousarray(data[i]).tobytes()}
                for key, lab in zip(self.label_keys, labels):
                    row[key.decode().rstrip("s") if key != b"labels" else "label"] = int(lab[i])
                rows.append(row)
        return rows

    def run(self, fields=None):
        label_fields = [k.decode().rstrip("s") if k != b"labels" else "label" for k in self.label_keys]
        schema = {"id": {"type": "int64"}, "data": {"type": "bytes"}}
        schema.update({f: {"type": "int64"} for f in label_fields})
        for suffix, names in (("", self.train_files), ("_test", self.test_files)):
            w = FileWriter(self.destination + suffix, 1, overwrite=True)
            w.add_schema(schema, type(self).__name__)
            w.add_index(list(fields) if fields else ["id"] + label_fields)
            w.write_raw_data(self._load(names))
            w.commit()
        return SUCCESS

    def transform(self, fields=None):
        return self.run(fields)


class Cifar10ToMR(_CifarToMR):
    """``source``: the python-version folder (data_batch_1..5, test_batch)."""
    train_files = tuple("data_batch_%d" % i for i in range(1, 6))
    test_files = ("test_batch",)
    label_keys = (b"labels",)


class Cifar100ToMR(_CifarToMR):
    """``source``: the python-version folder (train, test); fields fine_label and coarse_label."""
    train_files = ("train",)
    test_files = ("test",)
    label_keys = (b"fine_labels", b"coarse_labels")


class ImageNetToMR(_Converter):
    """``map_file``: lines ``<folder name> <label id>``; ``image_dir``: one folder of image files per class.
    Fields: file_name (string), label (int64), image (bytes: the encoded file as found)."""

    def __init__(self, map_file, image_dir, destination, partition_number=1):
        super().__init__(destination, partition_number)
        self.map_file, self.image_dir = map_file, image_dir

    def _schema(self):
        return {"file_name": {"type": "string"}, "label": {"type": "int64"}, "image": {"type": "bytes"}}

    def _index(self):
        return ["label"]

    def _rows(self):
        with open(self.map_file) as f:
            pairs = [ln.split() for ln in f if ln.strip()]
        for folder, label in pairs:
            d = os.path.join(self.image_dir, folder)
            if not os.path.isdir(d):
                continue
            for name in sorted(os.listdir(d)):
                with open(os.path.join(d, name), "rb") as img:
                    yield {"file_name": name, "label": int(label), "image": img.read()}


class TFRecordToMR(_Converter):
    """TFRecord files of ``tf.train.Example`` records; ``feature_dict`` maps feature names to
    ``{"type": ..., "shape": ...}`` in this module's schema vocabulary.  The framing (u64 length, crc, payload, crc)
    and the Example / Feature messages are decoded here, so TensorFlow is not needed."""

    def __init__(self, source, destination, feature_dict, bytes_fields=None):
        super().__init__(destination, 1)
        self.source, self.features = source, dict(feature_dict)
        self.bytes_fields = list(bytes_fields or [])

    def _schema(self):
        return {k: ({"type": "bytes"} if k in self.bytes_fields else v) for k, v in self.features.items()}

    @staticmethod
    def _varint(buf, pos):
        shift = val = 0
        while True:
            b = buf[pos]
            pos += 1
            val |= (b & 0x7F) << shift
            if not b & 0x80:
                return val, pos
            shift += 7

    @classmethod
    def _fields(cls, buf):
        pos, out = 0, []
        while pos < len(buf):
            key, pos = cls._varint(buf, pos)
            num, wire = key >> 3, key & 7
            if wire == 0:
                v, pos = cls._varint(buf, pos)
            elif wire == 1:
                v, pos = buf[pos:pos + 8], pos + 8
            elif wire == 2:
                n, pos = cls._varint(buf, pos)
                v, pos = buf[pos:pos + n], pos + n
            elif wire == 5:
                v, pos = buf[pos:pos + 4], pos + 4
            else:
                raise ValueError("unsupported protobuf wire type %d" % wire)
            out.append((num, wire, v))
        return out

    @classmethod
    def _feature(cls, buf):
        for num, _, v in cls._fields(buf):
            if num == 1:                                          # BytesList
                return [bytes(x) for n, _, x in cls._fields(v) if n == 1]
            if num == 2:                                          # FloatList (packed or not)
                vals = []
                for n, wire, x in cls._fields(v):
                    if n == 1:
                        vals += list(np.frombuffer(bytes(x), dtype="<f4"))
                return vals
            if num == 3:                                          # Int64List
                vals = []
                for n, wire, x in cls._fields(v):
                    if n != 1:
                        continue
                    if wire == 0:
                        vals.append(x)
                    else:
                        p = 0
                        while p < len(x):
                            val, p = cls._varint(x, p)
                            vals.append(val)
                return [val - (1 << 64) if val >= 1 << 63 else val for val in vals]
        return []

    def _examples(self):
        with open(self.source, "rb") as f:
            data = f.read()
        pos = 0
        while pos + 12 <= len(data):
            (n,) = struct.unpack_from("<Q", data, pos)
            payload = data[pos + 12:pos + 12 + n]
            pos += 12 + n + 4
            feats = {}
            for num, _, features in self._fields(payload):        # Example.features
                if num != 1:
                    continue
                for fnum, _, entry in self._fields(features):     # map<string, Feature> entries
                    if fnum != 1:
                        continue
                    kv = {k: v for k, _, v in self._fields(entry)}
                    feats[bytes(kv[1]).decode()] = self._feature(kv.get(2, b""))
            yield feats

    def _rows(self):
        for ex in self._examples():
            row = {}
            for name, spec in self._schema().items():
                if name not in ex:
                    raise ValueError("feature %s is missing from a record" % name)
                v = ex[name]
                if spec["type"] == "bytes":
                    row[name] = v[0]
                elif spec["type"] == "string":
                    row[name] = v[0].decode() if isinstance(v[0], bytes) else str(v[0])
                else:
                    row[name] = np.asarray(v, dtype=_TYPES[spec["type"]])
            yield row


__all__ = ["FileWriter", "FileReader", "MindPage", "Cifar10ToMR", "Cifar100ToMR", "CsvToMR", "ImageNetToMR",
           "MnistToMR", "TFRecordToMR", "set_enc_key", "set_enc_mode", "set_dec_mode", "set_hash_mode", "SUCCESS",
           "FAILED"]


# ---------------------------------------------------------------------------------------------------- the shard layer
class ShardHeader:
    """What a writer needs to know before the first row: the schema (``add_schema`` / ``build_schema``) and the index
    fields.  Parity: mindrecord/shardheader.py."""

    def __init__(self):
        self.schema, self.desc, self.index_fields = None, None, []

    @staticmethod
    def build_schema(content, desc=None):
        desc = desc if desc else ""
        if not isinstance(content, dict) or not content:
            raise ValueError("The schema content must be a non-empty dict")
        return {"schema": dict(content), "desc": desc}

    def add_schema(self, schema):
        built = schema if "schema" in schema and isinstance(schema["schema"], dict) else self.build_schema(schema)
        self.schema, self.desc = built["schema"], built.get("desc", "")
        return 0                                          # the id of the (one) schema

    def add_index_fields(self, index_fields):
        self.index_fields = list(index_fields)
        return SUCCESS

    @property
    def blob_fields(self):
        return [k for k, v in (self.schema or {}).items() if v.get("type") == "bytes" or "shape" in v]


class ShardWriter:
    """The writer under ``FileWriter`` as its own object: ``open`` -> ``set_shard_header`` -> ``write_raw_data`` ->
    ``commit``.  Parity: mindrecord/shardwriter.py."""

    def __init__(self):
        self._writer, self._paths = None, None

    def open(self, paths, override=False):
        paths = [paths] if isinstance(paths, str) else list(paths)
        self._paths = paths
        base = paths[0][:-1] if len(paths) > 1 and paths[0].endswith("0") else paths[0]
        self._writer = FileWriter(base, len(paths), overwrite=override)
        return SUCCESS

    def open_for_append(self, path):
        self._writer = FileWriter.open_for_append(path)
        return SUCCESS

    def set_header_size(self, header_size):
        return self._writer.set_header_size(header_size)

    def set_page_size(self, page_size):
        return self._writer.set_page_size(page_size)

    def set_shard_header(self, shard_header):
        self._writer.add_schema(shard_header.schema, shard_header.desc)
        if shard_header.index_fields:
            self._writer.add_index(shard_header.index_fields)
        return SUCCESS

    def write_raw_data(self, data, validate=True, parallel_writer=False):
        return self._writer.write_raw_data(data, parallel_writer)

    def commit(self):
        return self._writer.commit()

    def get_shard_files(self):
        return self._writer.get_shard_files()


class ShardReader:
    """Sequential reader of a dataset's rows: ``open`` -> ``launch`` -> ``get_next`` ... -> ``close``.
    Parity: mindrecord/shardreader.py."""

    def __init__(self):
        self._reader, self._it = None, None

    def open(self, file_name, num_consumer=4, columns=None, operator=None):
        self._reader = FileReader(file_name, num_consumer, columns, operator)
        return SUCCESS

    def launch(self):
        self._it = self._reader.get_next()
        return SUCCESS

    def get_next(self):
        if self._it is None:
            self.launch()
        return next(self._it, None)

    def get_blob_fields(self):
        return [k for k, v in self._reader.schema().items() if v.get("type") == "bytes" or "shape" in v]

    def get_header(self):
        head = ShardHeader()
        head.add_schema({"schema": self._reader.schema(), "desc": ""})
        head.add_index_fields(self._reader.index_fields)
        return head

    def len(self):
        return len(self._reader)

    def close(self):
        if self._reader is not None:
            self._reader.close()


class ShardIndexGenerator:
    """Rebuilds the ``.db`` index of one data file from its pages.  Parity: mindrecord/shardindexgenerator.py."""

    def __init__(self, path, append=False):
        self.path, self.append = path, append
        self._built = None

    def build(self):
        from . import mindrecord_format as F
        if not F.looks_like_mindrecord(self.path):
            raise RuntimeError("%s is not a MindRecord data file" % self.path)
        self._built = True
        return SUCCESS

    def write_to_db(self):
        from . import mindrecord_format as F
        if self._built is None:
            self.build()
        F.rebuild_index(self.path)
        return SUCCESS


class ShardSegment(MindPage):
    """The page reader under ``MindPage`` with the lower-level names (``open`` / ``close``).
    Parity: mindrecord/shardsegment.py."""

    def __init__(self):                                    # noqa: super().__init__ runs in `open`
        self._opened = False

    def open(self, file_name, num_consumer=4):
        MindPage.__init__(self, file_name, num_consumer)
        self._opened = True
        return SUCCESS

    def close(self):
        self._opened = False


class Cifar10:
    """The python-pickle CIFAR-10 folder as arrays: ``load_data()`` fills ``Train`` and ``Test`` (``.images`` NHWC
    uint8, ``.labels``; one-hot rows when ``one_hot``).  Parity: mindrecord/tools/cifar10.py."""
    converter = Cifar10ToMR
    num_classes = 10

    class _Split:
        def __init__(self, images, labels):
            self.images, self.labels = images, labels

    def __init__(self, path, one_hot=True):
        self.path, self.one_hot = path, one_hot
        self.Train = self.Test = None

    def _split(self, names):
        rows = self.converter(self.path, os.path.join(self.path, "unused"))._load(names)
        images = np.stack([np.frombuffer(r["data"], np.uint8).reshape(32, 32, 3) for r in rows])
        key = "label" if "label" in rows[0] else "fine_label"
        labels = np.array([r[key] for r in rows], np.int64)
        if self.one_hot:
            labels = np.eye(self.num_classes, dtype=np.float32)[labels]
        return self._Split(images, labels)

    def load_data(self):
        self.Train = self._split(self.converter.train_files)
        self.Test = self._split(self.converter.test_files)


class Cifar100(Cifar10):
    """CIFAR-100 (fine labels).  Parity: mindrecord/tools/cifar100.py."""
    converter = Cifar100ToMR
    num_classes = 100


__all__ += ["ShardHeader", "ShardWriter", "ShardReader", "ShardIndexGenerator", "ShardSegment", "Cifar10", "Cifar100"]
