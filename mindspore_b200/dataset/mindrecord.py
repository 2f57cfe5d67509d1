"""Record files: a schema'd, indexed container of rows (the role of MindRecord).

Layout of ``<name>``: magic ``MSB200RECORD\\0``, u32 header length, JSON header {schema, row offsets, row count},
then the rows; each row is the concatenation of its fields, a field being u64 byte length + payload (raw bytes for
``bytes`` / ``string`` fields, C-order array data for numeric fields whose shape is stored in the row's own small
JSON prefix when it is not fixed by the schema).  Random access by row through the offset table.
Parity (API): python/mindspore/mindrecord/filewriter.py (FileWriter.add_schema / write_raw_data / commit),
filereader.py (FileReader.get_next / close)."""
from __future__ import annotations

import json
import os
import struct

import numpy as np

_MAGIC = b"MSB200RECORD\0"
_TYPES = {"int32": np.int32, "int64": np.int64, "float32": np.float32, "float64": np.float64, "uint8": np.uint8,
          "float16": np.float16, "bytes": None, "string": None}


class FileWriter:
    def __init__(self, file_name, shard_num=1, overwrite=False):
        if shard_num != 1:
            raise ValueError("this writer produces one file per FileWriter (shard_num=1)")
        if os.path.exists(file_name) and not overwrite:
            raise RuntimeError("%s already exists (pass overwrite=True)" % file_name)
        self.file_name, self.schema, self.rows = file_name, None, []

    def add_schema(self, content, desc=None):
        for name, spec in content.items():
            if spec.get("type") not in _TYPES:
                raise ValueError("field %s: unsupported type %r" % (name, spec.get("type")))
        self.schema = content
        return 0

    def add_index(self, fields):
        return 0

    def write_raw_data(self, raw_data, parallel_writer=False):
        if self.schema is None:
            raise RuntimeError("add_schema must be called before write_raw_data")
        for row in raw_data:
            parts = []
            for name, spec in self.schema.items():
                if name not in row:
                    raise ValueError("row lacks field %s" % name)
                v = row[name]
                if spec["type"] == "bytes":
                    payload, meta = bytes(v), None
                elif spec["type"] == "string":
                    payload, meta = str(v).encode(), None
                else:
                    arr = np.ascontiguousarray(np.asarray(v, dtype=_TYPES[spec["type"]]))
                    payload, meta = arr.tobytes(), list(arr.shape)
                m = json.dumps(meta).encode()
                parts.append(struct.pack("<IQ", len(m), len(payload)) + m + payload)
            self.rows.append(b"".join(parts))
        return 0

    def commit(self):
        offsets, pos = [], 0
        for r in self.rows:
            offsets.append(pos)
            pos += len(r)
        header = json.dumps({"schema": self.schema, "offsets": offsets, "count": len(self.rows)}).encode()
        with open(self.file_name, "wb") as f:
            f.write(_MAGIC + struct.pack("<I", len(header)) + header)
            for r in self.rows:
                f.write(r)
        return 0


class FileReader:
    def __init__(self, file_name, num_consumer=4, columns=None, operator=None):
        self.f = open(file_name, "rb")
        if self.f.read(len(_MAGIC)) != _MAGIC:
            raise RuntimeError("%s is not a record file" % file_name)
        (hlen,) = struct.unpack("<I", self.f.read(4))
        head = json.loads(self.f.read(hlen))
        self.schema, self.offsets, self.count = head["schema"], head["offsets"], head["count"]
        self.base = len(_MAGIC) + 4 + hlen
        self.columns = list(columns) if columns else list(self.schema)

    def __len__(self):
        return self.count

    def read(self, i):
        self.f.seek(self.base + self.offsets[i])
        row = {}
        for name, spec in self.schema.items():
            mlen, plen = struct.unpack("<IQ", self.f.read(12))
            meta = json.loads(self.f.read(mlen))
            payload = self.f.read(plen)
            if spec["type"] == "bytes":
                v = np.frombuffer(payload, dtype=np.uint8)
            elif spec["type"] == "string":
                v = np.array(payload.decode())
            else:
                v = np.frombuffer(payload, dtype=_TYPES[spec["type"]]).reshape(meta)
            if name in self.columns:
                row[name] = v
        return row

    def get_next(self):
        for i in range(self.count):
            yield self.read(i)

    def close(self):
        self.f.close()
