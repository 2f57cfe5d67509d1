"""The MindRecord on-disk format: reading files the reference wrote, and writing files in the same layout.

One shard ``<name>`` (``<name>0 .. <name>N-1`` for N shards) plus its index database ``<name>.db``:

    u64 LE  length of the JSON header, the header, zero padding up to ``header_size``
    page 0, page 1, ...   each ``page_size`` bytes, page k at ``header_size + k * page_size``

The header lists the schema (``schema`` with per-field type / shape, ``blob_fields`` = the bytes and array fields),
the index fields, the shard file names and the page table.  A BLOB_DATA page holds, row after row, ``u64 LE length``
+ the row's blob: the single blob field's bytes, or for several blob fields ``u64 BE length + bytes`` per field in
``blob_fields`` order (arrays as raw little-endian values).  A RAW_DATA page holds ``u64 LE length`` + the msgpack
encoding of the row's remaining (scalar / string) fields.  Rows appear in the same order in both page kinds; each
blob page is one row group.  From format version 3.0 on, int32 / int64 arrays inside the blob are compressed: u32 BE
element count, a bitmap of two bits per element (0..3 = 1, 2, 4, 8 bytes; four elements per byte, first element in
the high bits), then each value little-endian at its minimal signed width.

The SQLite database has a table ``INDEXES`` with, per row, its raw / blob page ids and byte ranges, its row group and
the values of the index fields (columns ``<field>_<schema id>``), and a table ``SHARD_NAME``.

Parity: ccsrc/minddata/mindrecord/io/shard_writer.cc (page layout, FlushRawChunk / FlushBlobChunk, header),
meta/shard_header.cc (SerializeHeader), meta/shard_column.cc (CompressInt / UncompressInt),
io/shard_index_generator.cc (INDEXES), python/mindspore/mindrecord/shardwriter.py (_merge_blob)."""
from __future__ import annotations

import json
import os
import sqlite3
import struct

import numpy as np

VERSION = "3.0"
DEFAULT_HEADER_SIZE = 1 << 24
DEFAULT_PAGE_SIZE = 1 << 25
_NP = {"int32": np.int32, "int64": np.int64, "float32": np.float32, "float64": np.float64, "uint8": np.uint8,
       "float16": np.float16}


class MindRecordFormatError(RuntimeError):
    pass


def looks_like_mindrecord(path):
    try:
        with open(path, "rb") as f:
            head = f.read(24)
    except OSError:
        return False
    return len(head) >= 9 and head[8:9] == b"{" and 0 < struct.unpack("<Q", head[:8])[0] < (1 << 30)


def read_header(path):
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        raw = f.read(n)
    try:
        return json.loads(raw)
    except ValueError as e:
        raise MindRecordFormatError("%s: the header is not valid JSON (%s)" % (path, e)) from e


# ---------------------------------------------------------------------------------------------------- integers
def compress_ints(arr):
    """int32 / int64 array -> count, width bitmap, minimal-width little-endian values."""
    vals = np.asarray(arr).reshape(-1).astype(np.int64)
    n = len(vals)
    kinds = np.where((vals >= -128) & (vals <= 127), 0, np.where((vals >= -32768) & (vals <= 32767), 1, np.where(
        (vals >= -(1 << 31)) & (vals <= (1 << 31) - 1), 2, 3))).astype(np.uint8)
    bitmap = bytearray((n + 3) // 4)
    body = bytearray()
    for i, (v, k) in enumerate(zip(vals.tolist(), kinds.tolist())):
        bitmap[i // 4] |= k << (2 * (3 - i % 4))
        body += int(v).to_bytes(1 << k, "little", signed=True)
    return struct.pack(">I", n) + bytes(bitmap) + bytes(body)


def uncompress_ints(buf, dtype):
    (n,) = struct.unpack_from(">I", buf, 0)
    bitmap_at, pos = 4, 4 + (n + 3) // 4
    out = np.empty(n, dtype=dtype)
    for i in range(n):
        k = (buf[bitmap_at + i // 4] >> (2 * (3 - i % 4))) & 3
        width = 1 << k
        out[i] = int.from_bytes(buf[pos:pos + width], "little", signed=True)
        pos += width
    return out


# ---------------------------------------------------------------------------------------------------- rows
def _schema_parts(header):
    sch = header["schema"][0]
    return sch["schema"], list(sch.get("blob_fields", []))


def _compressed(header, schema):
    try:
        newer = float(header.get("version", "2.0")) >= 3.0
    except ValueError:
        newer = True
    return newer and any(s.get("type") in ("int32", "int64") and "shape" in s for s in schema.values())


def _decode_field(spec, payload, compressed):
    kind = spec["type"]
    if kind == "bytes":
        return np.frombuffer(payload, dtype=np.uint8)
    if kind == "string":
        return np.array(bytes(payload).decode())
    if compressed and kind in ("int32", "int64"):
        flat = uncompress_ints(payload, _NP[kind])
    else:
        flat = np.frombuffer(payload, dtype=_NP[kind])
    shape = spec.get("shape")
    return flat.reshape(shape) if shape else flat


def decode_blob(blob, schema, blob_fields, compressed):
    if not blob_fields:
        return {}
    if len(blob_fields) == 1:
        f = blob_fields[0]
        return {f: _decode_field(schema[f], blob, compressed)}
    out, pos = {}, 0
    for f in blob_fields:
        (n,) = struct.unpack_from(">Q", blob, pos)
        out[f] = _decode_field(schema[f], blob[pos + 8:pos + 8 + n], compressed)
        pos += 8 + n
    return out


def _encode_field(spec, value, compressed, name):
    kind = spec["type"]
    if kind == "bytes":
        return bytes(value)
    if kind == "string":
        return str(value).encode()
    arr = np.ascontiguousarray(np.asarray(value, dtype=_NP[kind]))
    want = spec.get("shape")
    if want is not None and (len(want) != arr.ndim or any(w not in (-1, s) for w, s in zip(want, arr.shape))):
        raise ValueError("field %s: shape %s does not match the schema's %s" % (name, list(arr.shape), want))
    if compressed and kind in ("int32", "int64"):
        return compress_ints(arr)
    return arr.tobytes()


def encode_blob(row, schema, blob_fields, compressed):
    if not blob_fields:
        return b""
    parts = [_encode_field(schema[f], row[f], compressed, f) for f in blob_fields]
    if len(parts) == 1:
        return parts[0]
    return b"".join(struct.pack(">Q", len(p)) + p for p in parts)


def _scalar(spec, v):
    if spec["type"] == "string":
        return v.decode() if isinstance(v, bytes) else str(v)
    if spec["type"] in ("float32", "float64"):
        return float(np.asarray(v).reshape(-1)[0])
    return int(np.asarray(v).reshape(-1)[0])


# ---------------------------------------------------------------------------------------------------- reading
class ShardFile:
    """The rows of one shard file, in order."""

    def __init__(self, path):
        import msgpack
        self._unpack = msgpack.unpackb
        self.path, self.header = path, read_header(path)
        self.schema, self.blob_fields = _schema_parts(self.header)
        self.compressed = _compressed(self.header, self.schema)
        with open(path, "rb") as f:
            self._data = f.read()
        hs, ps = self.header["header_size"], self.header["page_size"]
        raws, blobs = [], []
        for page in sorted(self.header["page"], key=lambda p: p["page_id"]):
            base = hs + ps * page["page_id"]
            pos, end = base, base + page["page_size"]
            dest = blobs if page["page_type"] == "BLOB_DATA" else raws
            while pos < end:
                (n,) = struct.unpack_from("<Q", self._data, pos)
                dest.append((pos + 8, n))
                pos += 8 + n
        if self.blob_fields and len(raws) != len(blobs):
            raise MindRecordFormatError("%s: %d raw rows but %d blob rows" % (path, len(raws), len(blobs)))
        self._raws, self._blobs = raws, blobs

    def __len__(self):
        return len(self._raws)

    def read(self, i, columns=None):
        at, n = self._raws[i]
        row = {}
        raw = self._unpack(self._data[at:at + n], raw=False) if n else {}
        for name, v in raw.items():
            spec = self.schema.get(name)
            if spec is None:
                continue
            row[name] = np.array(v) if spec["type"] == "string" else np.asarray(v, dtype=_NP.get(spec["type"]))
        if self.blob_fields:
            at, n = self._blobs[i]
            row.update(decode_blob(self._data[at:at + n], self.schema, self.blob_fields, self.compressed))
        ordered = {k: row[k] for k in self.schema if k in row}
        return {k: v for k, v in ordered.items() if columns is None or k in columns}

    def index_values(self, i, fields):
        at, n = self._raws[i]
        raw = self._unpack(self._data[at:at + n], raw=False) if n else {}
        return [raw.get(f) for f in fields]


def shard_paths(path):
    """All shard files of the dataset that ``path`` (any one of its shards) belongs to."""
    header = read_header(path)
    folder = os.path.dirname(os.path.abspath(path))
    names = header.get("shard_addresses") or [os.path.basename(path)]
    return [os.path.join(folder, os.path.basename(n)) for n in names]


# ---------------------------------------------------------------------------------------------------- writing
def write_dataset(paths, schema, desc, index_fields, rows_per_shard, header_size=DEFAULT_HEADER_SIZE,
                  page_size=DEFAULT_PAGE_SIZE):
    """Writes one file + database per entry of ``paths``; ``rows_per_shard[k]`` is the list of row dicts of shard k."""
    import msgpack
    blob_fields = [f for f, s in schema.items() if s["type"] == "bytes" or "shape" in s]
    compressed = any(s["type"] in ("int32", "int64") and "shape" in s for s in schema.values())
    names = [os.path.basename(p) for p in paths]
    schema_json = [{"blob_fields": blob_fields, "desc": desc or "", "schema": schema}]
    index_json = [{"index_field": f, "schema_id": 0} for f in index_fields]
    for shard_id, (path, rows) in enumerate(zip(paths, rows_per_shard)):
        raw_rows = [msgpack.packb({f: _scalar(s, r[f]) for f, s in schema.items() if f not in blob_fields},
                                  use_bin_type=True) for r in rows]
        blob_rows = [encode_blob(r, schema, blob_fields, compressed) for r in rows]
        too_big = max([len(b) + 8 for b in blob_rows + raw_rows] + [0])
        if too_big > page_size:
            raise ValueError("a row of %d bytes does not fit the page size %d; call set_page_size" % (too_big,
                                                                                                      page_size))
        # row groups: consecutive rows whose blobs (and raw parts) fit one page each
        groups, cur, nb, nr = [], [], 0, 0
        for i in range(len(rows)):
            b, r = len(blob_rows[i]) + 8, len(raw_rows[i]) + 8
            if cur and (nb + b > page_size or nr + r > page_size):
                groups.append(cur)
                cur, nb, nr = [], 0, 0
            cur.append(i)
            nb, nr = nb + b, nr + r
        if cur:
            groups.append(cur)
        pages, chunks, index_rows = [], {}, []
        raw_page, raw_used, raw_groups, raw_type_id, blob_type_id = None, 0, [], -1, -1
        next_page = 0

        def close_raw():
            if raw_page is not None:
                pages.append({"end_row_id": 0, "page_id": raw_page, "page_size": raw_used, "page_type": "RAW_DATA",
                              "page_type_id": raw_type_id, "row_group_ids": list(raw_groups), "shard_id": shard_id,
                              "start_row_id": 0})
        for g, members in enumerate(groups):
            blob_page = next_page
            next_page += 1
            blob_type_id += 1
            buf, offsets = bytearray(), []
            for i in members:
                offsets.append((len(buf), len(buf) + 8 + len(blob_rows[i])))
                buf += struct.pack("<Q", len(blob_rows[i])) + blob_rows[i]
            chunks[blob_page] = bytes(buf)
            pages.append({"end_row_id": members[-1] + 1, "page_id": blob_page, "page_size": len(buf),
                          "page_type": "BLOB_DATA", "page_type_id": blob_type_id,
                          "row_group_ids": [{"id": g, "offset": 0}], "shard_id": shard_id,
                          "start_row_id": members[0]})
            need = sum(len(raw_rows[i]) + 8 for i in members)
            if raw_page is None or raw_used + need > page_size:
                close_raw()
                raw_page, raw_used, raw_groups = next_page, 0, []
                raw_type_id += 1
                next_page += 1
                chunks[raw_page] = b""
            raw_groups.append({"id": g, "offset": raw_used})
            rbuf = bytearray(chunks[raw_page])
            for k, i in enumerate(members):
                start = len(rbuf)
                rbuf += struct.pack("<Q", len(raw_rows[i])) + raw_rows[i]
                index_rows.append((i, raw_page, start, len(rbuf), g, blob_page, offsets[k][0], offsets[k][1]))
            chunks[raw_page] = bytes(rbuf)
            raw_used = len(rbuf)
        close_raw()
        pages.sort(key=lambda p: p["page_id"])
        header = json.dumps({"header_size": header_size, "index_fields": index_json, "page": pages,
                             "page_size": page_size, "compression_size": 0, "schema": schema_json,
                             "shard_addresses": names, "shard_id": shard_id, "statistics": None,
                             "version": VERSION}, separators=(",", ":")).encode()
        if len(header) + 8 > header_size:
            raise ValueError("the header (%d bytes) does not fit the header size %d; call set_header_size"
                             % (len(header), header_size))
        with open(path, "wb") as f:
            f.write(struct.pack("<Q", len(header)) + header)
            for page_id in sorted(chunks):
                f.seek(header_size + page_size * page_id)
                f.write(chunks[page_id])
        _write_index(path + ".db", names[shard_id], schema, index_fields, rows, index_rows)


def _write_index(db_path, shard_name, schema, index_fields, rows, index_rows):
    if os.path.exists(db_path):
        os.remove(db_path)
    con = sqlite3.connect(db_path)
    kinds = {"string": "TEXT", "float32": "NUMERIC", "float64": "NUMERIC"}
    cols = "".join(", %s_0 %s" % (f, kinds.get(schema[f]["type"], "INTEGER")) for f in index_fields)
    con.execute("CREATE TABLE INDEXES(  ROW_ID               INT  NOT NULL, PAGE_ID_RAW          INT  NOT NULL, "
                "PAGE_OFFSET_RAW      INT  NOT NULL, PAGE_OFFSET_RAW_END  INT  NOT NULL, ROW_GROUP_ID         INT  NOT "
                "NULL, PAGE_ID_BLOB         INT  NOT NULL, PAGE_OFFSET_BLOB     INT  NOT NULL, PAGE_OFFSET_BLOB_END "
                "INT  NOT NULL,INC_0 INT%s, PRIMARY KEY(ROW_ID,INC_0))" % cols)
    con.execute("CREATE TABLE SHARD_NAME(NAME TEXT NOT NULL)")
    con.execute("INSERT INTO SHARD_NAME VALUES (?)", (shard_name,))
    marks = ",".join("?" * (9 + len(index_fields)))
    for rec in index_rows:
        vals = [_scalar(schema[f], rows[rec[0]][f]) for f in index_fields]
        con.execute("INSERT INTO INDEXES VALUES (%s)" % marks, tuple(rec) + (0,) + tuple(vals))
    con.commit()
    con.close()


def read_index(db_path):
    """[(row id, raw page, raw start, raw end, row group, blob page, blob start, blob end, ...index values)]."""
    con = sqlite3.connect("file:%s?mode=ro" % db_path, uri=True)
    try:
        return [tuple(r[:8]) + tuple(r[9:]) for r in con.execute("SELECT * FROM INDEXES ORDER BY ROW_ID")]
    finally:
        con.close()


def rebuild_index(path):
    """Writes ``<path>.db`` again from the pages of the data file (a lost or stale index)."""
    shard = ShardFile(path)
    head = shard.header
    hs, ps = head["header_size"], head["page_size"]
    data = shard._data
    raw_recs, blob_by_group = [], {}
    for page in sorted(head["page"], key=lambda p: p["page_id"]):
        base = hs + ps * page["page_id"]
        pos, end = 0, page["page_size"]
        entries = []
        while pos < end:
            (n,) = struct.unpack_from("<Q", data, base + pos)
            entries.append((pos, pos + 8 + n))
            pos += 8 + n
        groups = sorted(page.get("row_group_ids") or [], key=lambda g: g["offset"])
        if page["page_type"] == "BLOB_DATA":
            gid = groups[0]["id"] if groups else 0
            blob_by_group.setdefault(gid, []).extend((page["page_id"], s, e) for s, e in entries)
        else:
            for s, e in entries:
                gid = 0
                for g in groups:
                    if g["offset"] <= s:
                        gid = g["id"]
                raw_recs.append((page["page_id"], s, e, gid))
    taken = {}
    index_rows = []
    for row_id, (raw_page, s, e, gid) in enumerate(raw_recs):
        k = taken.get(gid, 0)
        taken[gid] = k + 1
        blobs = blob_by_group.get(gid, [])
        blob_page, bs, be = blobs[k] if k < len(blobs) else (-1, 0, 0)
        index_rows.append((row_id, raw_page, s, e, gid, blob_page, bs, be))
    index_fields = [f["index_field"] for f in head.get("index_fields", [])]
    rows = [dict(zip(index_fields, shard.index_values(i, index_fields))) for i in range(len(shard))]
    names = head.get("shard_addresses") or [os.path.basename(path)]
    _write_index(path + ".db", names[head.get("shard_id", 0)], shard.schema, index_fields, rows, index_rows)
    return len(index_rows)
