"""``SummaryRecord``: event files of scalars, histograms and tensors.

File name ``<prefix>events.out.events.summary.<time>.<host><suffix>_MS``; every record is framed like a TFRecord
(u64 length, masked CRC32C of the length, payload, masked CRC32C of the payload) and holds one ``Event`` message of
the reference's ``summary.proto`` (ccsrc/utils/summary.proto: Event{wall_time=1, step=2, version=3, summary=5},
Summary.Value{tag=1, scalar_value=3, tensor=8, histogram=9}).  The first record carries the version string.
Parity: python/mindspore/train/summary/summary_record.py (SummaryRecord.add_value / record / flush / close),
_writer_pool.py, _summary_adapter.py (package_summary_event)."""
from __future__ import annotations

import os
import socket
import struct
import time

import numpy as np

from ..utils import proto as pb

_CRC_TABLE = None


def _crc32c(data):
    global _CRC_TABLE
    if _CRC_TABLE is None:
        tab = []
        for i in range(256):
            c = i
            for _ in range(8):
                c = (c >> 1) ^ 0x82F63B78 if c & 1 else c >> 1
            tab.append(c)
        _CRC_TABLE = tab
    crc = 0xFFFFFFFF
    for b in data:
        crc = _CRC_TABLE[(crc ^ b) & 0xFF] ^ (crc >> 8)
    return crc ^ 0xFFFFFFFF


def _masked(data):
    c = _crc32c(data)
    return (((c >> 15) | (c << 17)) + 0xA282EAD8) & 0xFFFFFFFF


def frame(payload):
    head = struct.pack("<Q", len(payload))
    return head + struct.pack("<I", _masked(head)) + payload + struct.pack("<I", _masked(payload))


def read_frames(path):
    """Payloads of an event file (checks both checksums)."""
    out = []
    with open(path, "rb") as f:
        buf = f.read()
    pos = 0
    while pos < len(buf):
        head = buf[pos:pos + 8]
        (n,) = struct.unpack("<Q", head)
        if struct.unpack("<I", buf[pos + 8:pos + 12])[0] != _masked(head):
            raise ValueError("corrupt event file: bad length checksum at byte %d" % pos)
        payload = buf[pos + 12:pos + 12 + n]
        if struct.unpack("<I", buf[pos + 12 + n:pos + 16 + n])[0] != _masked(payload):
            raise ValueError("corrupt event file: bad payload checksum at byte %d" % pos)
        out.append(payload)
        pos += 16 + n
    return out


def _to_np(v):
    import torch
    if isinstance(v, torch.Tensor):
        return v.detach().float().cpu().numpy()
    return np.asarray(v)


def _histogram(arr, bins=10):
    a = arr.astype(np.float64).ravel()
    finite = a[np.isfinite(a)]
    msg = b""
    if finite.size:
        counts, edges = np.histogram(finite, bins=bins)
        for c, lo, hi in zip(counts, edges[:-1], edges[1:]):
            msg += pb.f_bytes(1, pb.f_double(1, float(lo)) + pb.f_double(2, float(hi - lo)) + pb.f_varint(3, int(c)))
        msg += pb.f_double(5, float(finite.max())) + pb.f_double(6, float(finite.min())) + \
            pb.f_double(7, float(finite.sum()))
    msg += pb.f_varint(2, int(np.isnan(a).sum())) + pb.f_varint(3, int(np.isposinf(a).sum())) + \
        pb.f_varint(4, int(np.isneginf(a).sum())) + pb.f_varint(8, int(a.size))
    return msg


def _tensor_proto(arr):
    arr = np.ascontiguousarray(arr.astype(np.float32))
    dims = b"".join(pb.f_varint(1, d) for d in arr.shape)
    return dims + pb.f_varint(2, 1) + pb.f_bytes(9, arr.tobytes())       # data_type FLOAT, raw_data


class SummaryRecord:
    def __init__(self, log_dir, file_prefix="events", file_suffix="_MS", num_process=32, network=None,
                 max_file_size=None, raise_exception=False, export_options=None):
        os.makedirs(log_dir, exist_ok=True)
        self.log_dir = os.path.abspath(log_dir)
        name = "%s.out.events.summary.%d.%s%s" % (file_prefix, int(time.time()), socket.gethostname(), file_suffix)
        self.file_name = os.path.join(self.log_dir, name)
        self._f = open(self.file_name, "wb")
        self._pending = []
        self._closed = False
        self.max_file_size = max_file_size
        self._write(pb.f_double(1, time.time()) + pb.f_bytes(3, "MindSpore.Event:1"))

    def _write(self, event):
        data = frame(event)
        if self.max_file_size and self._f.tell() + len(data) > self.max_file_size:
            return False
        self._f.write(data)
        return True

    def add_value(self, plugin, name, value):
        if plugin not in ("scalar", "histogram", "tensor", "image", "graph", "train_lineage", "eval_lineage",
                          "dataset_graph", "custom_lineage_data"):
            raise ValueError("For 'SummaryRecord.add_value', plugin %r is not supported" % (plugin,))
        if plugin in ("scalar", "histogram", "tensor"):
            self._pending.append((plugin, name, _to_np(value)))
        return True

    def set_mode(self, mode):
        if mode not in ("train", "eval"):
            raise ValueError("mode must be 'train' or 'eval'")
        self.mode = mode

    def record(self, step, train_network=None, plugin_filter=None):
        if self._closed:
            raise RuntimeError("The SummaryRecord is closed.")
        values = b""
        for plugin, name, arr in self._pending:
            if plugin_filter is not None and not plugin_filter(plugin):
                continue
            v = pb.f_bytes(1, "%s[:%s]" % (name, plugin))
            if plugin == "scalar":
                v += pb.f_float(3, float(arr.reshape(-1)[0]))
            elif plugin == "histogram":
                v += pb.f_bytes(9, _histogram(arr))
            else:
                v += pb.f_bytes(8, _tensor_proto(arr))
            values += pb.f_bytes(1, v)
        self._pending = []
        if values:
            self._write(pb.f_double(1, time.time()) + pb.f_varint(2, int(step)) + pb.f_bytes(5, values))
        return True

    def flush(self):
        self._f.flush()

    def close(self):
        if not self._closed:
            self._f.close()
            self._closed = True

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()


def parse_event(payload):
    """{wall_time, step, version | values: {tag: scalar or dict}} of one event payload (tests, tooling)."""
    out = {"values": {}}
    for f, wt, v in pb.parse(payload):
        if f == 1:
            out["wall_time"] = struct.unpack("<d", struct.pack("<Q", v))[0]
        elif f == 2:
            out["step"] = v
        elif f == 3:
            out["version"] = v.decode()
        elif f == 5:
            for f2, _wt, val in pb.parse(v):
                if f2 != 1:
                    continue
                tag, item = None, None
                for f3, wt3, x in pb.parse(val):
                    if f3 == 1:
                        tag = x.decode()
                    elif f3 == 3:
                        item = struct.unpack("<f", struct.pack("<I", x))[0]
                    elif f3 == 9:
                        item = {"histogram_fields": len(pb.parse(x))}
                    elif f3 == 8:
                        item = {"tensor_dims": pb.repeated_ints(pb.parse(x), 1)}
                out["values"][tag] = item
    return out
