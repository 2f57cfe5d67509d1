"""Minimal protobuf wire-format reader/writer (varint, length-delimited, fixed32/64) for the few schema-fixed
files this framework exchanges with the reference: checkpoints, strategy files, summaries."""
import struct


def varint(n):
    out = bytearray()
    n &= 0xFFFFFFFFFFFFFFFF
    while True:
        b = n & 0x7F
        n >>= 7
        if n:
            out.append(b | 0x80)
        else:
            out.append(b)
            return bytes(out)


def read_varint(buf, pos):
    shift = result = 0
    while True:
        b = buf[pos]
        pos += 1
        result |= (b & 0x7F) << shift
        if not b & 0x80:
            return result, pos
        shift += 7


def f_varint(field, value):
    return varint(field << 3) + varint(value)


def f_bytes(field, payload):
    if isinstance(payload, str):
        payload = payload.encode()
    return varint((field << 3) | 2) + varint(len(payload)) + bytes(payload)


def f_double(field, value):
    return varint((field << 3) | 1) + struct.pack("<d", value)


def f_float(field, value):
    return varint((field << 3) | 5) + struct.pack("<f", value)


def signed(v, bits=64):
    return v - (1 << bits) if v >= (1 << (bits - 1)) else v


def parse(buf):
    """[(field, wire_type, value)]: value is int for varint/fixed, bytes for length-delimited."""
    out, pos, n = [], 0, len(buf)
    buf = bytes(buf)
    while pos < n:
        key, pos = read_varint(buf, pos)
        field, wt = key >> 3, key & 7
        if wt == 0:
            v, pos = read_varint(buf, pos)
        elif wt == 2:
            ln, pos = read_varint(buf, pos)
            v = buf[pos:pos + ln]
            pos += ln
        elif wt == 1:
            v = struct.unpack_from("<Q", buf, pos)[0]
            pos += 8
        elif wt == 5:
            v = struct.unpack_from("<I", buf, pos)[0]
            pos += 4
        else:
            raise ValueError("unsupported protobuf wire type %d" % wt)
        out.append((field, wt, v))
    return out


def repeated_ints(fields, field):
    """Values of a repeated integer field, packed or not."""
    vals = []
    for f, wt, v in fields:
        if f != field:
            continue
        if wt == 0:
            vals.append(v)
        else:
            pos = 0
            while pos < len(v):
                x, pos = read_varint(v, pos)
                vals.append(x)
    return vals
