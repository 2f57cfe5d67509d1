"""The .ckpt byte layout: concatenated Checkpoint{Value{tag, TensorProto{dims, tensor_type, tensor_content}}}
messages (mindspore/ccsrc/utils/checkpoint.proto:17-44), checked against a hand-assembled protobuf."""
import numpy as np
import pytest
import torch

import mindspore_b200 as ms
from mindspore_b200.train import serialization as S


def _hand_assembled(tag, dims, tname, content):
    def varint(n):
        out = b""
        while True:
            b = n & 0x7F
            n >>= 7
            out += bytes([b | (0x80 if n else 0)])
            if not n:
                return out
    tensor = b"".join(b"\x08" + varint(d) for d in dims) + b"\x12" + varint(len(tname)) + tname.encode() + \
        b"\x1a" + varint(len(content)) + content
    value = b"\x0a" + varint(len(tag)) + tag.encode() + b"\x12" + varint(len(tensor)) + tensor
    return b"\x0a" + varint(len(value)) + value


def test_bytes_match_hand_assembled_protobuf(tmp_path):
    w = np.arange(6, dtype=np.float32).reshape(2, 3)
    path = ms.save_checkpoint([{"name": "fc.weight", "data": ms.Tensor(w)}], str(tmp_path / "a.ckpt"))
    assert open(path, "rb").read() == _hand_assembled("fc.weight", [2, 3], "Float32", w.tobytes())


def test_google_protobuf_parses_it(tmp_path):
    pb = pytest.importorskip("google.protobuf")
    from google.protobuf import descriptor_pb2, descriptor_pool, message_factory
    fd = descriptor_pb2.FileDescriptorProto(name="ckpt.proto", syntax="proto2")
    tp = fd.message_type.add(name="TensorProto")
    tp.field.add(name="dims", number=1, type=3, label=3)
    tp.field.add(name="tensor_type", number=2, type=9, label=2)
    tp.field.add(name="tensor_content", number=3, type=12, label=2)
    ck = fd.message_type.add(name="Checkpoint")
    val = ck.nested_type.add(name="Value")
    val.field.add(name="tag", number=1, type=9, label=2)
    val.field.add(name="tensor", number=2, type=11, label=1, type_name=".TensorProto")
    ck.field.add(name="value", number=1, type=11, label=3, type_name=".Checkpoint.Value")
    pool = descriptor_pool.DescriptorPool()
    pool.Add(fd)
    cls = message_factory.GetMessageClass(pool.FindMessageTypeByName("Checkpoint"))
    a = np.random.randn(4, 5).astype(np.float32)
    b = np.arange(3, dtype=np.int32)
    path = ms.save_checkpoint({"a": ms.Tensor(a), "b": ms.Tensor(b), "s": ms.Tensor(2.5)}, str(tmp_path / "m.ckpt"))
    msg = cls()
    msg.ParseFromString(open(path, "rb").read())   # concatenated messages merge their repeated fields
    assert [v.tag for v in msg.value] == ["a", "b", "s"]
    assert list(msg.value[0].tensor.dims) == [4, 5] and msg.value[0].tensor.tensor_type == "Float32"
    assert msg.value[0].tensor.tensor_content == a.tobytes()
    assert list(msg.value[2].tensor.dims) == [0]       # scalar convention


def test_dtypes_bf16_scalar_str_crc_filter(tmp_path):
    x = torch.randn(7, 3).bfloat16()
    path = ms.save_checkpoint({"x": ms.Tensor(x), "i8": ms.Tensor(np.array([1, -2], np.int8)),
                               "flag": ms.Tensor(True)}, str(tmp_path / "d.ckpt"), crc_check=True,
                              append_dict={"who": "me"})
    d = ms.load_checkpoint(path, crc_check=True)
    assert d["x"].dtype == torch.bfloat16 and torch.equal(d["x"].as_subclass(torch.Tensor), x)
    assert d["i8"].dtype == torch.int8 and d["flag"].dtype == torch.bool and d["who"] == "me"
    raw = bytearray(open(path, "rb").read())
    raw[20] ^= 0xFF
    bad = tmp_path / "bad.ckpt"
    bad.write_bytes(bytes(raw))
    with pytest.raises(ValueError, match="crc check"):
        ms.load_checkpoint(str(bad), crc_check=True)
    assert set(ms.load_checkpoint(path, filter_prefix="x")) == {"i8", "flag", "who"}
    assert set(ms.load_checkpoint(path, specify_prefix=["x", "i"])) == {"x", "i8"}


def test_large_tensor_is_chunked(tmp_path, monkeypatch):
    monkeypatch.setattr(S, "SLICE_SIZE", 1)  # 1 KB slices
    a = np.random.randn(1000).astype(np.float32)
    path = ms.save_checkpoint({"big": ms.Tensor(a)}, str(tmp_path / "big.ckpt"))
    tags = [t for t, _, _, _ in S.decode_stream(open(path, "rb").read())]
    assert tags == ["big"] * 4
    np.testing.assert_array_equal(ms.load_checkpoint(path)["big"].asnumpy(), a)


def test_errors(tmp_path):
    with pytest.raises(ValueError):
        ms.load_checkpoint(str(tmp_path / "missing.ckpt"))
    with pytest.raises(ValueError):
        ms.load_checkpoint("x.txt")
    with pytest.raises(TypeError):
        ms.save_checkpoint(3, str(tmp_path / "x.ckpt"))


@pytest.mark.parametrize("mode", ["AES-GCM", "AES-CBC"])
def test_encrypted_checkpoint_roundtrip(tmp_path, mode):
    import mindspore_b200 as ms
    key = bytes(range(16))
    w = torch.randn(5, 7)
    path = str(tmp_path / "enc.ckpt")
    ms.save_checkpoint([{"name": "w", "data": ms.Tensor(w)}], path, enc_key=key, enc_mode=mode)
    back = ms.load_checkpoint(path, dec_key=key, dec_mode=mode)
    torch.testing.assert_close(back["w"].as_subclass(torch.Tensor), w)
    with pytest.raises(ValueError):
        ms.load_checkpoint(path, dec_key=bytes(16), dec_mode=mode)


def test_safetensors_round_trip_and_check(tmp_path):
    import json
    import struct
    import numpy as np
    import torch
    import mindspore_b200 as ms
    from mindspore_b200 import nn, train
    ms.set_seed(3)
    net = nn.SequentialCell([nn.Dense(3, 4), nn.Dense(4, 2)])
    net[1].weight.set_data(net[1].weight.detach().to(torch.bfloat16))
    ck = str(tmp_path / "m.ckpt")
    ms.save_checkpoint(net, ck)
    assert train.check_checkpoint(ck) and not train.check_checkpoint(str(tmp_path / "missing.ckpt"))
    (tmp_path / "bad.ckpt").write_bytes(b"\x00\x01garbage")
    assert not train.check_checkpoint(str(tmp_path / "bad.ckpt"))
    out = train.ckpt_to_safetensors(ck)[0]
    raw = open(out, "rb").read()
    (n,) = struct.unpack_from("<Q", raw, 0)
    header = json.loads(raw[8:8 + n])
    assert header["0.weight"]["dtype"] == "F32" and header["1.weight"]["dtype"] == "BF16"
    assert header["0.weight"]["shape"] == [4, 3]
    st = train.load_safetensors(out)
    assert st["1.weight"].dtype == torch.bfloat16
    torch.testing.assert_close(st["0.weight"], net[0].weight.detach().as_subclass(torch.Tensor))
    back = train.safetensors_to_ckpt(out, save_path=str(tmp_path / "again"))[0]
    p = ms.load_checkpoint(back)
    assert np.allclose(p["0.bias"].numpy(), net[0].bias.detach().numpy())
    assert torch.equal(torch.as_tensor(p["1.weight"]).view(torch.int16),
                       net[1].weight.detach().as_subclass(torch.Tensor).view(torch.int16))


def _reference_style_file(path, values, crc=True):
    """Builds a checkpoint the way the reference writes one: google.protobuf ``SerializeToString`` of one
    ``Checkpoint`` message per value, then ``b'crc_num' + crc.to_bytes(10, 'big')``
    (mindspore/python/mindspore/train/serialization.py:255-302)."""
    import binascii
    from google.protobuf import descriptor_pb2, descriptor_pool, message_factory
    fd = descriptor_pb2.FileDescriptorProto(name="ckpt_ref.proto", syntax="proto2")
    tp = fd.message_type.add(name="TensorProto")
    tp.field.add(name="dims", number=1, type=3, label=3)
    tp.field.add(name="tensor_type", number=2, type=9, label=2)
    tp.field.add(name="tensor_content", number=3, type=12, label=2)
    ck = fd.message_type.add(name="Checkpoint")
    val = ck.nested_type.add(name="Value")
    val.field.add(name="tag", number=1, type=9, label=2)
    val.field.add(name="tensor", number=2, type=11, label=1, type_name=".TensorProto")
    ck.field.add(name="value", number=1, type=11, label=3, type_name=".Checkpoint.Value")
    pool = descriptor_pool.DescriptorPool()
    pool.Add(fd)
    cls = message_factory.GetMessageClass(pool.FindMessageTypeByName("Checkpoint"))
    blob, c = b"", 0
    for tag, dims, tname, content in values:
        m = cls()
        v = m.value.add()
        v.tag = tag
        v.tensor.dims.extend(dims)
        v.tensor.tensor_type = tname
        v.tensor.tensor_content = content
        b = m.SerializeToString()
        c = binascii.crc32(b, c)
        blob += b
    if crc:
        blob += b"crc_num" + c.to_bytes(10, byteorder="big")
    open(path, "wb").write(blob)
    return blob


def test_reads_reference_style_file_with_binary_crc_and_random_op(tmp_path):
    pytest.importorskip("google.protobuf")
    w = np.random.randn(3, 4).astype(np.float32)
    seed_state = bytes(range(40))
    path = str(tmp_path / "ref.ckpt")
    _reference_style_file(path, [("fc.weight", [3, 4], "Float32", w.tobytes()),
                                 ("random_op", [0], "random_op", seed_state)])
    for check in (True, False):
        d = ms.load_checkpoint(path, crc_check=check)
        np.testing.assert_array_equal(d["fc.weight"].asnumpy(), w)
        assert bytes(d["random_op"].numpy().tobytes()) == seed_state
    raw = bytearray(open(path, "rb").read())
    raw[30] ^= 0x55
    (tmp_path / "bad.ckpt").write_bytes(bytes(raw))
    with pytest.raises(ValueError, match="crc check"):
        ms.load_checkpoint(str(tmp_path / "bad.ckpt"), crc_check=True)


def test_written_trailer_is_the_reference_one(tmp_path):
    import binascii
    path = ms.save_checkpoint({"a": ms.Tensor(np.arange(5, dtype=np.float32))}, str(tmp_path / "c.ckpt"),
                              crc_check=True)
    raw = open(path, "rb").read()
    assert raw[-17:-10] == b"crc_num"
    assert int.from_bytes(raw[-10:], "big") == binascii.crc32(raw[:-17], 0)


def test_native_scanner_matches_python_decoder(tmp_path):
    path = ms.save_checkpoint({"a": ms.Tensor(np.arange(12, dtype=np.float32).reshape(3, 4)),
                               "s": ms.Tensor(np.int32(7))}, str(tmp_path / "n.ckpt"), append_dict={"note": "hi"})
    raw = open(path, "rb").read()
    a = [(t, d, n, bytes(c)) for t, d, n, c in S.decode_stream(raw, native=True)]
    b = [(t, d, n, bytes(c)) for t, d, n, c in S.decode_stream(raw, native=False)]
    assert a == b and [r[0] for r in a] == ["a", "s", "note"]
    assert S._decode_native(raw) is not None, "the host library's scanner was not used"


def test_encrypted_container_layout_and_legacy_blobs(tmp_path):
    """magic | tag (GCM) | block size | iv length | iv | cipher length | cipher, blocks concatenated."""
    import struct

    from mindspore_b200.train import crypto
    key = b"0123456789ABCDEF"
    blob = crypto.encrypt(b"x" * 100, key, "AES-GCM")
    magic, = struct.unpack_from("<I", blob, 0)
    block, iv_len = struct.unpack_from("<ii", blob, 20)
    cipher_len, = struct.unpack_from("<i", blob, 28 + 16)
    assert magic == 0x7F3A5ED8 and iv_len == 16 and cipher_len == 100 and block == 4 + 16 + 4 + 100
    assert len(blob) == 4 + 16 + 4 + block
    cbc = crypto.encrypt(b"x" * 100, key, "AES-CBC")
    assert struct.unpack_from("<I", cbc, 0)[0] == 0x7F3A5ED9 and struct.unpack_from("<i", cbc, 4 + 8 + 16)[0] == 112
    assert crypto.decrypt(blob + crypto.encrypt(b"y", key), key) == b"x" * 100 + b"y"
    with pytest.raises(ValueError):
        crypto.decrypt(blob, key, "AES-CBC")                       # wrong mode for this magic
    with pytest.raises(ValueError):
        crypto.decrypt(blob, b"F" * 16)
    with pytest.raises(ValueError):
        crypto.decrypt(blob[:-3], key)
    # a blob of the earlier layout (12-byte nonce | ciphertext | tag, no magic) is still read
    from cryptography.hazmat.primitives.ciphers.aead import AESGCM
    nonce = b"\x01" * 12
    assert crypto.decrypt(nonce + AESGCM(key).encrypt(nonce, b"old", None), key) == b"old"
    net = ms.nn.Dense(3, 2)
    path = str(tmp_path / "enc.ckpt")
    ms.save_checkpoint(net, path, enc_key=key, enc_mode="AES-GCM")
    raw = open(path, "rb").read()
    assert struct.unpack_from("<I", raw, 0)[0] == 0x7F3A5ED8
    back = ms.load_checkpoint(path, dec_key=key, dec_mode="AES-GCM")
    assert {"bias", "weight"} <= set(back)
