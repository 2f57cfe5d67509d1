"""Encryption of checkpoints and exported graphs in the reference's on-disk container
(core/utils/crypto.cc Encrypt / Decrypt, used by save_checkpoint(enc_key=..., enc_mode=...) and export / load).

An encrypted file is a sequence of blocks of at most 64 MiB of plaintext each:

    u32  magic           0x7F3A5ED8 (AES-GCM) or 0x7F3A5ED9 (AES-CBC), little endian
    16 B tag             AES-GCM only
    i32  block size      = 4 + iv length + 4 + cipher length
    i32  iv length       always 16
    16 B iv              (used as a 16-byte GCM nonce / the CBC initialisation vector)
    i32  cipher length
    ...  ciphertext      (CBC: PKCS7 padded)

so encrypted pieces can be concatenated and are decrypted by walking the blocks.  Keys are 16, 24 or 32 bytes.
Files written by earlier versions of this module (one ``nonce | ciphertext | tag`` or ``iv | ciphertext`` blob
without the magic number) are still read."""
from __future__ import annotations

import os
import struct

GCM_MAGIC, CBC_MAGIC = 0x7F3A5ED8, 0x7F3A5ED9
MAX_BLOCK = 64 * 1024 * 1024
_IV_LEN = 16


def _check(key, mode):
    if not isinstance(key, (bytes, bytearray)) or len(key) not in (16, 24, 32):
        raise ValueError("For encryption, the key must be bytes of length 16, 24 or 32")
    if mode not in ("AES-GCM", "AES-CBC"):
        raise ValueError("enc_mode / dec_mode must be 'AES-GCM' or 'AES-CBC', but got %r" % (mode,))


def _cbc(key, iv, data, encrypt):
    from cryptography.hazmat.primitives import padding
    from cryptography.hazmat.primitives.ciphers import Cipher, algorithms, modes
    cipher = Cipher(algorithms.AES(bytes(key)), modes.CBC(bytes(iv)))
    if encrypt:
        padder = padding.PKCS7(128).padder()
        padded = padder.update(bytes(data)) + padder.finalize()
        enc = cipher.encryptor()
        return enc.update(padded) + enc.finalize()
    dec = cipher.decryptor()
    padded = dec.update(bytes(data)) + dec.finalize()
    unp = padding.PKCS7(128).unpadder()
    return unp.update(padded) + unp.finalize()


def is_cipher(blob) -> bool:
    """Whether the bytes start with one of the container's magic numbers."""
    return len(blob) >= 4 and struct.unpack_from("<I", blob, 0)[0] in (GCM_MAGIC, CBC_MAGIC)


def encrypt(data: bytes, key: bytes, mode: str = "AES-GCM") -> bytes:
    _check(key, mode)
    data = bytes(data)
    out = bytearray()
    for off in range(0, max(len(data), 1), MAX_BLOCK):
        chunk = data[off:off + MAX_BLOCK]
        iv = os.urandom(_IV_LEN)
        if mode == "AES-GCM":
            from cryptography.hazmat.primitives.ciphers.aead import AESGCM
            sealed = AESGCM(bytes(key)).encrypt(iv, chunk, None)
            cipher, tag = sealed[:-16], sealed[-16:]
            out += struct.pack("<I", GCM_MAGIC) + tag
        else:
            cipher = _cbc(key, iv, chunk, True)
            out += struct.pack("<I", CBC_MAGIC)
        out += struct.pack("<i", 4 + _IV_LEN + 4 + len(cipher)) + struct.pack("<i", _IV_LEN) + iv
        out += struct.pack("<i", len(cipher)) + cipher
    return bytes(out)


def _fail(e):
    raise ValueError("Failed to decrypt the checkpoint: wrong key, wrong mode or corrupted data (%s)"
                     % type(e).__name__) from e


def _decrypt_legacy(blob, key, mode):
    try:
        if mode == "AES-GCM":
            from cryptography.hazmat.primitives.ciphers.aead import AESGCM
            return AESGCM(bytes(key)).decrypt(bytes(blob[:12]), bytes(blob[12:]), None)
        return _cbc(key, blob[:16], blob[16:], False)
    except Exception as e:  # noqa: BLE001
        _fail(e)


def decrypt(blob: bytes, key: bytes, mode: str = "AES-GCM") -> bytes:
    _check(key, mode)
    blob = bytes(blob)
    if not is_cipher(blob):
        return _decrypt_legacy(blob, key, mode)
    want = GCM_MAGIC if mode == "AES-GCM" else CBC_MAGIC
    out, pos = bytearray(), 0
    try:
        while pos < len(blob):
            (magic,) = struct.unpack_from("<I", blob, pos)
            pos += 4
            if magic != want:
                raise ValueError("the data is not an encrypted %s file and cannot be decrypted with that mode" % mode)
            tag = b""
            if mode == "AES-GCM":
                tag = blob[pos:pos + 16]
                pos += 16
            block_size, iv_len = struct.unpack_from("<ii", blob, pos)
            if iv_len != _IV_LEN or block_size < 4 + _IV_LEN + 4:
                raise ValueError("malformed block header (iv length %d, block size %d)" % (iv_len, block_size))
            iv = blob[pos + 8:pos + 8 + iv_len]
            (cipher_len,) = struct.unpack_from("<i", blob, pos + 8 + iv_len)
            if 4 + iv_len + 4 + cipher_len != block_size:
                raise ValueError("malformed block: the lengths do not add up")
            start = pos + 8 + iv_len + 4
            cipher = blob[start:start + cipher_len]
            if len(cipher) != cipher_len:
                raise ValueError("truncated block")
            pos = start + cipher_len
            if mode == "AES-GCM":
                from cryptography.hazmat.primitives.ciphers.aead import AESGCM
                out += AESGCM(bytes(key)).decrypt(iv, cipher + tag, None)
            else:
                out += _cbc(key, iv, cipher, False)
    except Exception as e:  # noqa: BLE001
        _fail(e)
    return bytes(out)
