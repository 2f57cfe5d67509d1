"""Checkpoint encryption: AES-GCM (default) and AES-CBC over each serialized block
(the role of core/utils/crypto.cc Encrypt / Decrypt used by save_checkpoint(enc_key=..., enc_mode=...)).

Block layout: AES-GCM  = 12-byte nonce | ciphertext | 16-byte tag;  AES-CBC = 16-byte IV | PKCS7-padded ciphertext.
Keys must be 16, 24 or 32 bytes."""
from __future__ import annotations

import os


def _check(key, mode):
    if not isinstance(key, (bytes, bytearray)) or len(key) not in (16, 24, 32):
        raise ValueError("For encryption, the key must be bytes of length 16, 24 or 32")
    if mode not in ("AES-GCM", "AES-CBC"):
        raise ValueError("enc_mode / dec_mode must be 'AES-GCM' or 'AES-CBC', but got %r" % (mode,))


def encrypt(data: bytes, key: bytes, mode: str = "AES-GCM") -> bytes:
    _check(key, mode)
    if mode == "AES-GCM":
        from cryptography.hazmat.primitives.ciphers.aead import AESGCM
        nonce = os.urandom(12)
        return nonce + AESGCM(bytes(key)).encrypt(nonce, bytes(data), None)
    from cryptography.hazmat.primitives import padding
    from cryptography.hazmat.primitives.ciphers import Cipher, algorithms, modes
    iv = os.urandom(16)
    padder = padding.PKCS7(128).padder()
    padded = padder.update(bytes(data)) + padder.finalize()
    enc = Cipher(algorithms.AES(bytes(key)), modes.CBC(iv)).encryptor()
    return iv + enc.update(padded) + enc.finalize()


def decrypt(blob: bytes, key: bytes, mode: str = "AES-GCM") -> bytes:
    _check(key, mode)
    try:
        if mode == "AES-GCM":
            from cryptography.hazmat.primitives.ciphers.aead import AESGCM
            return AESGCM(bytes(key)).decrypt(bytes(blob[:12]), bytes(blob[12:]), None)
        from cryptography.hazmat.primitives import padding
        from cryptography.hazmat.primitives.ciphers import Cipher, algorithms, modes
        dec = Cipher(algorithms.AES(bytes(key)), modes.CBC(bytes(blob[:16]))).decryptor()
        padded = dec.update(bytes(blob[16:])) + dec.finalize()
        unp = padding.PKCS7(128).unpadder()
        return unp.update(padded) + unp.finalize()
    except Exception as e:  # noqa: BLE001
        raise ValueError("Failed to decrypt the checkpoint: wrong key, wrong mode or corrupted data (%s)"
                         % type(e).__name__)
