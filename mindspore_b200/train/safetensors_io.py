"""Checkpoint <-> safetensors conversion and small checkpoint utilities.

The safetensors layout is: u64 little-endian header length, JSON header mapping each tensor name to
``{"dtype", "shape", "data_offsets": [begin, end]}`` (plus an optional ``__metadata__`` string map), then the raw
little-endian tensor bytes back to back.  Written and read here directly (train/serialization.py ``ckpt_to_safetensors``
/ ``safetensors_to_ckpt`` in the reference use the safetensors package)."""
from __future__ import annotations

import json
import os
import struct

import numpy as np
import torch

_ST = {torch.float32: "F32", torch.float16: "F16", torch.bfloat16: "BF16", torch.float64: "F64", torch.int64: "I64",
       torch.int32: "I32", torch.int16: "I16", torch.int8: "I8", torch.uint8: "U8", torch.bool: "BOOL"}
_TS = {v: k for k, v in _ST.items()}


def save_safetensors(tensors, path, metadata=None):
    header, blobs, off = {}, [], 0
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    for name, t in tensors.items():
        t = t.detach().cpu().contiguous() if isinstance(t, torch.Tensor) else torch.as_tensor(np.asarray(t))
        if t.dtype not in _ST:
            raise TypeError("dtype %s of %s cannot be stored in a safetensors file" % (t.dtype, name))
        raw = (t.view(torch.uint8) if t.dtype == torch.bfloat16 else t).numpy().tobytes()
        header[name] = {"dtype": _ST[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + len(raw)]}
        blobs.append(raw)
        off += len(raw)
    hj = json.dumps(header, separators=(",", ":")).encode()
    hj += b" " * ((8 - len(hj) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for b in blobs:
            f.write(b)
    return path


def load_safetensors(path):
    with open(path, "rb") as f:
        data = f.read()
    (n,) = struct.unpack_from("<Q", data, 0)
    header = json.loads(data[8:8 + n].decode())
    base = 8 + n
    out = {}
    for name, rec in header.items():
        if name == "__metadata__":
            continue
        dt = _TS[rec["dtype"]]
        b, e = rec["data_offsets"]
        raw = bytearray(data[base + b:base + e])
        if dt == torch.bfloat16:
            t = torch.frombuffer(raw, dtype=torch.uint8).view(torch.bfloat16) if raw else torch.empty(0, dtype=dt)
        else:
            t = torch.frombuffer(raw, dtype=dt) if raw else torch.empty(0, dtype=dt)
        out[name] = t.reshape(rec["shape"]).clone()
    return out


def _each_file(path, suffix):
    if os.path.isdir(path):
        for root, _, files in os.walk(path):
            for f in sorted(files):
                if f.endswith(suffix):
                    yield os.path.join(root, f)
    else:
        yield path


def ckpt_to_safetensors(file_path, save_path=None, backend="thread"):
    """Converts one ``.ckpt`` file, or every ``.ckpt`` under a directory (keeping the tree), to ``.safetensors``."""
    from .serialization import load_checkpoint
    written = []
    for src in _each_file(file_path, ".ckpt"):
        rel = os.path.relpath(src, file_path) if os.path.isdir(file_path) else os.path.basename(src)
        dst_dir = save_path or os.path.dirname(src)
        dst = os.path.join(dst_dir, os.path.splitext(rel)[0] + ".safetensors")
        os.makedirs(os.path.dirname(dst) or ".", exist_ok=True)
        params = load_checkpoint(src)
        save_safetensors({k: torch.as_tensor(v) for k, v in params.items()}, dst, {"format": "ms"})
        written.append(dst)
    return written


def safetensors_to_ckpt(file_path, save_path=None, backend="thread"):
    from .serialization import save_checkpoint
    written = []
    for src in _each_file(file_path, ".safetensors"):
        rel = os.path.relpath(src, file_path) if os.path.isdir(file_path) else os.path.basename(src)
        dst_dir = save_path or os.path.dirname(src)
        dst = os.path.join(dst_dir, os.path.splitext(rel)[0] + ".ckpt")
        os.makedirs(os.path.dirname(dst) or ".", exist_ok=True)
        save_checkpoint([{"name": k, "data": v} for k, v in load_safetensors(src).items()], dst)
        written.append(dst)
    return written


def check_checkpoint(ckpt_file_name):
    """True when the file parses as a checkpoint (framing, CRC where present) and holds at least one parameter."""
    from .serialization import load_checkpoint
    try:
        return len(load_checkpoint(ckpt_file_name)) > 0
    except Exception:          # noqa: BLE001  (any parse failure means "not a valid checkpoint")
        return False


def get_ckpt_path_with_strategy(cur_ckpt_path, cur_strategy_path):
    """Path of a checkpoint that holds the same slices as ``cur_ckpt_path`` (another rank's file with identical
    parameter layouts according to the strategy file), or None.  Used to recover a rank whose own file is damaged."""
    import re
    from ..parallel.checkpoint_transform import _load_strategy, _world_of, region
    m = re.search(r"rank_(\d+)", cur_ckpt_path)
    if m is None:
        return cur_ckpt_path if os.path.exists(cur_ckpt_path) else None
    rank = int(m.group(1))
    if os.path.exists(cur_ckpt_path) and check_checkpoint(cur_ckpt_path):
        return cur_ckpt_path
    sf = _load_strategy(cur_strategy_path)
    per, stages = _world_of(sf)
    stage, local = rank // per, rank % per

    def regions(r):
        out = {}
        for name, e in sf.layouts.items():
            if e.stage != stage:
                continue
            unit = [c * max(e.opt_shard_size, 1) if i == 0 else c for i, c in enumerate(e.split_counts())]
            out[name] = region(e.to_layout(full_shape=unit), r)
        return out
    mine = regions(local)
    for other in range(per):
        if other == local or regions(other) != mine:
            continue
        cand = cur_ckpt_path.replace("rank_%d" % rank, "rank_%d" % (stage * per + other))
        if os.path.exists(cand) and check_checkpoint(cand):
            return cand
    return None
