"""Checkpoint save / load in the reference's ``.ckpt`` layout.

A ``.ckpt`` file is a *concatenation of serialized ``Checkpoint`` protobuf messages*
(mindspore/ccsrc/utils/checkpoint.proto:17-44)::

    message Checkpoint { message Value { required string tag = 1;
                                         oneof value { TensorProto tensor = 2; MapTensorProto maptensor = 3; } }
                         repeated Value value = 1; }
    message TensorProto { repeated int64 dims = 1; required string tensor_type = 2;
                          required bytes tensor_content = 3; }

Tensors above 512 MB are written as several consecutive values with the same tag; an optional trailer
``crc_num`` + the CRC32 as 10 big-endian bytes follows when ``crc_check`` is on; AES-GCM/CBC encryption wraps
each block.  The bytes are produced here in Python; ``csrc/host/ckpt_codec.cpp`` is a native encoder / decoder of
the same wire format (``_native.host().msb_ckpt_*``) that ``tests/test_ckpt_format.py`` checks against this one.

Parity: mindspore/python/mindspore/train/serialization.py:255-375 (_exec_save), :436-583
(save_checkpoint), :1076-1128 (_load_into_param_dict), :1139-1252 (load_checkpoint), :1406-1438
(_parse_ckpt_proto), :1487-1573 (load_param_into_net), :312-321 (random_op), :2929 (async save).
"""
from __future__ import annotations

import binascii
import os
import stat
import threading

import numpy as np
import torch

from ..common import dtype as mstype
from ..common.parameter import Parameter
from ..common.tensor import Tensor
from ..nn.cell import Cell
from ..utils.log import logger

SLICE_SIZE = 512 * 1024          # KB: tensors larger than 512 MB are split (serialization.py:91)
_CRC_TAG = b"crc_num"
_ckpt_mutex = threading.RLock()
_async_threads = []


# ------------------------------------------------------------------------------------ protobuf wire helpers
def _varint(n):
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


def _read_varint(buf, pos):
    shift = result = 0
    while True:
        b = buf[pos]
        pos += 1
        result |= (b & 0x7F) << shift
        if not b & 0x80:
            return result, pos
        shift += 7


def _ld(field, payload):
    return _varint((field << 3) | 2) + _varint(len(payload)) + payload


def encode_value(tag, dims, type_name, content):
    """One ``Checkpoint`` message holding one ``Value`` (what the reference appends per slice)."""
    tp = b"".join(_varint((1 << 3) | 0) + _varint(d if d >= 0 else d + (1 << 64)) for d in dims)
    tp += _ld(2, type_name.encode()) + _ld(3, bytes(content))
    value = _ld(1, tag.encode()) + _ld(2, tp)
    return _ld(1, value)


def _decode_native(buf):
    """Indexes the stream with the C++ scanner (csrc/host/ckpt_codec.cpp) -> list of records, or None when the host
    library is not loadable or the image needs the Python decoder's error reporting."""
    import ctypes
    try:
        from .. import _native
        lib = _native.host()
        scan = lib.msb_ckpt_scan
    except Exception:  # noqa: BLE001
        return None
    scan.restype = ctypes.c_int
    n = len(buf)
    raw = (ctypes.c_ubyte * n).from_buffer_copy(buf) if not isinstance(buf, bytearray) else \
        (ctypes.c_ubyte * n).from_buffer(buf)
    cap, dcap = 4096, 16384
    while True:
        rec = (ctypes.c_int64 * (4 * cap))()
        dims = (ctypes.c_int64 * dcap)()
        didx = (ctypes.c_int32 * (2 * cap))()
        types = ctypes.create_string_buffer(16 * cap)
        r = scan(raw, ctypes.c_uint64(n), cap, rec, dims, dcap, didx, types)
        if r == -1:
            cap, dcap = cap * 4, dcap * 4
            continue
        if r < 0:
            return None
        break
    view = memoryview(raw).cast("B")
    out = []
    for i in range(r):
        to, tl, co, cl = rec[4 * i:4 * i + 4]
        d0, dn = didx[2 * i], didx[2 * i + 1]
        dd = [d - (1 << 64) if d >= (1 << 63) else d for d in dims[d0:d0 + dn]]
        out.append((bytes(view[to:to + tl]).decode(), dd, types.raw[16 * i:16 * i + 16].rstrip(b"\0").decode(),
                    view[co:co + cl]))
    return out


def decode_stream(buf, native=True):
    """Yields (tag, dims, type_name, content_memoryview) for every Value in a concatenated stream.  The index is
    built by the native scanner when the host library is available; the Python decoder below is the fallback and
    the one that reports where a corrupt image breaks."""
    if native and len(buf) > 0:
        recs = _decode_native(buf)
        if recs is not None:
            yield from recs
            return
    view = memoryview(buf)
    pos, n = 0, len(buf)
    while pos < n:
        key, pos = _read_varint(buf, pos)
        if key != ((1 << 3) | 2):
            raise ValueError("corrupt checkpoint: unexpected field key %d at byte %d" % (key, pos))
        ln, pos = _read_varint(buf, pos)
        end = pos + ln
        tag, dims, tname, content = None, [], None, b""
        while pos < end:
            k, pos = _read_varint(buf, pos)
            l2, pos = _read_varint(buf, pos)
            if k == ((1 << 3) | 2):
                tag = bytes(view[pos:pos + l2]).decode()
            elif k == ((2 << 3) | 2):
                p2, e2 = pos, pos + l2
                while p2 < e2:
                    kk, p2 = _read_varint(buf, p2)
                    if kk == ((1 << 3) | 0):
                        d, p2 = _read_varint(buf, p2)
                        dims.append(d - (1 << 64) if d >= (1 << 63) else d)
                    elif kk == ((1 << 3) | 2):  # packed dims
                        l3, p2 = _read_varint(buf, p2)
                        e3 = p2 + l3
                        while p2 < e3:
                            d, p2 = _read_varint(buf, p2)
                            dims.append(d)
                    elif kk == ((2 << 3) | 2):
                        l3, p2 = _read_varint(buf, p2)
                        tname = bytes(view[p2:p2 + l3]).decode()
                        p2 += l3
                    elif kk == ((3 << 3) | 2):
                        l3, p2 = _read_varint(buf, p2)
                        content = view[p2:p2 + l3]
                        p2 += l3
                    else:
                        raise ValueError("corrupt checkpoint: unknown TensorProto field %d" % kk)
            pos += l2
        yield tag, dims, tname, content
        pos = end


# ------------------------------------------------------------------------------------ tensor <-> bytes
def _tensor_bytes(t):
    t = t.detach().as_subclass(torch.Tensor).cpu().contiguous()
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).numpy().tobytes()
    return t.numpy().tobytes()


def _bytes_tensor(content, dims, type_name):
    if type_name == "str":
        return bytes(content).decode()
    if type_name == "random_op":        # raw generator state (reference serialization.py:312-321)
        return torch.from_numpy(np.frombuffer(content, dtype=np.uint8).copy())
    try:
        dt = mstype.ckpt_type_from_name(type_name)
    except KeyError:
        raise ValueError("unknown tensor_type %r in checkpoint" % type_name)
    shape = () if list(dims) == [0] else tuple(dims)
    if dt == torch.bfloat16:
        arr = np.frombuffer(content, dtype=np.int16).copy()
        t = torch.from_numpy(arr).view(torch.bfloat16)
    else:
        arr = np.frombuffer(content, dtype=mstype.dtype_to_nptype(dt)).copy()
        t = torch.from_numpy(arr)
    return t.reshape(shape)


def _check_name(ckpt_file_name):
    if not isinstance(ckpt_file_name, str):
        raise TypeError("For 'save_checkpoint', 'ckpt_file_name' must be string, but got %s" % type(ckpt_file_name))
    if ckpt_file_name.endswith("/") or os.path.isdir(ckpt_file_name):
        raise ValueError("For 'save_checkpoint', 'ckpt_file_name' must be a file path, but got %r" % ckpt_file_name)
    if not ckpt_file_name.endswith(".ckpt"):
        ckpt_file_name += ".ckpt"
    d = os.path.dirname(os.path.abspath(ckpt_file_name))
    os.makedirs(d, exist_ok=True)
    return os.path.abspath(ckpt_file_name)


def _collect(save_obj, integrated_save, choice_func):
    """-> list of (name, tensor or str)"""
    items = []
    if isinstance(save_obj, Cell):
        if integrated_save:
            from ..parallel.checkpoint import gather_full_parameters
            params = gather_full_parameters(save_obj)
        else:
            params = [(p.name, p) for p in save_obj.get_parameters()]
        seen = set()
        for name, p in params:
            if name in seen:
                continue
            seen.add(name)
            if choice_func is None or choice_func(name):
                items.append((name, p))
    elif isinstance(save_obj, dict):
        for k, v in save_obj.items():
            if not isinstance(k, str):
                raise TypeError("For 'save_checkpoint', dict keys must be str")
            if choice_func is None or choice_func(k):
                items.append((k, v))
    elif isinstance(save_obj, list):
        for it in save_obj:
            if not (isinstance(it, dict) and "name" in it and "data" in it):
                raise TypeError("For 'save_checkpoint', list items must be dicts with 'name' and 'data'")
            if choice_func is None or choice_func(it["name"]):
                items.append((it["name"], it["data"]))
    else:
        raise TypeError("For 'save_checkpoint', 'save_obj' must be nn.Cell, list or dict, but got %s" % type(save_obj))
    return items


def _to_records(items, append_dict):
    recs = []
    for name, v in items:
        if isinstance(v, str):
            recs.append((name, [0], "str", v.encode()))
            continue
        if name == "random_op" and isinstance(v, (bytes, bytearray)):
            recs.append((name, [0], "random_op", bytes(v)))
            continue
        if not isinstance(v, torch.Tensor):
            v = Tensor(v)
        if name == "random_op":
            recs.append((name, [0], "random_op", _tensor_bytes(v.to(torch.uint8))))
            continue
        dims = list(v.shape) if v.dim() > 0 else [0]
        recs.append((name, dims, mstype.ckpt_type_name(v.dtype), v))
    if append_dict:
        if not isinstance(append_dict, dict):
            raise TypeError("For 'save_checkpoint', 'append_dict' must be dict")
        for k, v in append_dict.items():
            if not isinstance(k, str):
                raise TypeError("For 'save_checkpoint', keys of 'append_dict' must be str")
            if isinstance(v, str):
                recs.append((k, [0], "str", v.encode()))
            elif isinstance(v, (int, float, bool, torch.Tensor, np.ndarray, np.generic)):
                t = v if isinstance(v, torch.Tensor) else Tensor(v)
                recs.append((k, list(t.shape) if t.dim() > 0 else [0], mstype.ckpt_type_name(t.dtype), t))
            else:
                raise TypeError("For 'save_checkpoint', values of 'append_dict' must be int, float, bool, str or "
                                "Tensor, but got %s" % type(v))
    return recs


def _write(path, recs, enc_key, enc_mode, crc_check):
    tmp = path + ".tmp%d" % os.getpid()
    crc = 0
    enc = None
    if enc_key is not None:
        from . import crypto
        enc = lambda b: crypto.encrypt(b, enc_key, enc_mode)  # noqa: E731
    with _ckpt_mutex:
        if os.path.exists(path):
            os.chmod(path, stat.S_IWUSR)
            os.remove(path)
        with open(tmp, "wb") as f:
            for name, dims, tname, payload in recs:
                raw = payload if isinstance(payload, (bytes, bytearray)) else _tensor_bytes(payload)
                step = SLICE_SIZE * 1024
                for off in range(0, max(len(raw), 1), step):
                    block = encode_value(name, dims, tname, raw[off:off + step])
                    if enc is not None:
                        block = enc(block)                # self-delimiting: blocks are simply concatenated
                    if crc_check:
                        crc = binascii.crc32(block, crc)
                    f.write(block)
            if crc_check:
                f.write(_CRC_TAG + crc.to_bytes(10, "big"))          # reference serialization.py:302
        os.replace(tmp, path)
        os.chmod(path, stat.S_IRUSR | stat.S_IWUSR)


def save_checkpoint(save_obj, ckpt_file_name, integrated_save=True, async_save=False, append_dict=None,
                    enc_key=None, enc_mode="AES-GCM", choice_func=None, crc_check=False, **kwargs):
    path = _check_name(ckpt_file_name)
    if choice_func is not None and not callable(choice_func):
        raise TypeError("For 'save_checkpoint', 'choice_func' must be callable")
    items = _collect(save_obj, integrated_save, choice_func)
    if isinstance(save_obj, Cell):
        from ..common.seed import get_rng_state
        items.append(("random_op", get_rng_state().to(torch.uint8)))
    recs = _to_records(items, append_dict)
    if async_save:
        # snapshot to host first so that training may mutate parameters while the file is written
        recs = [(n, d, t, p if isinstance(p, (bytes, bytearray)) else _tensor_bytes(p)) for n, d, t, p in recs]
        th = threading.Thread(target=_write, args=(path, recs, enc_key, enc_mode, crc_check), name="asyn_save_ckpt")
        th.start()
        _async_threads.append(th)
    else:
        _write(path, recs, enc_key, enc_mode, crc_check)
    logger.info("Saved checkpoint to %s", path)
    return path


def async_ckpt_thread_status():
    _async_threads[:] = [t for t in _async_threads if t.is_alive()]
    return bool(_async_threads)


def wait_async_save():
    for t in list(_async_threads):
        t.join()
    _async_threads.clear()


def _read_file(path, dec_key, dec_mode, crc_check):
    with open(path, "rb") as f:
        data = f.read()
    # trailer = b"crc_num" + 10 big-endian bytes (reference serialization.py:1417-1425); files written by older
    # versions of this module carried 10 ASCII digits instead and are still accepted
    has_crc = len(data) >= 17 and data[-17:-10] == _CRC_TAG
    if has_crc:
        tail = data[-10:]
        expect = int(tail) if tail.isdigit() and tail[:1] != b"\x00" else int.from_bytes(tail, "big")
        data = data[:-17]
        if crc_check and binascii.crc32(data) != expect:
            raise ValueError("For 'load_checkpoint', the crc check has failed. Please check whether the ckpt file "
                             "is damaged.")
    elif crc_check:
        logger.warning("crc_check is on but %s carries no crc trailer", path)
    if dec_key is not None:
        from . import crypto
        if crypto.is_cipher(data):
            data = crypto.decrypt(data, dec_key, dec_mode)
        else:                                             # files of earlier versions: u64 length + blob, repeated
            out, pos = bytearray(), 0
            while pos < len(data):
                ln = int.from_bytes(data[pos:pos + 8], "little")
                pos += 8
                out += crypto.decrypt(bytes(data[pos:pos + ln]), dec_key, dec_mode)
                pos += ln
            data = bytes(out)
    return data


def load_checkpoint(ckpt_file_name, net=None, strict_load=False, filter_prefix=None, dec_key=None,
                    dec_mode="AES-GCM", specify_prefix=None, choice_func=None, crc_check=False,
                    remove_redundancy=False, **kwargs):
    if not isinstance(ckpt_file_name, str) or not ckpt_file_name.endswith(".ckpt"):
        raise ValueError("For 'load_checkpoint', the checkpoint file should end with '.ckpt', please input the "
                         "correct 'ckpt_file_name'.")
    if not os.path.exists(ckpt_file_name):
        raise ValueError("For 'load_checkpoint', the checkpoint file: %s does not exist, please check whether the "
                         "'ckpt_file_name' is correct." % ckpt_file_name)
    for name, v in (("filter_prefix", filter_prefix), ("specify_prefix", specify_prefix)):
        if v is not None and not isinstance(v, (str, list, tuple)):
            raise TypeError("For 'load_checkpoint', '%s' must be str, list[str] or tuple[str]" % name)
    filt = (filter_prefix,) if isinstance(filter_prefix, str) else tuple(filter_prefix or ())
    spec = (specify_prefix,) if isinstance(specify_prefix, str) else tuple(specify_prefix or ())
    try:
        data = _read_file(ckpt_file_name, dec_key, dec_mode, crc_check)
        chunks, order = {}, []
        for tag, dims, tname, content in decode_stream(data):
            if tag not in chunks:
                chunks[tag] = [dims, tname, []]
                order.append(tag)
            chunks[tag][2].append(content)
    except ValueError:
        raise
    except Exception as e:  # noqa: BLE001
        raise ValueError("Failed to read the checkpoint file %s (%s). May not have permission to read it, or the "
                         "file is damaged / encrypted." % (ckpt_file_name, e))
    out = {}
    for tag in order:
        if filt and tag.startswith(filt):
            continue
        if spec and not tag.startswith(spec):
            continue
        if choice_func is not None and not choice_func(tag):
            continue
        dims, tname, parts = chunks[tag]
        content = parts[0] if len(parts) == 1 else b"".join(bytes(p) for p in parts)
        val = _bytes_tensor(content, dims, tname)
        if isinstance(val, str):
            out[tag] = val
        elif tag == "random_op":
            out[tag] = val
        else:
            out[tag] = Parameter(val, name=tag, device="cpu")
    if not out:
        raise ValueError("The loaded parameter dict is empty after filter or specify, please check whether "
                         "'filter_prefix' or 'specify_prefix' are set correctly.")
    if net is not None:
        load_param_into_net(net, out, strict_load)
    return out


def load_param_into_net(net, parameter_dict, strict_load=False, remove_redundancy=False):
    if not isinstance(net, Cell):
        raise TypeError("For 'load_param_into_net', the argument 'net' should be a Cell, but got %s" % type(net))
    if not isinstance(parameter_dict, dict):
        raise TypeError("For 'load_param_into_net', the argument 'parameter_dict' should be a dict, but got %s"
                        % type(parameter_dict))
    for k, v in parameter_dict.items():
        if not isinstance(k, str) or not isinstance(v, (torch.Tensor, str)):
            raise TypeError("For 'load_param_into_net', the element in 'parameter_dict' should be 'str' and "
                            "'Parameter', but got %s and %s" % (type(k), type(v)))
    if "random_op" in parameter_dict:
        from ..common.seed import set_rng_state
        try:
            set_rng_state(parameter_dict["random_op"].detach().as_subclass(torch.Tensor).to(torch.uint8).cpu())
        except Exception:  # noqa: BLE001
            logger.warning("could not restore the RNG state stored in the checkpoint")
    not_loaded, loaded = [], set()
    params = list(net.parameters_and_names())

    def _assign(p, new, name):
        new = new.detach().as_subclass(torch.Tensor)
        if tuple(new.shape) != tuple(p.shape):
            if p.param_layout is not None and p.full_shape is not None and tuple(new.shape) == tuple(p.full_shape):
                from ..parallel.layout import slice_for_rank
                from .. import context
                new = slice_for_rank(new, p.param_layout, context.get_auto_parallel_context("global_rank"))
            elif new.numel() == p.numel() and new.dim() <= 1 and p.dim() <= 1:
                new = new.reshape(p.shape)
            else:
                raise RuntimeError("For 'load_param_into_net', %s in the argument 'net' should have the same shape "
                                   "as %s in the argument 'parameter_dict'. But got its shape %s in the argument "
                                   "'net' and shape %s in the argument 'parameter_dict'. May you need to check "
                                   "whether the checkpoint you loaded is correct or the batch size and so on in "
                                   "the 'net' and 'parameter_dict' are same." % (name, name, tuple(p.shape),
                                                                                 tuple(new.shape)))
        if new.dtype != p.dtype:
            if strict_load and not (new.is_floating_point() and p.is_floating_point()):
                raise RuntimeError("For 'load_param_into_net', %s has dtype %s in the net but %s in the "
                                   "checkpoint (strict_load)" % (name, p.dtype, new.dtype))
            new = new.to(p.dtype)
        with torch.no_grad():
            torch.Tensor.copy_(p, new.to(p.device))
        if ("fp32_master." + name) not in parameter_dict and "fp32_master.opt_shard" not in parameter_dict:
            # no exact master in the checkpoint: the master (whole, or this rank's slice) follows the loaded weights
            from ..common.parameter import sync_master
            sync_master(p, new)

    for _, p in params:
        if p.name in parameter_dict and isinstance(parameter_dict[p.name], torch.Tensor):
            _assign(p, parameter_dict[p.name], p.name)
            loaded.add(p.name)
        else:
            not_loaded.append(p.name)
    if not_loaded and not strict_load:
        # retry with a common prefix stripped / added (reference: _load_dismatch_prefix_params)
        ck_names = [k for k in parameter_dict if k not in loaded and isinstance(parameter_dict[k], torch.Tensor)]
        still = []
        for _, p in params:
            if p.name not in not_loaded:
                continue
            cand = [k for k in ck_names if k.endswith("." + p.name) or p.name.endswith("." + k)]
            if len(cand) == 1 and tuple(parameter_dict[cand[0]].shape) == tuple(p.shape):
                _assign(p, parameter_dict[cand[0]], p.name)
                loaded.add(cand[0])
            else:
                still.append(p.name)
        not_loaded = still
    ckpt_not_loaded = [k for k in parameter_dict if k not in loaded and k != "random_op"
                       and isinstance(parameter_dict[k], torch.Tensor)]
    if "global_step" in loaded:
        # the host-side step drives the learning-rate schedule and Adam's bias correction
        for _, cell in net.cells_and_names():
            if hasattr(cell, "sync_step_from_checkpoint") and \
                    any(q is getattr(cell, "global_step", None) for _, q in params):
                cell.sync_step_from_checkpoint()
    if not_loaded:
        logger.warning("For 'load_param_into_net', %d parameters in the 'net' are not loaded: %s", len(not_loaded),
                       not_loaded[:8])
    return not_loaded, ckpt_not_loaded


def load_segmented_checkpoints(ckpt_file_dir, net=None, strict_load=False, filter_prefix=None, dec_key=None,
                               dec_mode="AES-GCM", specify_prefix=None, choice_func=None):
    files = sorted(os.path.join(ckpt_file_dir, f) for f in os.listdir(ckpt_file_dir) if f.endswith(".ckpt"))
    merged = {}
    for f in files:
        merged.update(load_checkpoint(f, None, strict_load, filter_prefix, dec_key, dec_mode, specify_prefix,
                                      choice_func))
    if net is not None:
        load_param_into_net(net, merged, strict_load)
    return merged


def parse_print(print_file_name):
    """Reads a file written by the ``Print`` operator (``context.set_context(print_file_path=...)``): one record per
    printed value, returned as a list of strings (scalars / text) and numpy arrays (tensors), in print order.  The
    file is this framework's checkpoint container (a list of named values), so the reader is the checkpoint reader."""
    import os
    if not os.path.isfile(print_file_name):
        raise ValueError("The print_file_name %r does not exist" % (print_file_name,))
    with open(print_file_name, "rb") as f:
        data = f.read()
    if not data:
        return []
    try:
        records = decode_stream(data)
    except Exception:  # noqa: BLE001  (a plain-text print file: one value per line)
        return data.decode(errors="replace").splitlines()
    out = []
    for rec in records:
        value = rec[1] if isinstance(rec, (tuple, list)) and len(rec) > 1 else rec
        out.append(value.numpy() if hasattr(value, "numpy") else value)
    return out


def load_checkpoint_async(ckpt_file_name, net=None, strict_load=False, filter_prefix=None, dec_key=None,
                          dec_mode="AES-GCM", specify_prefix=None, choice_func=None):
    """Starts ``load_checkpoint`` on a worker thread and returns a future-like object: ``result()`` waits and returns
    the parameter dict (the reference overlaps the file read with graph compilation the same way)."""
    from concurrent.futures import ThreadPoolExecutor
    pool = ThreadPoolExecutor(max_workers=1, thread_name_prefix="ckpt-load")
    fut = pool.submit(load_checkpoint, ckpt_file_name, net, strict_load, filter_prefix, dec_key, dec_mode,
                      specify_prefix, choice_func)
    fut.add_done_callback(lambda _f: pool.shutdown(wait=False))
    return fut


def export_split_mindir(net, *inputs, file_name, devices_num=8, **kwargs):
    """Exports the graph once per device of a model-parallel job (``<file_name>_rank_<r>.mindir``): every file holds
    this rank's slices of the sharded parameters.  Runs on each rank for its own file; ``devices_num`` is checked
    against the parallel context."""
    from .. import context
    n = context.get_auto_parallel_context("device_num")
    if devices_num != n:
        raise ValueError("export_split_mindir: devices_num %d differs from the parallel context's device_num %d"
                         % (devices_num, n))
    rank = context.get_auto_parallel_context("global_rank")
    base = file_name[:-7] if file_name.endswith(".mindir") else file_name
    return export(net, *inputs, file_name="%s_rank_%d" % (base, rank), file_format="MINDIR", **kwargs)


def export(net, *inputs, file_name, file_format, **kwargs):
    """Exports ``net`` traced on ``inputs``.  MINDIR: one ``<file_name>.mindir`` file holding the forward graph and the
    weights, in the reference's protobuf layout (``graph/mindir_proto.py``) when every node is a primitive, else in
    this framework's own container (``graph/mindir.py``; ``container="native"`` forces it, ``container="proto"``
    insists on protobuf); ``enc_key`` / ``enc_mode`` encrypt it like a checkpoint.  ONNX: ``<file_name>.onnx`` at opset
    17 (``graph/onnx_proto.py``).  AIR targets the Ascend graph engine and is not produced."""
    if file_format not in ("MINDIR", "ONNX", "AIR"):
        raise ValueError("For 'export', 'file_format' must be one of AIR, ONNX, MINDIR, but got %r" % file_format)
    if file_format == "AIR":
        raise NotImplementedError("AIR files feed the Ascend graph engine and are not produced by this build")
    from ..graph import jit as _jit
    from ..graph import mindir
    was_training = getattr(net, "training", False)
    net.set_train(False)
    try:
        g = _jit.trace_cell(net, inputs)
    finally:
        net.set_train(was_training)
    if file_format == "ONNX":
        from ..graph import onnx_proto
        return onnx_proto.save_onnx(g, file_name if file_name.endswith(".onnx") else file_name + ".onnx")
    path = file_name if file_name.endswith(".mindir") else file_name + ".mindir"
    container = kwargs.get("container", "auto")
    if container not in ("auto", "proto", "native"):
        raise ValueError("For 'export', 'container' must be auto, proto or native, but got %r" % container)
    written = False
    if container in ("auto", "proto"):
        from ..graph import mindir_proto
        try:
            mindir_proto.save_model_proto(g, path)
            written = True
        except mindir.MindIRError:
            if container == "proto":
                raise
    if not written:
        mindir.save_mindir(g, path)
    enc_key = kwargs.get("enc_key")
    if enc_key is not None:
        from . import crypto
        with open(path, "rb") as f:
            raw = f.read()
        with open(path, "wb") as f:
            f.write(crypto.encrypt(raw, enc_key, kwargs.get("enc_mode", "AES-GCM")))
    return path


def load(file_name, **kwargs):
    """Loads a graph written by ``export`` (``dec_key`` / ``dec_mode`` for an encrypted file); wrap the result in
    ``nn.GraphCell`` to use it as a network."""
    from ..graph import mindir, mindir_proto
    dec_key = kwargs.get("dec_key")
    with open(file_name, "rb") as f:
        raw = f.read()
    if dec_key is not None:
        from . import crypto
        raw = crypto.decrypt(raw, dec_key, kwargs.get("dec_mode", "AES-GCM"))
    if raw[:8] != mindir.MAGIC and mindir_proto.looks_like_model_proto(raw):
        return mindir_proto.load_model_proto(raw)          # the reference's protobuf layout
    if dec_key is None:
        return mindir.load_mindir(file_name)
    import tempfile
    with tempfile.NamedTemporaryFile(suffix=".mindir") as tmp:
        tmp.write(raw)
        tmp.flush()
        return mindir.load_mindir(tmp.name)


def save_mindir(model, file_name):
    """Writes a loaded graph back to ``file_name`` (``.mindir`` appended when missing): a protobuf model message as
    its serialized bytes, a ``FuncGraph`` in the native container.  Parity: serialization.py (save_mindir)."""
    if not isinstance(file_name, str):
        raise TypeError("For 'save_mindir', 'file_name' must be string, but got %s" % type(file_name))
    if not file_name.endswith(".mindir"):
        file_name += ".mindir"
    folder = os.path.dirname(os.path.abspath(file_name))
    os.makedirs(folder, exist_ok=True)
    if hasattr(model, "SerializeToString"):
        with open(file_name, "wb") as f:
            f.write(model.SerializeToString())
        return
    from ..graph.ir import FuncGraph
    from ..graph.mindir import save_mindir as _save_native
    fg = model if isinstance(model, FuncGraph) else getattr(model, "fg", getattr(model, "graph", None))
    if not isinstance(fg, FuncGraph):
        raise TypeError("For 'save_mindir', 'model' must be a model protobuf message or a loaded graph, but got %s"
                        % type(model))
    _save_native(fg, file_name)


def convert_model(mindir_file, convert_file, file_format):
    """Converts a MindIR file to another format.  Only ``file_format='MINDIR'`` (a verified copy: the file is loaded
    and written again) is available; ONNX export needs a converter that this build does not ship."""
    if file_format == "ONNX":
        raise NotImplementedError("convert_model: ONNX output is not available in this build")
    if file_format != "MINDIR":
        raise ValueError("For 'convert_model', 'file_format' must be 'ONNX' or 'MINDIR', but got %r" % (file_format,))
    graph = load(mindir_file)
    with open(mindir_file, "rb") as src:
        data = src.read()
    del graph                                   # parsed only to reject files that are not loadable graphs
    with open(convert_file, "wb") as dst:
        dst.write(data)


from .safetensors_io import (check_checkpoint, ckpt_to_safetensors, get_ckpt_path_with_strategy,  # noqa: E402,F401
                             safetensors_to_ckpt)
