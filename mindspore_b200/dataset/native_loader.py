"""``NativeBatchLoader``: shuffle / shard / (image transform) / batch of in-memory columns on C++ worker threads.

    loader = NativeBatchLoader({"image": images_u8, "label": labels}, batch_size=256, shuffle=True,
                               num_parallel_workers=8, pin_memory=True)
    loader.set_image_transform("image", out_size=(224, 224), flip=True, mean=[...], std=[...])
    for epoch in range(E):
        for batch in loader.epoch(epoch):            # dict of CPU tensors that view the (pinned) slot
            x = batch["image"].cuda(non_blocking=True)
            ...

The batches of an epoch come back in order; a batch's buffers are handed back to the workers when the next batch
is requested (or explicitly with ``batch.release()`` after the host->device copy has been enqueued and an event
recorded).  The work itself is ``csrc/host/data_pipeline.cpp``; see there for the mapping to the reference's C++
dataset ops.  ``Dataset.batch`` pipelines built from ``NumpySlicesDataset`` can be converted with
``NativeBatchLoader.from_numpy_slices``."""
from __future__ import annotations

import ctypes

import numpy as np
import torch

from .. import _native

_sig_done = False


def _lib():
    global _sig_done
    lib = _native.host()
    if not _sig_done:
        I, L, P, D = ctypes.c_int, ctypes.c_longlong, ctypes.c_void_p, ctypes.c_double
        PP = ctypes.POINTER(P)
        lib.msb_dp_create.restype = I
        lib.msb_dp_create.argtypes = [I, PP, ctypes.POINTER(L), L, I, I, I, ctypes.c_ulonglong, I, I, I, I, PP]
        lib.msb_dp_set_image_transform.argtypes = [I, I, I, I, I, I, I, I, ctypes.POINTER(ctypes.c_float),
                                                   ctypes.POINTER(ctypes.c_float)]
        lib.msb_dp_start_epoch.restype = L
        lib.msb_dp_start_epoch.argtypes = [I, L]
        lib.msb_dp_next.restype = I
        lib.msb_dp_next.argtypes = [I, PP, ctypes.POINTER(I), D]
        lib.msb_dp_release.argtypes = [I, I]
        lib.msb_dp_destroy.argtypes = [I]
        _sig_done = True
    return lib


class Batch(dict):
    """Dict of column tensors; ``release()`` gives the underlying slot back to the loader."""

    def __init__(self, loader, slot, items):
        super().__init__(items)
        self._loader, self._slot = loader, slot

    def release(self):
        if self._slot is not None:
            _lib().msb_dp_release(self._loader._h, self._slot)
            self._slot = None


class NativeBatchLoader:
    def __init__(self, columns, batch_size, shuffle=False, drop_remainder=True, seed=0, num_shards=1, shard_id=0,
                 num_parallel_workers=4, prefetch=4, pin_memory=False, timeout=600.0):
        if not columns:
            raise ValueError("NativeBatchLoader needs at least one column")
        self.names = list(columns)
        self._src = []
        n = None
        for k in self.names:
            a = columns[k]
            a = a.numpy() if isinstance(a, torch.Tensor) else np.asarray(a)
            a = np.ascontiguousarray(a)
            if n is None:
                n = a.shape[0]
            elif a.shape[0] != n:
                raise ValueError("column %r has %d rows, expected %d" % (k, a.shape[0], n))
            self._src.append(a)
        self.num_rows, self.batch_size = int(n), int(batch_size)
        self.pin_memory = bool(pin_memory) and torch.cuda.is_available()
        self.timeout = float(timeout)
        self._slots = max(2, int(prefetch))
        self._row_shape = [a.shape[1:] for a in self._src]
        self._dtype = [torch.from_numpy(a[:0]).dtype for a in self._src]
        self._cfg = (bool(shuffle), bool(drop_remainder), int(seed), int(num_shards), int(shard_id),
                     max(1, int(num_parallel_workers)))
        self._transforms = {}
        self._h = 0
        self._pending = None

    @classmethod
    def from_numpy_slices(cls, data, column_names=None, **kw):
        if isinstance(data, dict):
            return cls(data, **kw)
        if not isinstance(data, (tuple, list)):
            data = (data,)
        names = column_names or ["column_%d" % i for i in range(len(data))]
        return cls(dict(zip(names, data)), **kw)

    def set_image_transform(self, column, out_size, flip=True, mean=None, std=None):
        """uint8 [H, W, C] rows of ``column`` become float32 [C, out_h, out_w]: random crop, optional random
        horizontal flip, per-channel normalisation."""
        if self._h:
            raise RuntimeError("set_image_transform must be called before the first epoch")
        i = self.names.index(column)
        a = self._src[i]
        if a.dtype != np.uint8 or a.ndim != 4:
            raise ValueError("image transform needs a uint8 [N, H, W, C] column")
        oh, ow = out_size
        c = a.shape[3]
        self._transforms[i] = (a.shape[1], a.shape[2], c, int(oh), int(ow), bool(flip),
                               list(mean) if mean is not None else [0.0] * c,
                               list(std) if std is not None else [1.0] * c)
        self._row_shape[i] = (c, int(oh), int(ow))
        self._dtype[i] = torch.float32

    # ------------------------------------------------------------------ lifecycle
    def _build(self):
        lib = _lib()
        nc = len(self._src)
        P = ctypes.c_void_p
        col_ptrs = (P * nc)(*[a.ctypes.data for a in self._src])
        row_bytes = (ctypes.c_longlong * nc)(*[int(a.strides[0]) if a.shape[0] else 0 for a in self._src])
        self._bufs = []
        for s in range(self._slots):
            row = []
            for i in range(nc):
                t = torch.empty((self.batch_size,) + tuple(self._row_shape[i]), dtype=self._dtype[i],
                                pin_memory=self.pin_memory)
                row.append(t)
            self._bufs.append(row)
        out_ptrs = (P * (self._slots * nc))(*[t.data_ptr() for row in self._bufs for t in row])
        shuffle, drop, seed, shards, shard_id, workers = self._cfg
        h = lib.msb_dp_create(nc, col_ptrs, row_bytes, self.num_rows, self.batch_size, int(drop), int(shuffle),
                              seed, shards, shard_id, workers, self._slots, out_ptrs)
        if h <= 0:
            raise ValueError("could not create the native pipeline (bad argument)")
        self._h = h
        for i, (ih, iw, c, oh, ow, flip, mean, std) in self._transforms.items():
            fm = (ctypes.c_float * c)(*mean)
            fs = (ctypes.c_float * c)(*std)
            rc = lib.msb_dp_set_image_transform(h, i, ih, iw, c, oh, ow, int(flip), fm, fs)
            if rc:
                raise ValueError("image transform rejected for column %r" % self.names[i])

    def get_dataset_size(self):
        shuffle, drop, seed, shards, shard_id, _ = self._cfg
        n = len(range(shard_id, self.num_rows, shards))
        return n // self.batch_size if drop else (n + self.batch_size - 1) // self.batch_size

    def epoch(self, epoch=0):
        if not self._h:
            self._build()
        lib = _lib()
        if self._pending is not None:
            self._pending.release()
            self._pending = None
        nb = lib.msb_dp_start_epoch(self._h, int(epoch))
        if nb < 0:
            raise RuntimeError("start_epoch failed")
        nc = len(self.names)
        ptrs = (ctypes.c_void_p * nc)()
        rows = ctypes.c_int(0)
        for _ in range(nb):
            if self._pending is not None:
                self._pending.release()
                self._pending = None
            slot = lib.msb_dp_next(self._h, ptrs, ctypes.byref(rows), self.timeout)
            if slot == -1:
                return
            if slot < 0:
                raise RuntimeError("native data pipeline: %s" % ("timed out" if slot == -2 else "bad handle"))
            items = [(self.names[i], self._bufs[slot][i][:rows.value]) for i in range(nc)]
            self._pending = Batch(self, slot, items)
            yield self._pending

    def __iter__(self):
        return self.epoch(0)

    def close(self):
        if self._h:
            _lib().msb_dp_destroy(self._h)
            self._h = 0

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
