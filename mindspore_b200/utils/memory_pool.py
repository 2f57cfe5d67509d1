"""Best-fit dynamic memory pool (``csrc/host/mem_pool.hpp``): the host-heap form for tests and host buffers, and the
switch that makes it the device allocator of the process.

``enable_device_pool()`` installs the pool as torch's CUDA allocator (``torch.cuda.memory.CUDAPluggableAllocator``
over ``msb_cuda_pool_malloc`` / ``msb_cuda_pool_free``); it has to run before the first CUDA allocation of the
process.  Block size and limit default to the context options ``mempool_block_size`` and ``max_device_memory``
(python/mindspore/context.py: the same two keys configure the reference's DynamicMemPoolBestFit).  CUDA-graph capture
needs the allocator's own capture pools, which a pluggable allocator does not provide, so the pool and
``enable_cuda_graph`` exclude each other.
"""
from __future__ import annotations

import ctypes

from .. import _native

_U64 = ctypes.c_ulonglong
_FIELDS = ("used", "reserved", "peak_used", "peak_reserved", "blocks", "largest_idle", "idle_bufs")


def _parse_size(v, default):
    if v in (None, ""):
        return default
    if isinstance(v, (int, float)):
        return int(v)
    s = str(v).strip().upper()
    for suffix, mul in (("GB", 2 ** 30), ("MB", 2 ** 20), ("KB", 2 ** 10), ("B", 1)):
        if s.endswith(suffix):
            return int(float(s[:-len(suffix)]) * mul)
    return int(float(s))


class BestFitPool:
    """The pool over the C heap: ``alloc(size, stream=0)`` returns an address, ``free(addr)`` gives it back."""

    def __init__(self, block_size=1 << 20, max_size=0):
        lib = _native.host()
        lib.msb_pool_create.restype = ctypes.c_void_p
        lib.msb_pool_create.argtypes = [_U64, _U64]
        lib.msb_pool_alloc.restype = ctypes.c_void_p
        lib.msb_pool_alloc.argtypes = [ctypes.c_void_p, _U64, _U64]
        lib.msb_pool_free.restype = _U64
        lib.msb_pool_free.argtypes = [ctypes.c_void_p, ctypes.c_void_p]
        lib.msb_pool_destroy.argtypes = [ctypes.c_void_p]
        lib.msb_pool_mark_synchronized.argtypes = [ctypes.c_void_p]
        lib.msb_pool_release_idle.restype = _U64
        lib.msb_pool_release_idle.argtypes = [ctypes.c_void_p]
        lib.msb_pool_stats.argtypes = [ctypes.c_void_p, ctypes.POINTER(_U64)]
        self._lib = lib
        self._pool = lib.msb_pool_create(int(block_size), int(max_size))

    def alloc(self, size, stream=0):
        p = self._lib.msb_pool_alloc(self._pool, int(size), int(stream))
        if not p:
            raise MemoryError("the pool cannot serve %d bytes within its limit" % size)
        return int(p)

    def free(self, addr):
        if self._lib.msb_pool_free(self._pool, ctypes.c_void_p(addr)) == 0:
            raise ValueError("address %#x is not a live buffer of this pool" % addr)

    def mark_synchronized(self):
        self._lib.msb_pool_mark_synchronized(self._pool)

    def release_idle(self):
        return int(self._lib.msb_pool_release_idle(self._pool))

    def stats(self):
        out = (_U64 * 7)()
        self._lib.msb_pool_stats(self._pool, out)
        return dict(zip(_FIELDS, (int(x) for x in out)))

    def close(self):
        if self._pool:
            self._lib.msb_pool_destroy(self._pool)
            self._pool = None

    def __del__(self):
        try:
            self.close()
        except Exception:  # noqa: BLE001
            pass


_device_pool_on = False


def enable_device_pool(block_size=None, max_size=None):
    """Makes the best-fit pool the CUDA allocator of this process.  Call before anything allocates on the device."""
    global _device_pool_on
    import torch
    from .. import context
    if _device_pool_on:
        return
    if context.get_context("enable_cuda_graph"):
        raise RuntimeError("the best-fit device pool and enable_cuda_graph exclude each other (graph capture needs "
                           "the caching allocator's capture pools)")
    if torch.cuda.is_initialized() and torch.cuda.memory_allocated() > 0:
        raise RuntimeError("enable_device_pool() must run before the first CUDA allocation of the process")
    lib = _native.cuda()
    block = _parse_size(block_size if block_size is not None else context.get_context("mempool_block_size"), 1 << 30)
    limit = _parse_size(max_size if max_size is not None else context.get_context("max_device_memory"), 0)
    if limit >= 1 << 40:
        limit = 0                       # the context default ("1024GB") means no limit
    lib.msb_cuda_pool_configure.argtypes = [_U64, _U64]
    lib.msb_cuda_pool_configure(block, limit)
    from .._native import build as _build
    alloc = torch.cuda.memory.CUDAPluggableAllocator(_build.CUDA_LIB, "msb_cuda_pool_malloc", "msb_cuda_pool_free")
    torch.cuda.memory.change_current_allocator(alloc)
    _device_pool_on = True


def device_pool_enabled():
    return _device_pool_on


def device_pool_stats(device=None):
    import torch
    lib = _native.cuda()
    out = (_U64 * 7)()
    lib.msb_cuda_pool_stats.argtypes = [ctypes.c_int, ctypes.POINTER(_U64)]
    lib.msb_cuda_pool_stats(torch.cuda.current_device() if device is None else int(device), out)
    return dict(zip(_FIELDS, (int(x) for x in out)))


def device_pool_release_idle(device=None):
    """Synchronises the device, lets every stream reuse what is idle and returns idle blocks to the driver."""
    import torch
    lib = _native.cuda()
    dev = torch.cuda.current_device() if device is None else int(device)
    torch.cuda.synchronize(dev)
    lib.msb_cuda_pool_mark_synchronized.argtypes = [ctypes.c_int]
    lib.msb_cuda_pool_mark_synchronized(dev)
    lib.msb_cuda_pool_release_idle.restype = _U64
    lib.msb_cuda_pool_release_idle.argtypes = [ctypes.c_int]
    return int(lib.msb_cuda_pool_release_idle(dev))
