"""Host (CPU) ring collectives over TCP - the native counterpart of the reference's MCCL backend.

    comm = HostCommunicator(rank, world, ["127.0.0.1:29610", "127.0.0.1:29611"])
    comm.all_reduce(t)                       # in place, CPU tensor or numpy array (fp32/fp64/int32/int64/uint8)
    out = comm.all_gather(t)
    part = comm.reduce_scatter(t)
    comm.broadcast(t, root=0)
    comm.barrier()

The ring algorithms and the sockets are C++ (``csrc/host/host_collectives.cpp``); this module converts tensors to
pointers and picks the peers.  ``HostCommunicator.from_env()`` derives the peer list of a single-node job from
``MASTER_ADDR`` / ``MASTER_PORT`` / ``RANK`` / ``WORLD_SIZE`` (ports ``MASTER_PORT + 200 + rank``);
``from_store(client, ...)`` publishes ``host:port`` through the cluster metadata store, which is how ranks of a
multi-node job find each other (the reference exchanges the same through its scheduler:
plugin/device/cpu/hal/hardware/ms_collective_comm_lib.cc, distributed/cluster/topology/compute_graph_node.cc).

Half-precision tensors are reduced in fp32 (converted before, cast back after)."""
from __future__ import annotations

import ctypes
import os
import socket

import numpy as np
import torch

from .. import _native

_DT = {torch.float32: 0, torch.float64: 1, torch.int32: 2, torch.int64: 3, torch.uint8: 4}
_OPS = {"sum": 0, "prod": 1, "max": 2, "min": 3}
_ERR = {1: "bad argument", 2: "socket error", 3: "timed out", 4: "peer closed the connection", 5: "bad handle"}
_sig_done = False


class HostCollectiveError(RuntimeError):
    pass


def _lib():
    global _sig_done
    lib = _native.host()
    if not _sig_done:
        I, L, P, D = ctypes.c_int, ctypes.c_longlong, ctypes.c_void_p, ctypes.c_double
        lib.msb_hc_create.restype = I
        lib.msb_hc_create.argtypes = [I, I, ctypes.c_char_p, D]
        lib.msb_hc_destroy.argtypes = [I]
        lib.msb_hc_all_reduce.argtypes = [I, P, L, I, I]
        lib.msb_hc_reduce_scatter.argtypes = [I, P, P, L, I, I]
        lib.msb_hc_all_gather.argtypes = [I, P, P, L]
        lib.msb_hc_broadcast.argtypes = [I, P, L, I]
        lib.msb_hc_barrier.argtypes = [I]
        lib.msb_hc_send_next.argtypes = [I, P, L]
        lib.msb_hc_recv_prev.argtypes = [I, P, L]
        lib.msb_hc_set_timeout.argtypes = [I, D]
        _sig_done = True
    return lib


def _check(rc, what):
    if rc != 0:
        raise HostCollectiveError("%s failed: %s" % (what, _ERR.get(rc, "error %d" % rc)))


def _as_tensor(x):
    if isinstance(x, np.ndarray):
        return torch.from_numpy(x)
    if not isinstance(x, torch.Tensor):
        raise TypeError("host collectives take a CPU tensor or a numpy array, got %s" % type(x).__name__)
    if x.device.type != "cpu":
        raise ValueError("host collectives work on CPU tensors; got a tensor on %s" % x.device)
    return x


class HostCommunicator:
    def __init__(self, rank, world, peers, timeout=60.0):
        self.rank, self.world = int(rank), int(world)
        self.peers = list(peers)
        h = _lib().msb_hc_create(self.rank, self.world, ",".join(self.peers).encode(), float(timeout))
        if h <= 0:
            raise HostCollectiveError("could not build the ring (rank %d of %d): %s"
                                      % (self.rank, self.world, _ERR.get(-h, "error %d" % -h)))
        self._h = h

    # ------------------------------------------------------------------ construction helpers
    @classmethod
    def from_env(cls, timeout=60.0, port_offset=200):
        rank = int(os.environ.get("RANK", os.environ.get("RANK_ID", "0")))
        world = int(os.environ.get("WORLD_SIZE", os.environ.get("MS_WORKER_NUM", "1")))
        host = os.environ.get("MASTER_ADDR", os.environ.get("MS_SCHED_HOST", "127.0.0.1"))
        base = int(os.environ.get("MASTER_PORT", os.environ.get("MS_SCHED_PORT", "29500"))) + port_offset
        return cls(rank, world, ["%s:%d" % (host, base + r) for r in range(world)], timeout)

    @classmethod
    def from_store(cls, client, rank, world, host=None, timeout=60.0, prefix="hc"):
        """``client``: a ``communication.cluster.WorkerClient`` (put / get on the scheduler's key-value store)."""
        host = host or socket.gethostbyname(socket.gethostname())
        with socket.socket() as s:
            s.bind(("", 0))
            port = s.getsockname()[1]
        client.put("%s/%d" % (prefix, rank), "%s:%d" % (host, port))
        peers = [client.wait_for("%s/%d" % (prefix, r), timeout) for r in range(world)]
        return cls(rank, world, [p.decode() if isinstance(p, bytes) else p for p in peers], timeout)

    def close(self):
        if getattr(self, "_h", 0):
            _lib().msb_hc_destroy(self._h)
            self._h = 0

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def set_timeout(self, seconds):
        _check(_lib().msb_hc_set_timeout(self._h, float(seconds)), "set_timeout")

    # ------------------------------------------------------------------ collectives
    @staticmethod
    def _work_copy(t):
        """(contiguous tensor of a supported dtype, needs copy-back)"""
        if t.dtype in (torch.float16, torch.bfloat16):
            return t.float().contiguous(), True
        if t.dtype == torch.bool:
            return t.to(torch.uint8).contiguous(), True
        if t.dtype not in _DT:
            raise TypeError("host collectives do not support dtype %s" % t.dtype)
        return (t, False) if t.is_contiguous() else (t.contiguous(), True)

    def all_reduce(self, x, op="sum"):
        t = _as_tensor(x)
        w, copied = self._work_copy(t)
        _check(_lib().msb_hc_all_reduce(self._h, w.data_ptr(), w.numel(), _DT[w.dtype], _OPS[op]), "all_reduce")
        if copied:
            t.copy_(w.to(t.dtype))
        return x

    def reduce_scatter(self, x, op="sum"):
        t = _as_tensor(x)
        if t.shape[0] % self.world:
            raise ValueError("reduce_scatter: dim 0 (%d) is not divisible by the group size %d"
                             % (t.shape[0], self.world))
        w, _ = self._work_copy(t)
        out = torch.empty((t.shape[0] // self.world,) + tuple(t.shape[1:]), dtype=w.dtype)
        _check(_lib().msb_hc_reduce_scatter(self._h, w.data_ptr(), out.data_ptr(), out.numel(), _DT[w.dtype],
                                            _OPS[op]), "reduce_scatter")
        return out.to(t.dtype)

    def all_gather(self, x):
        t = _as_tensor(x).contiguous()
        out = torch.empty((self.world * t.shape[0],) + tuple(t.shape[1:]), dtype=t.dtype)
        _check(_lib().msb_hc_all_gather(self._h, t.data_ptr(), out.data_ptr(), t.numel() * t.element_size()),
               "all_gather")
        return out

    def broadcast(self, x, root=0):
        t = _as_tensor(x)
        w = t if t.is_contiguous() else t.contiguous()
        _check(_lib().msb_hc_broadcast(self._h, w.data_ptr(), w.numel() * w.element_size(), int(root)), "broadcast")
        if w is not t:
            t.copy_(w)
        return x

    def barrier(self):
        _check(_lib().msb_hc_barrier(self._h), "barrier")

    def send_next(self, x):
        t = _as_tensor(x).contiguous()
        _check(_lib().msb_hc_send_next(self._h, t.data_ptr(), t.numel() * t.element_size()), "send_next")

    def recv_prev(self, x):
        t = _as_tensor(x)
        if not t.is_contiguous():
            raise ValueError("recv_prev needs a contiguous destination")
        _check(_lib().msb_hc_recv_prev(self._h, t.data_ptr(), t.numel() * t.element_size()), "recv_prev")
        return x
