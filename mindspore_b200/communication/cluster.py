"""Cluster bootstrap on top of the native scheduler / worker library (``csrc/host/cluster.cpp``).

``Scheduler`` is the metadata server (role ``MS_SCHED``): workers register under a node id and get a rank, send
heartbeats, and share small values through a key-value store.  ``WorkerClient`` is the worker side; its heartbeat
thread learns from every reply how many nodes the scheduler considers lost, and ``check_health`` turns that into an
exception on the host *before* the next collective is launched - no device ever waits on a dead peer.

Parity: ccsrc/distributed/cluster/cluster_context.cc (roles from MS_ROLE, MS_SCHED_HOST/PORT, MS_WORKER_NUM,
MS_NODE_ID), topology/meta_server_node.cc:149-343 (register / heartbeat / metadata), :454-527 (node timeout),
compute_graph_node.cc:158-319 (heartbeat loop and abnormal-node handling)."""
from __future__ import annotations

import ctypes
import os
import threading
import time

from .. import _native


class ClusterError(RuntimeError):
    pass


_sig_done = False


def _lib():
    global _sig_done
    lib = _native.host()
    if not _sig_done:
        c_int, c_dbl, c_str = ctypes.c_int, ctypes.c_double, ctypes.c_char_p
        lib.msb_sched_start.restype = c_int
        lib.msb_sched_start.argtypes = [c_int, c_int, c_dbl]
        lib.msb_sched_stop.restype = None
        lib.msb_sched_abnormal_nodes.restype = c_int
        lib.msb_sched_registered.restype = c_int
        lib.msb_worker_register.restype = c_int
        lib.msb_worker_register.argtypes = [c_str, c_int, c_str, ctypes.POINTER(c_int), c_dbl]
        lib.msb_worker_heartbeat.restype = c_int
        lib.msb_worker_heartbeat.argtypes = [c_str, c_int, c_str, ctypes.POINTER(c_int), c_dbl]
        lib.msb_worker_unregister.restype = c_int
        lib.msb_worker_unregister.argtypes = [c_str, c_int, c_str, c_dbl]
        lib.msb_store_put.restype = c_int
        lib.msb_store_put.argtypes = [c_str, c_int, c_str, c_str, c_int, c_dbl]
        lib.msb_store_get.restype = c_int
        lib.msb_store_get.argtypes = [c_str, c_int, c_str, ctypes.c_char_p, c_int, c_dbl]
        lib.msb_store_delete.restype = c_int
        lib.msb_store_delete.argtypes = [c_str, c_int, c_str, c_dbl]
        lib.msb_store_add.restype = ctypes.c_longlong
        lib.msb_store_add.argtypes = [c_str, c_int, c_str, ctypes.c_longlong, c_dbl]
        lib.msb_sched_snapshot.restype = c_int
        lib.msb_sched_snapshot.argtypes = [ctypes.c_char_p, c_int]
        lib.msb_sched_restore.restype = c_int
        lib.msb_sched_restore.argtypes = [ctypes.c_char_p, c_int]
        _sig_done = True
    return lib


class Scheduler:
    """The metadata server of one job (one per process).  ``port=0`` picks a free port."""

    def __init__(self, port=0, expected_workers=1, node_timeout_s=30.0, persist_path=None, persist_interval_s=1.0):
        """``persist_path``: file the scheduler's state (node -> rank table and the metadata store) is written to
        every ``persist_interval_s`` seconds and on ``stop``; a scheduler started with an existing file continues
        from it, so a restarted scheduler hands every node its old rank and still knows the job's metadata
        (reference: cluster/topology/meta_server_node.cc:561-635, MS_ENABLE_RECOVERY / MS_RECOVERY_PATH)."""
        self.port = _lib().msb_sched_start(int(port), int(expected_workers), float(node_timeout_s))
        if self.port <= 0:
            raise ClusterError("scheduler could not listen on port %s (already running in this process?)" % port)
        self.expected = expected_workers
        self.persist_path = persist_path
        self._persist_stop = threading.Event()
        self._persist_thread = None
        if persist_path:
            if os.path.isfile(persist_path):
                with open(persist_path, "rb") as f:
                    data = f.read()
                self.restored = _lib().msb_sched_restore(data, len(data))
            else:
                self.restored = 0

            def loop():
                while not self._persist_stop.wait(persist_interval_s):
                    self.persist()
            self._persist_thread = threading.Thread(target=loop, name="msb-sched-persist", daemon=True)
            self._persist_thread.start()

    def snapshot(self):
        cap = 1 << 16
        while True:
            buf = ctypes.create_string_buffer(cap)
            n = _lib().msb_sched_snapshot(buf, cap)
            if n >= 0:
                return buf.raw[:n]
            cap = -n + 1024

    def persist(self):
        if not self.persist_path:
            return
        tmp = self.persist_path + ".tmp"
        with open(tmp, "wb") as f:
            f.write(self.snapshot())
        os.replace(tmp, self.persist_path)

    def registered(self):
        return _lib().msb_sched_registered()

    def abnormal_nodes(self):
        return _lib().msb_sched_abnormal_nodes()

    def wait_registered(self, timeout_s):
        deadline = time.time() + timeout_s
        while time.time() < deadline:
            if self.registered() >= self.expected:
                return True
            time.sleep(0.05)
        return False

    def stop(self):
        self._persist_stop.set()
        if self._persist_thread is not None:
            self._persist_thread.join(5)
            self._persist_thread = None
        self.persist()
        _lib().msb_sched_stop()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.stop()


class WorkerClient:
    """Worker side: registration, heartbeat thread, metadata store."""

    def __init__(self, host, port, node_id, timeout_s=5.0):
        self.host, self.port, self.node_id = host.encode(), int(port), str(node_id).encode()
        self.timeout_s = timeout_s
        self.rank = self.world = None
        self.abnormal = 0
        self.ready = False
        self.scheduler_lost = False
        self._stop = threading.Event()
        self._thread = None
        self._missed = 0

    def register(self, retry_s=30.0):
        world = ctypes.c_int(0)
        deadline = time.time() + retry_s
        while True:
            rank = _lib().msb_worker_register(self.host, self.port, self.node_id, ctypes.byref(world), self.timeout_s)
            if rank >= 0:
                self.rank, self.world = rank, world.value
                return rank
            if time.time() > deadline:
                raise ClusterError("node %s could not register with the scheduler at %s:%d"
                                   % (self.node_id.decode(), self.host.decode(), self.port))
            time.sleep(0.2)

    def heartbeat(self):
        """One heartbeat; returns the scheduler's count of abnormal nodes (or -1 if it did not answer)."""
        ready = ctypes.c_int(0)
        n = _lib().msb_worker_heartbeat(self.host, self.port, self.node_id, ctypes.byref(ready), self.timeout_s)
        if n < 0:
            self._missed += 1
            if self._missed >= 3:
                self.scheduler_lost = True
            return -1
        self._missed = 0
        self.abnormal, self.ready = n, bool(ready.value)
        return n

    def start_heartbeat(self, interval_s=1.0):
        if self._thread is not None:
            return

        def loop():
            while not self._stop.wait(interval_s):
                self.heartbeat()

        self._thread = threading.Thread(target=loop, name="msb-heartbeat", daemon=True)
        self._thread.start()

    def stop_heartbeat(self):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(5)
            self._thread = None

    def check_health(self):
        """Raises ``ClusterError`` when the scheduler has lost a node (or this worker has lost the scheduler)."""
        if self.abnormal > 0:
            raise ClusterError("%d node(s) of the cluster stopped sending heartbeats" % self.abnormal)
        if self.scheduler_lost:
            raise ClusterError("the scheduler does not answer heartbeats")

    def unregister(self):
        self.stop_heartbeat()
        _lib().msb_worker_unregister(self.host, self.port, self.node_id, self.timeout_s)

    # ------------------------------------------------------------------ metadata store
    def put(self, key, value: bytes):
        if isinstance(value, str):
            value = value.encode()
        rc = _lib().msb_store_put(self.host, self.port, key.encode(), value, len(value), self.timeout_s)
        if rc != 0:
            raise ClusterError("store put(%s) failed" % key)

    def get(self, key, capacity=1 << 20):
        buf = ctypes.create_string_buffer(capacity)
        n = _lib().msb_store_get(self.host, self.port, key.encode(), buf, capacity, self.timeout_s)
        if n == -2:
            return None
        if n < 0:
            raise ClusterError("store get(%s) failed" % key)
        return buf.raw[:n]

    def wait_for(self, key, timeout_s=30.0):
        deadline = time.time() + timeout_s
        while time.time() < deadline:
            v = self.get(key)
            if v is not None:
                return v
            time.sleep(0.05)
        raise ClusterError("key %s did not appear within %.1f s" % (key, timeout_s))

    def delete(self, key):
        _lib().msb_store_delete(self.host, self.port, key.encode(), self.timeout_s)

    def add(self, key, delta=0):
        """Atomic counter in the metadata store: adds ``delta`` and returns the new value (``delta=0`` reads)."""
        v = _lib().msb_store_add(self.host, self.port, key.encode(), int(delta), self.timeout_s)
        if v < 0:
            raise ClusterError("store add(%s) failed" % key)
        return int(v)


_worker = None


def worker_from_env(start_heartbeat=True):
    """The process-wide ``WorkerClient`` described by MS_SCHED_HOST / MS_SCHED_PORT / MS_NODE_ID, or None when the
    process was not started under a scheduler."""
    global _worker
    if _worker is not None:
        return _worker
    host, port = os.environ.get("MS_SCHED_HOST"), os.environ.get("MS_SCHED_PORT")
    if not host or not port or os.environ.get("MS_ROLE", "MS_WORKER") != "MS_WORKER" \
            or os.environ.get("MSB_CLUSTER_PORT") is None:
        return None
    node = os.environ.get("MS_NODE_ID", os.environ.get("RANK", "0"))
    w = WorkerClient(host, int(os.environ["MSB_CLUSTER_PORT"]), node)
    w.register(float(os.environ.get("MS_CLUSTER_TIMEOUT", "600")))
    if start_heartbeat:
        w.start_heartbeat(float(os.environ.get("MSB_HEARTBEAT_INTERVAL", "1.0")))
    _worker = w
    return w


def check_cluster_health():
    """Host-side check to run between steps: raises when a peer is gone."""
    if _worker is not None:
        _worker.check_health()
