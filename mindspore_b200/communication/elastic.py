"""Communicator (re)initialisation through the cluster scheduler: what lets a job re-form after a rank was lost.

The scheduler (``communication.cluster.Scheduler``, run by the launcher, not by a worker) holds a *generation*
counter of the job's communicators.  Every (re)start of the collective layer is a rendezvous for one generation:

* rank 0 opens a fresh TCP store on a free port and publishes ``comm/<generation>/master`` in the scheduler's
  metadata store; the others wait for that key - no fixed MASTER_PORT is reused, so a store left behind by a dead
  process never gets in the way;
* the process group is created in a watchdog thread: if it does not come up within the timeout the caller gets a
  ``CommInitTimeout`` instead of a hung process (reference: distributed/collective/collective_manager.cc:80-118);
* a worker that registers and finds that its node already took part in the current generation knows it is a
  *restart*: it raises the generation.  Survivors notice - between steps, through ``need_reinit()`` (a changed
  generation, or the heartbeat reporting a lost node), or because their next collective ended with an error under a
  short process-group timeout - and call ``reinit()``: groups are destroyed, the new generation is joined, named
  groups are re-created (reference: collective_manager.cc:120-146,278-358, ``need_reinit``).

``agree_on_checkpoint`` then makes all ranks pick the newest checkpoint that EVERY rank has, by all-gathering the
(epoch, step) lists over the fresh communicator - no shared file system is assumed (reference:
distributed/recovery/recovery_context.cc:137-323, ObtainGlobalLatestCkptInfo).
"""
from __future__ import annotations

import datetime
import os
import threading
import time

import torch
import torch.distributed as dist

from . import management as M
from .cluster import ClusterError


class CommInitTimeout(RuntimeError):
    pass


def run_with_watchdog(fn, timeout_s, what):
    """Runs ``fn`` in a helper thread and gives up after ``timeout_s``: the caller gets an exception, the helper is
    left behind as a daemon thread (it holds no lock the caller needs)."""
    box = {}

    def target():
        try:
            box["value"] = fn()
        except BaseException as e:  # noqa: BLE001
            box["error"] = e

    th = threading.Thread(target=target, name="msb-comm-init", daemon=True)
    th.start()
    th.join(timeout_s)
    if th.is_alive():
        raise CommInitTimeout("%s did not finish within %.1f s" % (what, timeout_s))
    if "error" in box:
        raise box["error"]
    return box.get("value")


class ElasticComm:
    def __init__(self, worker, backend="gloo", host="127.0.0.1", init_timeout_s=60.0, op_timeout_s=30.0):
        self.worker, self.backend, self.host = worker, backend, host
        self.init_timeout_s, self.op_timeout_s = init_timeout_s, op_timeout_s
        self.generation = None
        self.store = None
        self.named_groups = {}          # name -> ranks, re-created after every reinit

    # ------------------------------------------------------------------ rendezvous
    def _join_key(self, gen):
        return "comm/%d/joined/%s" % (gen, self.worker.node_id.decode())

    def start(self):
        """First initialisation of this process.  A restarted process (its node already joined the current
        generation) opens the next generation."""
        w = self.worker
        if w.rank is None:
            w.register()
        gen = w.add("comm/generation", 0)
        if w.get(self._join_key(gen)) is not None:
            gen = w.add("comm/generation", 1)
        self._rendezvous(gen)
        return self

    def need_reinit(self):
        """True when the job's communicators are stale: another generation was opened, or a node is reported
        lost by the scheduler's heartbeat monitor."""
        try:
            return self.worker.add("comm/generation", 0) != self.generation or self.worker.abnormal > 0
        except ClusterError:
            return True

    def wait_for_new_generation(self, timeout_s=60.0):
        deadline = time.time() + timeout_s
        while time.time() < deadline:
            g = self.worker.add("comm/generation", 0)
            if g != self.generation:
                return g
            time.sleep(0.05)
        raise ClusterError("no new communicator generation was opened within %.1f s" % timeout_s)

    def reinit(self, timeout_s=60.0):
        """Leaves the current communicators and joins the newest generation (waiting for a restarted rank to open
        it).  Collective on the surviving + restarted ranks."""
        gen = self.wait_for_new_generation(timeout_s)
        self._teardown()
        self._rendezvous(gen)
        for name, ranks in list(self.named_groups.items()):
            M.create_group(name, ranks)

    def _teardown(self):
        if dist.is_initialized():
            try:
                dist.destroy_process_group()
            except Exception:  # noqa: BLE001  (a communicator with a dead peer may refuse a clean shutdown)
                pass
        M._state.groups.clear()
        M.GlobalComm.INITED = False
        self.store = None

    def _rendezvous(self, gen):
        w = self.worker
        rank, world = w.rank, w.world
        key = "comm/%d/master" % gen
        if rank == 0:
            store = dist.TCPStore(self.host, 0, world, is_master=True,
                                  timeout=datetime.timedelta(seconds=self.init_timeout_s), wait_for_workers=False)
            w.put(key, ("%s:%d" % (self.host, store.port)).encode())
        else:
            host, port = w.wait_for(key, self.init_timeout_s).decode().rsplit(":", 1)
            store = run_with_watchdog(
                lambda: dist.TCPStore(host, int(port), world, is_master=False,
                                      timeout=datetime.timedelta(seconds=self.init_timeout_s)),
                self.init_timeout_s, "connecting to the rendezvous store of generation %d" % gen)
        torch_backend = "nccl" if self.backend == "nccl" else "gloo"
        kw = {}
        if torch_backend == "nccl":
            kw["device_id"] = torch.device("cuda", torch.cuda.current_device())
        run_with_watchdog(
            lambda: dist.init_process_group(torch_backend, store=store, rank=rank, world_size=world,
                                            timeout=datetime.timedelta(seconds=self.op_timeout_s), **kw),
            self.init_timeout_s, "creating the world group of generation %d" % gen)
        self.store, self.generation = store, gen
        world_name = M.NCCL_WORLD_COMM_GROUP if self.backend == "nccl" else M.MCCL_WORLD_COMM_GROUP
        M._state.rank, M._state.world, M._state.local_rank = rank, world, rank
        M._state.simulation = False
        M._state.groups[world_name] = M._Group(world_name, range(world), dist.group.WORLD)
        M.GlobalComm.BACKEND = "nccl" if self.backend == "nccl" else "mccl"
        M.GlobalComm.WORLD_COMM_GROUP = world_name
        M.GlobalComm.INITED = True
        w.put(self._join_key(gen), b"1")

    def create_group(self, name, ranks):
        self.named_groups[name] = list(ranks)
        M.create_group(name, ranks)


def agree_on_checkpoint(local_records, device=None):
    """``local_records``: this rank's checkpoints as [(epoch, step), ...].  Returns the newest (epoch, step) present
    on EVERY rank, or None - an all-gather of fixed-size lists, no file is read across ranks."""
    cap = 64
    recs = sorted(set((int(e), int(s)) for e, s in local_records))[-cap:]
    t = torch.full((cap, 2), -1, dtype=torch.int64, device=device or "cpu")
    for i, (e, s) in enumerate(recs):
        t[i, 0], t[i, 1] = e, s
    world = dist.get_world_size()
    out = [torch.empty_like(t) for _ in range(world)]
    dist.all_gather(out, t)
    common = None
    for o in out:
        have = {(int(e), int(s)) for e, s in o.tolist() if e >= 0}
        common = have if common is None else (common & have)
    return max(common) if common else None
