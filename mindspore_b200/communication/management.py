"""Collective communication bootstrap and the group registry.

``init()`` brings up one process per device: NCCL over NVLink for GPU ranks, gloo for CPU ranks, or the
dummy backend when ``MS_SIMULATION_LEVEL`` is set (compile / run one rank of a large virtual cluster on a
single device, reference: ccsrc/distributed/collective/collective_manager.cc:168-175).  Rendezvous reads
either torchrun's variables (RANK, WORLD_SIZE, MASTER_ADDR, MASTER_PORT) or msrun's
(MS_WORKER_NUM, MS_SCHED_HOST, MS_SCHED_PORT, MS_NODE_ID / RANK_ID).

Parity: mindspore/python/mindspore/communication/management.py:108-206 (init), :239 (get_rank), :283
(get_local_rank), :332 (get_group_size), :534 (create_group), :584 (destroy_group);
communication/_comm_helper.py:58-123 (world group names, GlobalComm).
"""
from __future__ import annotations

import datetime
import os
import threading

import torch
import torch.distributed as dist

from .. import context
from ..utils.log import logger

HCCL_WORLD_COMM_GROUP = "hccl_world_group"
NCCL_WORLD_COMM_GROUP = "nccl_world_group"
MCCL_WORLD_COMM_GROUP = "mccl_world_group"


class GlobalComm:
    BACKEND = None
    WORLD_COMM_GROUP = NCCL_WORLD_COMM_GROUP
    INITED = False
    CHECK_ENVS = True


class _Group:
    def __init__(self, name, ranks, pg):
        self.name, self.ranks, self.pg = name, list(ranks), pg

    @property
    def size(self):
        return len(self.ranks)


class _State:
    def __init__(self):
        self.groups = {}
        self.rank = 0
        self.world = 1
        self.local_rank = 0
        self.simulation = False
        self.lock = threading.Lock()


_state = _State()


def _simulation_level():
    v = os.environ.get("MS_SIMULATION_LEVEL", "")
    return int(v) if v != "" else None


def is_simulation():
    return _state.simulation


def _env_int(*names, default=None):
    for n in names:
        v = os.environ.get(n)
        if v not in (None, ""):
            return int(v)
    return default


def init(backend_name=None):
    """Initialises the world group.  Safe to call twice."""
    if GlobalComm.INITED:
        return
    target = context.get_context("device_target")
    if backend_name is None:
        backend_name = "nccl" if target == "GPU" else "mccl"
    if backend_name not in ("nccl", "mccl", "hccl", "gloo"):
        raise ValueError("For 'init', the argument 'backend_name' must be one of 'nccl', 'mccl', 'hccl', "
                         "but got %r" % (backend_name,))
    if backend_name == "hccl":
        raise RuntimeError("backend 'hccl' needs Ascend devices, which this build does not drive")
    if backend_name == "nccl" and target != "GPU":
        raise RuntimeError("For 'init', backend 'nccl' needs device_target GPU, but it is %s" % target)
    sim = _simulation_level()
    world_name = {"nccl": NCCL_WORLD_COMM_GROUP, "mccl": MCCL_WORLD_COMM_GROUP, "gloo": MCCL_WORLD_COMM_GROUP}[backend_name]
    if sim is not None:
        _state.simulation = True
        _state.rank = _env_int("RANK_ID", "RANK", default=0)
        _state.world = _env_int("RANK_SIZE", "WORLD_SIZE", default=1)
        _state.local_rank = _state.rank % max(1, torch.cuda.device_count() or 8)
        _state.groups[world_name] = _Group(world_name, range(_state.world), None)
        logger.warning("MS_SIMULATION_LEVEL=%d: dummy collectives, rank %d of %d", sim, _state.rank, _state.world)
    else:
        world = _env_int("WORLD_SIZE", "MS_WORKER_NUM", "RANK_SIZE", default=1)
        rank = _env_int("RANK", "MS_NODE_ID", "RANK_ID", default=0)
        local_rank = _env_int("LOCAL_RANK", "DEVICE_ID", default=rank)
        os.environ.setdefault("MASTER_ADDR", os.environ.get("MS_SCHED_HOST", "127.0.0.1"))
        os.environ.setdefault("MASTER_PORT", os.environ.get("MS_SCHED_PORT", "29500"))
        os.environ.setdefault("RANK", str(rank))
        os.environ.setdefault("WORLD_SIZE", str(world))
        torch_backend = "nccl" if backend_name == "nccl" else "gloo"
        if torch_backend == "nccl":
            torch.cuda.set_device(local_rank % torch.cuda.device_count())
        if not dist.is_initialized():
            timeout = datetime.timedelta(seconds=int(os.environ.get("MS_CLUSTER_TIMEOUT", "600")))
            kw = {}
            if torch_backend == "nccl":
                kw["device_id"] = torch.device("cuda", torch.cuda.current_device())
            # the rendezvous runs under a watchdog: ranks that never arrive end this call with an error after
            # MS_CLUSTER_TIMEOUT instead of leaving the process blocked (collective_manager.cc:80-118)
            from .elastic import run_with_watchdog
            run_with_watchdog(lambda: dist.init_process_group(torch_backend, rank=rank, world_size=world,
                                                              timeout=timeout, **kw),
                              timeout.total_seconds() + 30, "init_process_group(%s)" % torch_backend)
        _state.rank, _state.world, _state.local_rank = dist.get_rank(), dist.get_world_size(), local_rank
        _state.groups[world_name] = _Group(world_name, range(_state.world), dist.group.WORLD)
    GlobalComm.BACKEND = backend_name
    GlobalComm.WORLD_COMM_GROUP = world_name
    GlobalComm.INITED = True
    if sim is None:
        from . import cluster
        cluster.worker_from_env()      # registers with the scheduler and starts heartbeats when launched by msrun
    os.environ["RANK_ID"] = str(_state.rank)
    os.environ["RANK_SIZE"] = str(_state.world)


def release():
    from . import cluster
    if cluster._worker is not None:
        cluster._worker.unregister()
        cluster._worker = None
    if GlobalComm.INITED and not _state.simulation and dist.is_initialized():
        dist.destroy_process_group()
    _state.groups.clear()
    _state.simulation = False
    _state.rank, _state.world = 0, 1
    GlobalComm.INITED = False
    GlobalComm.BACKEND = None


def _check_inited():
    if not GlobalComm.INITED:
        raise RuntimeError("Distributed communication has not been initialized: call "
                           "mindspore_b200.communication.init() first")


def _group(name=None):
    _check_inited()
    name = name or GlobalComm.WORLD_COMM_GROUP
    if isinstance(name, _Group):
        return name
    g = _state.groups.get(name)
    if g is None:
        raise ValueError("The communication group %r does not exist; create it with create_group()" % (name,))
    return g


def get_rank(group=None):
    g = _group(group)
    if g.name == GlobalComm.WORLD_COMM_GROUP:
        return _state.rank
    if _state.rank not in g.ranks:
        raise ValueError("rank %d is not a member of group %s" % (_state.rank, g.name))
    return g.ranks.index(_state.rank)


def get_local_rank(group=None):
    _group(group)
    return _state.local_rank


def get_group_size(group=None):
    return _group(group).size


def get_local_rank_size(group=None):
    _group(group)
    return _env_int("LOCAL_WORLD_SIZE", default=min(_state.world, max(1, torch.cuda.device_count() or _state.world)))


def get_world_rank_from_group_rank(group, group_rank_id):
    g = _group(group)
    if not isinstance(group_rank_id, int) or group_rank_id < 0 or group_rank_id >= g.size:
        raise ValueError("group_rank_id %r is out of range for group %s" % (group_rank_id, g.name))
    return g.ranks[group_rank_id]


def get_group_rank_from_world_rank(world_rank_id, group):
    g = _group(group)
    if world_rank_id not in g.ranks:
        raise ValueError("world rank %r is not in group %s" % (world_rank_id, g.name))
    return g.ranks.index(world_rank_id)


def get_process_group_ranks(group=None):
    return list(_group(group).ranks)


def create_group(group, rank_ids):
    """Registers a named group.  Its members must call it with the same arguments; ranks outside it may call it too
    or not at all (groups are often made lazily by the ranks that need them: the model-parallel group of one pipeline
    stage, a ring of one data-parallel slice).  That is why the process group is created with local synchronisation:
    torch then derives the group's rendezvous prefix from its ranks, so two disjoint groups made at the same moment
    by different ranks do not meet under one counter-based name."""
    _check_inited()
    if not isinstance(group, str):
        raise TypeError("For 'create_group', the argument 'group' must be type of string")
    if not isinstance(rank_ids, (list, tuple)) or len(rank_ids) < 1 or len(set(rank_ids)) != len(rank_ids):
        raise ValueError("For 'create_group', 'rank_ids' must be a non-empty list without duplicates, got %r"
                         % (rank_ids,))
    if group in (HCCL_WORLD_COMM_GROUP, NCCL_WORLD_COMM_GROUP, MCCL_WORLD_COMM_GROUP):
        raise ValueError("The group name %r is reserved for the world group" % group)
    rank_ids = sorted(int(r) for r in rank_ids)
    if any(r < 0 or r >= _state.world for r in rank_ids):
        raise ValueError("rank_ids %r out of range for world size %d" % (rank_ids, _state.world))
    with _state.lock:
        if group in _state.groups:
            if _state.groups[group].ranks != rank_ids:
                raise ValueError("group %r already exists with different ranks" % group)
            return
        pg = None
        if not _state.simulation:
            if len(rank_ids) == _state.world:
                pg = dist.group.WORLD
            elif _state.rank in rank_ids:
                pg = dist.new_group(rank_ids, use_local_synchronization=True)
            else:
                pg = None                      # not a member: nothing to create, the name is only recorded
        _state.groups[group] = _Group(group, rank_ids, pg)


def destroy_group(group):
    _check_inited()
    if group == GlobalComm.WORLD_COMM_GROUP:
        raise ValueError("The world group can not be destroyed")
    g = _state.groups.pop(group, None)
    if g is None:
        raise ValueError("group %r does not exist" % group)
    if g.pg is not None and g.pg is not dist.group.WORLD and not _state.simulation:
        try:
            dist.destroy_process_group(g.pg)
        except Exception:  # group may be shared by another name
            pass


def group_exists(name):
    return name in _state.groups


def stage_rank_list_name(ranks):
    """Deterministic group name every member derives alone: "<n>-<hash of sorted ranks>"
    (reference: frontend/parallel/device_manager.cc:403-423)."""
    ranks = sorted(ranks)
    h = 1469598103934665603
    for r in ranks:
        h = ((h ^ (r + 0x9e3779b9)) * 1099511628211) & 0xFFFFFFFFFFFFFFFF
    return "%d-%d" % (len(ranks), h)


def group_for_ranks(ranks):
    """Finds or creates the group with exactly these ranks (collective across the world when creating)."""
    ranks = sorted(ranks)
    if len(ranks) == _state.world:
        return GlobalComm.WORLD_COMM_GROUP
    name = stage_rank_list_name(ranks)
    if name not in _state.groups:
        create_group(name, ranks)
    return name
