"""Spawns ``world`` CPU ranks (gloo rendezvous on 127.0.0.1) and collects one result per rank, failing fast when
a rank dies."""
import os
import queue as _q
import sys
import time

import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
_port_salt = [0]


def _entry(fn, rank, world, port, q, args):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port),
                      LOCAL_RANK=str(rank))
    q.put((rank, fn(rank, world, *args)))


def run_ranks(fn, world, *args, timeout=300):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    _port_salt[0] += 1
    port = 21000 + (os.getpid() * 7 + _port_salt[0] * 131) % 8000
    procs = [ctx.Process(target=_entry, args=(fn, r, world, port, q, args)) for r in range(world)]
    for p in procs:
        p.start()
    res, deadline = {}, time.time() + timeout
    while len(res) < world:
        try:
            r, v = q.get(timeout=1)
            res[r] = v
        except _q.Empty:
            dead = [p.exitcode for p in procs if p.exitcode not in (None, 0)]
            if dead or time.time() > deadline:
                for p in procs:
                    p.kill()
                raise AssertionError("worker failed or timed out: exit codes %s" % [p.exitcode for p in procs])
    for p in procs:
        p.join(60)
        assert p.exitcode == 0
    return [res[r] for r in range(world)]
