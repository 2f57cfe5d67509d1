"""A job that loses a rank between two steps re-forms: the survivors learn of the loss on the host (heartbeat
monitor, or the error of their next collective under a short process-group timeout), the restarted rank (same
node id -> same rank) opens a new communicator generation through the scheduler, all ranks agree by all-gather on
the newest checkpoint every one of them has, reload it and finish - ending where an uninterrupted run ends.
CPU ranks over gloo only; no device is involved.  Also: the scheduler's state survives a scheduler restart, and a
communicator that cannot come up ends in a timeout error instead of a hang.
Reference: distributed/collective/collective_manager.cc:80-146,278-358; cluster/topology/meta_server_node.cc:561-635;
distributed/recovery/recovery_context.cc:137-323; python/mindspore/train/model.py:1016-1064."""
import os
import subprocess
import sys
import textwrap
import time

import pytest
import torch

from mindspore_b200.communication.cluster import Scheduler, WorkerClient

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = r'''
import os, sys, json, time
sys.path.insert(0, %(root)r)
import torch
import torch.distributed as dist
import mindspore_b200 as ms
from mindspore_b200 import nn
from mindspore_b200.communication.cluster import WorkerClient, ClusterError
from mindspore_b200.communication.elastic import ElasticComm
from mindspore_b200.parallel.recovery import RecoveryContext

port, node, out_dir, die_after, total = int(sys.argv[1]), sys.argv[2], sys.argv[3], int(sys.argv[4]), int(sys.argv[5])
os.environ["MS_ENABLE_RECOVERY"] = "1"
os.environ["MS_RECOVERY_PATH"] = os.path.join(out_dir, "recovery_" + node)      # private per rank: no shared files
ms.set_context(device_target="CPU")
w = WorkerClient("127.0.0.1", port, node, timeout_s=2.0)
w.register()
w.start_heartbeat(0.1)
comm = ElasticComm(w, backend="gloo", init_timeout_s=60.0, op_timeout_s=4.0).start()
rank, world = w.rank, w.world
rc = RecoveryContext()

ms.set_seed(1)
net = nn.SequentialCell([nn.Dense(4, 8), nn.Tanh(), nn.Dense(8, 2)])
opt = nn.Momentum(net.trainable_params(), learning_rate=0.1, momentum=0.9)
loss_fn = nn.MSELoss()
params = list(net.trainable_params())


def batch(step, r):
    g = torch.Generator().manual_seed(1000 * step + r)
    return torch.randn(6, 4, generator=g), torch.randn(6, 2, generator=g)


def save(step):
    path = os.path.join(rc.rank_dir(rank), "recovery-0_%%d.ckpt" %% step)
    ms.save_checkpoint([{"name": p.name, "data": p} for p in params] +
                       [{"name": m.name, "data": m} for m in opt.moments], path)
    rc.record_all(rank, 0, step, path)


def train_step(step):
    x, y = batch(step, rank)
    for p in params:
        p.grad = None
    loss_fn(net(ms.Tensor(x)), ms.Tensor(y)).backward()
    grads = []
    for p in params:
        g = p.grad.detach().clone()
        dist.all_reduce(g)                       # raises under the short timeout when a peer is gone
        grads.append(g / world)
    opt(tuple(grads))


def load(path):
    loaded = ms.load_checkpoint(path)
    with torch.no_grad():
        for p in list(params) + list(opt.moments):
            torch.Tensor.copy_(p, loaded[p.name].to(p.dtype))


def recover():
    comm.reinit(timeout_s=60.0)
    rec = rc.agree(rank)
    load(rec["path"])
    return rec["step"]


step, start_step = 0, 0
hist = rc.local_history(rank)
if hist:                                         # this process is a restart: join the others' recovery
    rec = rc.agree(rank)
    load(rec["path"])
    step = rec["step"]
recoveries = 0
while step < total:
    try:
        if comm.need_reinit():
            raise ClusterError("a node was lost or a new generation was opened")
        train_step(step + 1)
    except (ClusterError, RuntimeError) as e:
        if recoveries >= 4:                          # (a loaded test machine may miss a heartbeat window)
            raise
        recoveries += 1
        step = recover()
        continue
    step += 1
    save(step)
    if die_after and step == die_after and not hist:
        os._exit(17)                             # leaves between two steps, nothing in flight
dist.barrier()
json.dump({"rank": rank, "recoveries": recoveries, "generation": comm.generation,
           "params": [p.detach().reshape(-1).tolist() for p in params]},
          open(os.path.join(out_dir, "result_%%s.json" %% node), "w"))
w.unregister()
'''


def _reference(total, world=3):
    import mindspore_b200 as ms
    from mindspore_b200 import nn
    ms.set_context(device_target="CPU")
    ms.set_seed(1)
    net = nn.SequentialCell([nn.Dense(4, 8), nn.Tanh(), nn.Dense(8, 2)])
    opt = nn.Momentum(net.trainable_params(), learning_rate=0.1, momentum=0.9)
    loss_fn = nn.MSELoss()
    params = list(net.trainable_params())
    for step in range(1, total + 1):
        acc = [torch.zeros_like(p) for p in params]
        for r in range(world):
            g = torch.Generator().manual_seed(1000 * step + r)
            x, y = torch.randn(6, 4, generator=g), torch.randn(6, 2, generator=g)
            for p in params:
                p.grad = None
            loss_fn(net(ms.Tensor(x)), ms.Tensor(y)).backward()
            for a, p in zip(acc, params):
                a += p.grad
        opt(tuple(a / world for a in acc))
    return [p.detach().reshape(-1).tolist() for p in params]


def test_job_reforms_after_a_rank_left_between_steps(tmp_path):
    import json
    script = tmp_path / "worker.py"
    script.write_text(WORKER % {"root": ROOT})
    total, die_after = 6, 3
    with Scheduler(0, expected_workers=3, node_timeout_s=3.0, persist_path=str(tmp_path / "sched.state")) as sched:
        def launch(node, die):
            return subprocess.Popen([sys.executable, str(script), str(sched.port), node, str(tmp_path), str(die),
                                     str(total)], stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        procs = {"n0": launch("n0", 0), "n1": launch("n1", die_after), "n2": launch("n2", 0)}
        assert procs["n1"].wait(timeout=120) == 17, procs["n1"].stdout.read()[-2000:]
        time.sleep(0.5)
        procs["n1"] = launch("n1", 0)                       # restarted with the same node id
        for name, p in procs.items():
            try:
                rc = p.wait(timeout=180)
            except subprocess.TimeoutExpired:
                for q in procs.values():
                    q.kill()
                raise AssertionError("worker %s hung:\n%s" % (name, p.stdout.read()[-3000:]))
            assert rc == 0, "worker %s failed:\n%s" % (name, p.stdout.read()[-3000:])
    want = _reference(total)
    for node in ("n0", "n1", "n2"):
        res = json.load(open(tmp_path / ("result_%s.json" % node)))
        assert res["generation"] == 1
        if node != "n1":
            assert res["recoveries"] == 1
        for a, b in zip(res["params"], want):
            torch.testing.assert_close(torch.tensor(a), torch.tensor(b), rtol=1e-5, atol=1e-6)


def test_scheduler_state_survives_a_restart(tmp_path):
    state = str(tmp_path / "sched.state")
    sched = Scheduler(0, expected_workers=2, node_timeout_s=5.0, persist_path=state, persist_interval_s=0.1)
    a, b = WorkerClient("127.0.0.1", sched.port, "alpha"), WorkerClient("127.0.0.1", sched.port, "beta")
    ra, rb = a.register(), b.register()
    a.put("job/config", b"\x00binary\xff")
    assert a.add("comm/generation", 1) == 1 and a.add("comm/generation", 1) == 2
    sched.stop()                                            # the scheduler process "dies" ...
    assert os.path.isfile(state)
    again = Scheduler(0, expected_workers=2, node_timeout_s=5.0, persist_path=state)      # ... and comes back
    try:
        assert again.restored >= 4 and again.registered() == 2
        a2, b2 = WorkerClient("127.0.0.1", again.port, "alpha"), WorkerClient("127.0.0.1", again.port, "beta")
        assert (b2.register(), a2.register()) == (rb, ra)   # ranks are what they were
        assert a2.get("job/config") == b"\x00binary\xff" and a2.add("comm/generation", 0) == 2
        with pytest.raises(Exception):
            WorkerClient("127.0.0.1", again.port, "gamma").register(retry_s=0.3)
    finally:
        again.stop()


def test_communicator_init_times_out_instead_of_hanging(tmp_path):
    from mindspore_b200.communication.elastic import CommInitTimeout, ElasticComm, run_with_watchdog
    with pytest.raises(CommInitTimeout):
        run_with_watchdog(lambda: time.sleep(5), 0.2, "a rendezvous nobody joins")
    with Scheduler(0, expected_workers=2, node_timeout_s=5.0) as sched:
        w = WorkerClient("127.0.0.1", sched.port, "late", timeout_s=1.0)
        w.register()
        assert w.rank == 0
        comm = ElasticComm(w, backend="gloo", init_timeout_s=1.5, op_timeout_s=1.0)
        t0 = time.time()
        with pytest.raises((CommInitTimeout, RuntimeError)):
            comm.start()                                    # rank 1 never arrives
        assert time.time() - t0 < 30
