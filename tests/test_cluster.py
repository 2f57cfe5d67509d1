"""Cluster bootstrap, metadata store, heartbeat-based failure detection and the msrun launcher.
Failures are made on the host only: a worker that stops heartbeating, a worker process that raises."""
import os
import subprocess
import sys
import textwrap
import time

import pytest

from mindspore_b200.communication.cluster import ClusterError, Scheduler, WorkerClient

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_register_store_and_heartbeat_timeout():
    with Scheduler(0, expected_workers=2, node_timeout_s=0.6) as sched:
        a = WorkerClient("127.0.0.1", sched.port, "node-a")
        b = WorkerClient("127.0.0.1", sched.port, "node-b")
        assert {a.register(), b.register()} == {0, 1}
        assert a.world == 2 and sched.registered() == 2
        again = WorkerClient("127.0.0.1", sched.port, "node-a")
        assert again.register() == a.rank                      # a restarted node keeps its rank
        extra = WorkerClient("127.0.0.1", sched.port, "node-c")
        with pytest.raises(ClusterError):
            extra.register(retry_s=0.3)                          # the job is full
        a.put("unique_id", b"\x00\x01binary\n\xff")
        assert b.get("unique_id") == b"\x00\x01binary\n\xff"
        assert b.get("missing") is None
        b.delete("unique_id")
        assert a.get("unique_id") is None
        assert a.heartbeat() == 0 and a.ready
        a.check_health()
        a.start_heartbeat(0.1)                                   # b never heartbeats again
        deadline = time.time() + 5
        while a.abnormal == 0 and time.time() < deadline:
            time.sleep(0.05)
        assert a.abnormal == 1 and sched.abnormal_nodes() == 1
        with pytest.raises(ClusterError, match="stopped sending heartbeats"):
            a.check_health()
        b.heartbeat()                                            # b comes back
        time.sleep(0.3)
        assert a.heartbeat() == 0
        a.unregister()


def test_worker_notices_lost_scheduler():
    sched = Scheduler(0, 1, 5.0)
    w = WorkerClient("127.0.0.1", sched.port, "n0", timeout_s=0.5)
    w.register()
    sched.stop()
    for _ in range(3):
        assert w.heartbeat() == -1
    with pytest.raises(ClusterError, match="scheduler"):
        w.check_health()


def _script(tmp_path, body):
    path = tmp_path / "task.py"
    path.write_text("import sys\nsys.path.insert(0, %r)\n" % ROOT + textwrap.dedent(body))
    return str(path)


def _msrun(tmp_path, script, port, extra=()):
    cmd = [sys.executable, "-m", "mindspore_b200.msrun", "--worker_num", "2", "--local_worker_num", "2",
           "--master_port", str(port), "--log_dir", str(tmp_path / "logs"), "--join", "True",
           "--heartbeat_timeout", "3", *extra, script]
    return subprocess.run(cmd, cwd=ROOT, capture_output=True, text=True, timeout=240)


def test_msrun_runs_collective_job(tmp_path):
    script = _script(tmp_path, """
        import torch
        import mindspore_b200 as ms
        from mindspore_b200.communication import init, get_rank, get_group_size, release
        from mindspore_b200.communication import cluster
        ms.set_context(device_target="CPU")
        init("mccl")
        assert cluster._worker is not None and cluster._worker.rank is not None
        t = torch.ones(4) * (get_rank() + 1)
        torch.distributed.all_reduce(t)
        assert float(t[0]) == 3.0 and get_group_size() == 2
        cluster.check_cluster_health()
        print("rank", get_rank(), "done", flush=True)
        release()
    """)
    res = _msrun(tmp_path, script, 23000 + os.getpid() % 2000)
    logs = {i: (tmp_path / "logs" / ("worker_%d.log" % i)).read_text() for i in range(2)}
    assert res.returncode == 0, (res.stdout, res.stderr, logs)
    assert "done" in logs[0] and "done" in logs[1]


def test_msrun_stops_job_when_a_rank_raises(tmp_path):
    script = _script(tmp_path, """
        import os, time
        if os.environ["RANK"] == "1":
            raise RuntimeError("injected host failure before joining the job")
        time.sleep(120)        # rank 0 would wait for its peer; the launcher must end it
    """)
    t0 = time.time()
    res = _msrun(tmp_path, script, 25000 + os.getpid() % 2000)
    assert res.returncode != 0
    assert "worker 1 exited" in res.stdout
    assert time.time() - t0 < 60
    assert "injected host failure" in (tmp_path / "logs" / "worker_1.log").read_text()
