"""``python -m mindspore_b200.msrun``: the dynamic-networking launcher.

Starts the scheduler inside the launcher process and one worker process per local device, each with the
environment the communication layer reads (MS_ROLE, MS_WORKER_NUM, MS_SCHED_HOST, MS_SCHED_PORT, MS_NODE_ID, plus
RANK / WORLD_SIZE / LOCAL_RANK / MASTER_ADDR / MASTER_PORT for the NCCL rendezvous).  Worker output goes to
``<log_dir>/worker_<rank>.log``.  With ``--join`` the launcher waits, watches the workers and the scheduler's
heartbeat table, and when a worker exits with an error (or stops sending heartbeats) it terminates the others by
their process ids and returns the failing exit code.

Parity: mindspore/python/mindspore/parallel/cluster/run.py (msrun entry), process_entity/_api.py:83-333
(_ProcessManager: start_scheduler / start_workers / join_processes / log monitoring), _utils.py (bind_core)."""
from __future__ import annotations

import argparse
import os
import signal
import subprocess
import sys
import time


def parse(argv=None):
    ap = argparse.ArgumentParser(prog="msrun", description="Launch a distributed job on this node")
    ap.add_argument("--worker_num", type=int, default=8, help="total number of worker processes of the job")
    ap.add_argument("--local_worker_num", type=int, default=None, help="workers started on this node")
    ap.add_argument("--master_addr", default="127.0.0.1")
    ap.add_argument("--master_port", type=int, default=8118)
    ap.add_argument("--node_rank", type=int, default=0)
    ap.add_argument("--log_dir", default="")
    ap.add_argument("--join", type=lambda s: str(s).lower() in ("1", "true", "yes"), default=False)
    ap.add_argument("--cluster_time_out", type=int, default=600)
    ap.add_argument("--bind_core", type=lambda s: str(s).lower() in ("1", "true", "yes"), default=False)
    ap.add_argument("--sim_level", type=int, default=-1)
    ap.add_argument("--sim_rank_id", type=int, default=-1)
    ap.add_argument("--rank_table_file", default="")
    ap.add_argument("--heartbeat_timeout", type=float, default=30.0)
    ap.add_argument("task_script")
    ap.add_argument("task_script_args", nargs=argparse.REMAINDER)
    args = ap.parse_args(argv)
    if args.local_worker_num is None:
        args.local_worker_num = args.worker_num
    if args.local_worker_num > args.worker_num:
        ap.error("--local_worker_num must not exceed --worker_num")
    return args


def _core_ranges(n):
    cores = sorted(os.sched_getaffinity(0))
    per = max(1, len(cores) // max(n, 1))
    return [cores[i * per:(i + 1) * per] or cores for i in range(n)]


class ProcessManager:
    def __init__(self, args):
        self.args = args
        self.workers = []      # (rank, Popen, log file handle)
        self.scheduler = None
        self.cluster_port = None

    def start_scheduler(self):
        if self.args.node_rank != 0 or self.args.sim_level >= 0:
            return
        from .communication.cluster import Scheduler
        # with MS_ENABLE_RECOVERY the scheduler keeps its node table and metadata store in MS_RECOVERY_PATH, so a
        # restarted launcher hands every node its old rank (cluster/topology/meta_server_node.cc:561-635)
        persist = None
        if os.environ.get("MS_ENABLE_RECOVERY", "0") == "1" and os.environ.get("MS_RECOVERY_PATH"):
            os.makedirs(os.environ["MS_RECOVERY_PATH"], exist_ok=True)
            persist = os.path.join(os.environ["MS_RECOVERY_PATH"], "scheduler.state")
        self.scheduler = Scheduler(0, self.args.worker_num, self.args.heartbeat_timeout, persist_path=persist)
        self.cluster_port = self.scheduler.port

    def _env(self, rank, local_rank):
        a = self.args
        env = dict(os.environ)
        env.update(MS_ROLE="MS_WORKER", MS_WORKER_NUM=str(a.worker_num), MS_SCHED_HOST=a.master_addr,
                   MS_SCHED_PORT=str(a.master_port), MS_NODE_ID=str(rank), RANK=str(rank), RANK_ID=str(rank),
                   WORLD_SIZE=str(a.worker_num), RANK_SIZE=str(a.worker_num), LOCAL_RANK=str(local_rank),
                   DEVICE_ID=str(local_rank), MASTER_ADDR=a.master_addr, MASTER_PORT=str(a.master_port),
                   MS_CLUSTER_TIMEOUT=str(a.cluster_time_out))
        if self.cluster_port:
            env["MSB_CLUSTER_PORT"] = str(self.cluster_port)
        if a.sim_level >= 0:
            env["MS_SIMULATION_LEVEL"] = str(a.sim_level)
        if a.rank_table_file:
            env["RANK_TABLE_FILE"] = a.rank_table_file
        return env

    def start_workers(self):
        a = self.args
        if a.log_dir:
            os.makedirs(a.log_dir, exist_ok=True)
        ranks = [a.sim_rank_id] if a.sim_level >= 0 and a.sim_rank_id >= 0 else \
            [a.node_rank * a.local_worker_num + i for i in range(a.local_worker_num)]
        cores = _core_ranges(len(ranks)) if a.bind_core else None
        for i, rank in enumerate(ranks):
            cmd = [sys.executable, a.task_script] + list(a.task_script_args)
            if a.task_script.endswith(".py") is False and os.access(a.task_script, os.X_OK):
                cmd = [a.task_script] + list(a.task_script_args)
            log = open(os.path.join(a.log_dir, "worker_%d.log" % rank), "w") if a.log_dir else None
            p = subprocess.Popen(cmd, env=self._env(rank, i), stdout=log or None,
                                 stderr=subprocess.STDOUT if log else None, start_new_session=True)
            if cores:
                try:
                    os.sched_setaffinity(p.pid, cores[i])
                except OSError:
                    pass
            self.workers.append((rank, p, log))

    def _terminate_others(self, except_pid=None):
        for _rank, p, _log in self.workers:
            if p.poll() is None and p.pid != except_pid:
                try:
                    os.killpg(p.pid, signal.SIGTERM)
                except OSError:
                    pass
        deadline = time.time() + 10
        for _rank, p, _log in self.workers:
            while p.poll() is None and time.time() < deadline:
                time.sleep(0.05)
            if p.poll() is None:
                try:
                    os.killpg(p.pid, signal.SIGKILL)
                except OSError:
                    pass

    def join(self):
        """Waits for the workers.  Returns 0 when all succeed, else the first failing exit code (after stopping
        the remaining workers)."""
        rc = 0
        try:
            while True:
                running = 0
                for rank, p, _log in self.workers:
                    code = p.poll()
                    if code is None:
                        running += 1
                    elif code != 0 and rc == 0:
                        rc = code if code > 0 else 128 - code
                        print("[msrun] worker %d exited with code %d; stopping the job" % (rank, code), flush=True)
                        self._terminate_others(p.pid)
                if rc == 0 and self.scheduler is not None and self.scheduler.abnormal_nodes() > 0 and running:
                    print("[msrun] %d node(s) stopped sending heartbeats; stopping the job"
                          % self.scheduler.abnormal_nodes(), flush=True)
                    rc = 1
                    self._terminate_others()
                if running == 0 or rc != 0:
                    break
                time.sleep(0.2)
        finally:
            self.close()
        return rc

    def close(self):
        for _rank, _p, log in self.workers:
            if log:
                log.close()
        if self.scheduler is not None:
            self.scheduler.stop()
            self.scheduler = None


def main(argv=None):
    args = parse(argv)
    pm = ProcessManager(args)
    pm.start_scheduler()
    pm.start_workers()
    if args.join:
        return pm.join()
    # detached mode: the scheduler must outlive the launcher's foreground, so keep serving until workers end
    return pm.join() if pm.scheduler is not None else 0


if __name__ == "__main__":
    sys.exit(main())
