"""Parameter-server training: parameters marked with ``Parameter.set_param_ps()`` live on a server process; workers
pull their values before the forward pass and push gradients after backward, and the server applies the optimizer.

    # server process (role MS_PSERVER)
    server = ParameterServer(("127.0.0.1", 29700), num_workers=2, optimizer="sgd", learning_rate=0.1)
    server.serve_forever()                      # returns when every worker has said goodbye

    # worker processes (role MS_WORKER)
    worker = PSWorker(("127.0.0.1", 29700), rank)
    worker.init_params(net)                     # first worker's values become the server's tables
    for batch in data:
        worker.pull(net)
        loss = ...; loss.backward()
        worker.push(net)                        # synchronous: the update is applied once all workers have pushed

Embedding tables can be pushed sparsely (``push(net, sparse=True)`` sends only the rows with a non-zero gradient).
The update rules are SGD with momentum and Adam, applied on the server in fp32.

The reference's server / worker / scheduler nodes speak its own TCP protocol with node recovery
(ccsrc/ps/core/*, ps/parameter_server.cc, ps/worker.cc; Python side ``set_ps_context``, ``Parameter.set_param_ps``,
``nn.EmbeddingLookup(target='CPU')``).  Here the transport is ``multiprocessing.connection`` (length-prefixed pickled
messages over TCP, authenticated with a shared key); the training semantics (synchronous push / pull, sparse rows)
are the same."""
from __future__ import annotations

import threading
from multiprocessing.connection import Client, Listener

import numpy as np
import torch

_AUTH = b"mindspore_b200-ps"


def _ps_params(net):
    return [(p.name, p) for p in net.get_parameters() if getattr(p, "is_param_ps", False) and p.requires_grad]


class ParameterServer:
    def __init__(self, address, num_workers, optimizer="sgd", learning_rate=0.01, momentum=0.0, beta1=0.9, beta2=0.999,
                 eps=1e-8, weight_decay=0.0):
        if optimizer not in ("sgd", "adam"):
            raise ValueError("ParameterServer supports 'sgd' and 'adam', got %r" % (optimizer,))
        self.address, self.num_workers = tuple(address), int(num_workers)
        self.kind, self.lr, self.momentum, self.b1, self.b2, self.eps, self.wd = \
            optimizer, learning_rate, momentum, beta1, beta2, eps, weight_decay
        self.tables, self.state, self.version = {}, {}, 0
        self._pending, self._pushed = {}, 0
        self._lock = threading.Condition()
        self._alive = self.num_workers
        self._listener = None

    # ------------------------------------------------------------------ update rule
    def _apply(self, name, grad, rows=None):
        w = self.tables[name]
        st = self.state.setdefault(name, {})
        if rows is not None:                              # sparse rows: expand to dense only for the touched rows
            g = np.zeros_like(w)
            np.add.at(g, rows, grad)
            touched = np.zeros(w.shape[0], dtype=bool)
            touched[rows] = True
        else:
            g, touched = grad, None
        if self.wd:
            g = g + self.wd * w
        if self.kind == "sgd":
            if self.momentum:
                m = st.setdefault("m", np.zeros_like(w))
                if touched is None:
                    m[:] = self.momentum * m + g
                    w -= self.lr * m
                else:
                    m[touched] = self.momentum * m[touched] + g[touched]
                    w[touched] -= self.lr * m[touched]
            elif touched is None:
                w -= self.lr * g
            else:
                w[touched] -= self.lr * g[touched]
            return
        m, v = st.setdefault("m", np.zeros_like(w)), st.setdefault("v", np.zeros_like(w))
        t = st["t"] = st.get("t", 0) + 1
        sel = slice(None) if touched is None else touched
        m[sel] = self.b1 * m[sel] + (1 - self.b1) * g[sel]
        v[sel] = self.b2 * v[sel] + (1 - self.b2) * g[sel] ** 2
        lr_t = self.lr * np.sqrt(1 - self.b2 ** t) / (1 - self.b1 ** t)
        w[sel] -= lr_t * m[sel] / (np.sqrt(v[sel]) + self.eps)

    # ------------------------------------------------------------------ request handling
    def _handle(self, conn):
        try:
            while True:
                try:
                    msg = conn.recv()
                except (EOFError, OSError):
                    break
                op = msg[0]
                if op == "init":
                    with self._lock:
                        for name, value in msg[1].items():
                            self.tables.setdefault(name, np.array(value, dtype=np.float32))
                    conn.send(("ok",))
                elif op == "pull":
                    with self._lock:
                        conn.send(("values", {n: self.tables[n] for n in msg[1]}, self.version))
                elif op == "push":
                    with self._lock:
                        for name, payload in msg[1].items():
                            self._pending.setdefault(name, []).append(payload)
                        self._pushed += 1
                        target = self.version + 1
                        if self._pushed == self._alive:                  # last worker of the round: apply
                            for name, items in self._pending.items():
                                dense = [g for g in items if not isinstance(g, tuple)]
                                if dense:
                                    self._apply(name, sum(dense) / self.num_workers)
                                sparse = [g for g in items if isinstance(g, tuple)]
                                if sparse:
                                    rows = np.concatenate([r for r, _ in sparse])
                                    vals = np.concatenate([v for _, v in sparse]) / self.num_workers
                                    self._apply(name, vals, rows)
                            self._pending, self._pushed = {}, 0
                            self.version = target
                            self._lock.notify_all()
                        else:
                            self._lock.wait_for(lambda: self.version >= target, timeout=120)
                    conn.send(("ok", self.version))
                elif op == "bye":
                    conn.send(("ok",))
                    break
                else:
                    conn.send(("error", "unknown request %r" % (op,)))
        finally:
            with self._lock:
                self._alive -= 1
                if self._alive and self._pushed == self._alive and self._pending:
                    self._lock.notify_all()
                self._lock.notify_all()
            conn.close()

    def serve_forever(self):
        self._listener = Listener(self.address, authkey=_AUTH)
        threads = []
        for _ in range(self.num_workers):
            conn = self._listener.accept()
            t = threading.Thread(target=self._handle, args=(conn,), daemon=True)
            t.start()
            threads.append(t)
        for t in threads:
            t.join()
        self._listener.close()

    def start(self):
        """Serves in a background thread (tests / single-host jobs)."""
        th = threading.Thread(target=self.serve_forever, daemon=True)
        th.start()
        return th


class PSWorker:
    def __init__(self, address, rank=0, retries=50):
        import time
        last = None
        for _ in range(retries):
            try:
                self.conn = Client(tuple(address), authkey=_AUTH)
                break
            except (ConnectionRefusedError, OSError) as e:
                last = e
                time.sleep(0.1)
        else:
            raise ConnectionError("parameter server at %s:%s is not reachable: %s" % (address[0], address[1], last))
        self.rank = rank

    def _call(self, *msg):
        self.conn.send(msg)
        reply = self.conn.recv()
        if reply[0] == "error":
            raise RuntimeError(reply[1])
        return reply

    def init_params(self, net):
        self._call("init", {n: p.detach().float().cpu().numpy() for n, p in _ps_params(net)})

    def pull(self, net):
        params = _ps_params(net)
        _, values, version = self._call("pull", [n for n, _ in params])
        with torch.no_grad():
            for n, p in params:
                p.copy_(torch.from_numpy(values[n]).to(p.device, p.dtype))
        return version

    def push(self, net, sparse=False):
        payload = {}
        for n, p in _ps_params(net):
            g = getattr(p, "main_grad", None)
            g = g if g is not None and p.grad is None else p.grad
            if g is None:
                g = torch.zeros_like(p)
            g = g.detach().float().cpu().numpy()
            if sparse and g.ndim >= 2:
                rows = np.nonzero(np.abs(g).reshape(g.shape[0], -1).sum(1))[0]
                payload[n] = (rows, g[rows])
            else:
                payload[n] = g
            p.grad = None
        return self._call("push", payload)[1]

    def close(self):
        try:
            self._call("bye")
        finally:
            self.conn.close()
