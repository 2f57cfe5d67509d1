"""Recovery context: per-rank bookkeeping of the latest checkpoints and agreement on the latest one that
every rank has, for ``MS_ENABLE_RECOVERY=1`` restarts.

Environment: ``MS_ENABLE_RECOVERY`` (0/1), ``MS_RECOVERY_PATH`` (directory), ``MS_RECOVERY_INTERVAL`` (seconds).
Each rank records ``{"epoch", "step", "path"}`` in ``<path>/rank_<r>/latest.json`` after a save; on restart all
ranks gather everyone's record and take the minimum (epoch, step).
Parity: mindspore/ccsrc/distributed/recovery/recovery_context.cc:80-135 (init), :137-323
(ObtainGlobalLatestCkptInfo), python/mindspore/parallel/_recovery_context.py.
"""
import json
import os


class RecoveryContext:
    def __init__(self):
        self.refresh()

    def refresh(self):
        self.enabled = os.environ.get("MS_ENABLE_RECOVERY", "0") == "1"
        self.path = os.environ.get("MS_RECOVERY_PATH", "")
        self.interval = int(os.environ.get("MS_RECOVERY_INTERVAL", "30"))
        if self.enabled and not self.path:
            raise ValueError("MS_ENABLE_RECOVERY=1 needs MS_RECOVERY_PATH")

    def rank_dir(self, rank):
        d = os.path.join(self.path, "rank_%d" % rank)
        os.makedirs(d, exist_ok=True)
        return d

    def record(self, rank, epoch, step, ckpt_path):
        tmp = os.path.join(self.rank_dir(rank), "latest.json.tmp")
        with open(tmp, "w") as f:
            json.dump({"epoch": epoch, "step": step, "path": ckpt_path}, f)
        os.replace(tmp, os.path.join(self.rank_dir(rank), "latest.json"))

    def record_all(self, rank, epoch, step, ckpt_path, keep=8):
        """Appends to this rank's history (``history.json``, newest last, ``keep`` entries) besides ``latest.json``:
        after a failure the ranks agree on the newest point that all of them still have."""
        self.record(rank, epoch, step, ckpt_path)
        hp = os.path.join(self.rank_dir(rank), "history.json")
        hist = []
        if os.path.exists(hp):
            with open(hp) as f:
                hist = json.load(f)
        hist = [h for h in hist if (h["epoch"], h["step"]) != (epoch, step)] + \
            [{"epoch": epoch, "step": step, "path": ckpt_path}]
        hist = hist[-keep:]
        with open(hp + ".tmp", "w") as f:
            json.dump(hist, f)
        os.replace(hp + ".tmp", hp)

    def local_history(self, rank):
        hp = os.path.join(self.path, "rank_%d" % rank, "history.json")
        if not os.path.exists(hp):
            one = self.local_latest(rank)
            return [one] if one else []
        with open(hp) as f:
            return [h for h in json.load(f) if os.path.exists(h["path"])]

    def agree(self, rank):
        """The newest checkpoint every rank has, found by an all-gather over the current communicator (each rank
        reads only its own directory).  Returns this rank's record for it, or None."""
        from ..communication.elastic import agree_on_checkpoint
        hist = self.local_history(rank)
        point = agree_on_checkpoint([(h["epoch"], h["step"]) for h in hist])
        if point is None:
            return None
        return next(h for h in hist if (h["epoch"], h["step"]) == point)

    def local_latest(self, rank):
        p = os.path.join(self.path, "rank_%d" % rank, "latest.json")
        if not os.path.exists(p):
            return None
        with open(p) as f:
            return json.load(f)

    def latest_common_checkpoint(self, rank=None, world=None):
        """(epoch, step) = min over ranks, read from every rank's directory: only for jobs whose ranks share
        ``MS_RECOVERY_PATH`` (one node).  ``agree`` is the general form.  Returns this rank's file or None."""
        from ..communication import management as M
        if rank is None:
            rank = M._state.rank if M.GlobalComm.INITED else 0
        if world is None:
            world = M._state.world if M.GlobalComm.INITED else 1
        mine = self.local_latest(rank)
        records = [self.local_latest(r) for r in range(world)]
        if any(r is None for r in records):
            return None
        epoch, step = min((r["epoch"], r["step"]) for r in records)
        if mine["epoch"] == epoch and mine["step"] == step:
            return mine
        cand = os.path.join(os.path.dirname(mine["path"]), "recovery-%d_%d.ckpt" % (epoch, step))
        return {"epoch": epoch, "step": step, "path": cand} if os.path.exists(cand) else None


_ctx = None


def recovery_context():
    global _ctx
    if _ctx is None:
        _ctx = RecoveryContext()
    else:
        _ctx.refresh()
    return _ctx
