"""Flight recorder: the last N runtime events of this process (collectives, step boundaries, checkpoint writes,
user marks), dumped to ``<MS_RDR_PATH>/rank_<r>/rdr.txt`` when the process dies with an exception (mode 1) or
always at exit (mode 2).

Switches follow the reference's RDR (ccsrc/debug/rdr/recorder_manager.cc; env ``MS_RDR_ENABLE``, ``MS_RDR_MODE``,
``MS_RDR_PATH``; ``set_context(env_config_path=...)`` json key ``rdr``).  The ring itself is native
(``csrc/host/flight_recorder.cpp``); recording costs one atomic add and a 128-byte store."""
from __future__ import annotations

import atexit
import ctypes
import os
import struct
import sys

from .. import _native

CATEGORIES = {"user": 0, "kernel": 1, "collective": 2, "step": 3, "checkpoint": 4, "memory": 5, "cluster": 6}
_NAMES = {v: k for k, v in CATEGORIES.items()}
_enabled = False
_sig_done = False
_state = {"path": None, "mode": 1, "failed": False, "hooked": False, "step": 0}


def _lib():
    global _sig_done
    lib = _native.host()
    if not _sig_done:
        I, L = ctypes.c_int, ctypes.c_longlong
        lib.msb_fr_configure.argtypes = [I]
        lib.msb_fr_record.restype = ctypes.c_ulonglong
        lib.msb_fr_record.argtypes = [I, I, L, L, ctypes.c_char_p]
        lib.msb_fr_count.restype = ctypes.c_ulonglong
        lib.msb_fr_snapshot.argtypes = [ctypes.c_void_p, I]
        lib.msb_fr_dump.argtypes = [ctypes.c_char_p]
        _sig_done = True
    return lib


def enabled():
    return _enabled


def enable(path=None, mode=1, capacity=4096):
    """Turns recording on.  ``mode`` 1: dump when the process ends with an uncaught exception; 2: dump at every exit."""
    global _enabled
    _lib().msb_fr_configure(int(capacity))
    rank = os.environ.get("RANK", os.environ.get("RANK_ID", "0"))
    _state["path"] = os.path.join(path or os.environ.get("MS_RDR_PATH", "./rdr"), "rank_%s" % rank)
    _state["mode"] = int(mode)
    _enabled = True
    if not _state["hooked"]:
        _state["hooked"] = True
        prev = sys.excepthook

        def hook(tp, val, tb):
            _state["failed"] = True
            record("user", "uncaught %s: %s" % (tp.__name__, str(val)[:50]))
            prev(tp, val, tb)

        sys.excepthook = hook
        atexit.register(_at_exit)


def disable():
    global _enabled
    _enabled = False


def enable_from_env():
    if os.environ.get("MS_RDR_ENABLE", "0") == "1" and not _enabled:
        enable(os.environ.get("MS_RDR_PATH"), int(os.environ.get("MS_RDR_MODE", "1")))
    return _enabled


def set_step(step):
    _state["step"] = int(step)


def record(category, text="", a=0, b=0, step=None):
    if not _enabled:
        return
    cat = CATEGORIES.get(category, 0) if isinstance(category, str) else int(category)
    _lib().msb_fr_record(cat, _state["step"] if step is None else int(step), int(a), int(b),
                         text.encode("utf-8", "replace")[:79])


def snapshot(max_events=4096):
    """Most recent events, oldest first: dicts with seq, t_ns, category, step, a, b, text."""
    buf = ctypes.create_string_buffer(max_events * 144)
    n = _lib().msb_fr_snapshot(buf, max_events)
    out = []
    for i in range(n):
        seq, t, cat, step, a, b, _, _ = struct.unpack_from("<8q", buf.raw, i * 144)
        text = buf.raw[i * 144 + 64:i * 144 + 144].split(b"\0", 1)[0].decode("utf-8", "replace")
        out.append({"seq": seq, "t_ns": t, "category": _NAMES.get(cat, str(cat)), "step": step, "a": a, "b": b,
                    "text": text})
    return out


def dump(path=None):
    path = path or os.path.join(_state["path"] or "./rdr", "rdr.txt")
    os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
    if _lib().msb_fr_dump(path.encode()):
        raise OSError("could not write %s" % path)
    return path


def _at_exit():
    if _enabled and (_state["mode"] == 2 or _state["failed"]):
        try:
            dump()
        except OSError:
            pass
