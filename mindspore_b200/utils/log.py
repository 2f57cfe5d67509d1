"""Logging with the reference's environment contract: ``GLOG_v`` (0 DEBUG .. 4 CRITICAL, default 2
WARNING), ``GLOG_logtostderr`` and ``GLOG_log_dir``.  Parity: mindspore/python/mindspore/log.py:72."""
import logging
import os
import sys

_LEVELS = {"0": logging.DEBUG, "1": logging.INFO, "2": logging.WARNING, "3": logging.ERROR, "4": logging.CRITICAL}


def _build():
    lg = logging.getLogger("mindspore_b200")
    if lg.handlers:
        return lg
    lg.setLevel(_LEVELS.get(os.environ.get("GLOG_v", "2"), logging.WARNING))
    fmt = logging.Formatter("[%(levelname)s] %(name)s(%(process)d):%(asctime)s [%(filename)s:%(lineno)d] %(message)s")
    if os.environ.get("GLOG_logtostderr", "1") == "0" and os.environ.get("GLOG_log_dir"):
        os.makedirs(os.environ["GLOG_log_dir"], exist_ok=True)
        h = logging.FileHandler(os.path.join(os.environ["GLOG_log_dir"], "mindspore_b200.%d.log" % os.getpid()))
    else:
        h = logging.StreamHandler(sys.stderr)
    h.setFormatter(fmt)
    lg.addHandler(h)
    lg.propagate = False
    return lg


logger = _build()


def get_level():
    return str({v: k for k, v in _LEVELS.items()}[logger.level])


def get_log_config():
    """The logging environment in effect, under the reference's variable names."""
    cfg = {"GLOG_v": get_level()}
    to_stderr = os.environ.get("GLOG_logtostderr", "1")
    cfg["GLOG_logtostderr"] = to_stderr
    if to_stderr == "0" and os.environ.get("GLOG_log_dir"):
        cfg["GLOG_log_dir"] = os.environ["GLOG_log_dir"]
    for k in ("GLOG_stderrthreshold", "MS_SUBMODULE_LOG_v", "logger_maxBytes", "logger_backupCount"):
        if os.environ.get(k) is not None:
            cfg[k] = os.environ[k]
    return cfg


def debug(msg, *a, **k): logger.debug(msg, *a, **k)
def info(msg, *a, **k): logger.info(msg, *a, **k)
def warning(msg, *a, **k): logger.warning(msg, *a, **k)
def error(msg, *a, **k): logger.error(msg, *a, **k)
def critical(msg, *a, **k): logger.critical(msg, *a, **k)
