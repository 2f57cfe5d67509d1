"""``dataset.core.config`` as a module: every ``set_*`` / ``get_*`` / ``load`` of the pipeline configuration, so that
``from ...dataset.core.config import set_seed`` works.  The state lives on ``dataset.config``.
Parity: mindspore/python/mindspore/dataset/core/config.py."""
from .engine import ErrorSamplesMode, config as _config

__all__ = sorted(n for n in dir(type(_config)) if n.startswith(("set_", "get_")) or n == "load") + ["ErrorSamplesMode"]


def __getattr__(name):
    try:
        return getattr(_config, name)
    except AttributeError:
        raise AttributeError("module 'dataset.core.config' has no attribute %r" % name)
