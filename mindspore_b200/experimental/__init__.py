"""Experimental API: torch-style optimizers and learning-rate schedulers (python/mindspore/experimental/optim)."""
from . import optim  # noqa: F401
from .map_parameter import MapParameter  # noqa: E402,F401
