"""SciPy-like numerical routines on tensors: ``linalg``, ``optimize`` and ``sparse.linalg``
(python/mindspore/scipy in the reference)."""
from . import fft, linalg, optimize, sparse  # noqa: F401
