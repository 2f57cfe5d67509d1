"""SciPy-like numerical routines on tensors: ``linalg``, ``optimize`` and ``sparse.linalg``
(python/mindspore/scipy in the reference)."""
from . import linalg, optimize, sparse  # noqa: F401
