"""Layers over double numbers (second unit squared = 1); see ``_algebra``."""
from ._algebra import make_namespace as _make

globals().update(_make(1))
__all__ = list(_make(1))
