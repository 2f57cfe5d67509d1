"""Layers over dual numbers (second unit squared = 0); see ``_algebra``."""
from ._algebra import make_namespace as _make

globals().update(_make(0))
__all__ = list(_make(0))
