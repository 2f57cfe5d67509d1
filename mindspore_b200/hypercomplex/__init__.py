"""Neural-network layers over complex, dual and double (hyperbolic) numbers, on ``[2, N, ...]`` tensors."""
from . import complex, double, dual, utils  # noqa: A004

__all__ = ["complex", "dual", "double", "utils"]
