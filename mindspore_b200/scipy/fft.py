"""Discrete cosine transforms (``scipy.fft.dct`` / ``idct`` semantics, types 1-4).  Parity: python/mindspore/scipy/fft.py."""
from __future__ import annotations

import math

import torch

from ..ops.primitive import _wrap_out

__all__ = ["dct", "idct"]


def _matrix(n, kind, norm, inverse=False):
    k = torch.arange(n, dtype=torch.float64)[:, None]
    j = torch.arange(n, dtype=torch.float64)[None, :]
    if kind == 2:
        m = 2 * torch.cos(math.pi * k * (2 * j + 1) / (2 * n))
        if norm == "ortho":
            m = m * math.sqrt(1 / (2 * n))
            m[0] = m[0] / math.sqrt(2)
    elif kind == 3:
        m = 2 * torch.cos(math.pi * j * (2 * k + 1) / (2 * n))
        m[:, 0] = 1.0
        if norm == "ortho":
            m = m * math.sqrt(1 / (2 * n))
            m[:, 0] = math.sqrt(1 / n)
    elif kind == 4:
        m = 2 * torch.cos(math.pi * (2 * k + 1) * (2 * j + 1) / (4 * n))
        if norm == "ortho":
            m = m * math.sqrt(1 / (2 * n))
    elif kind == 1:
        if n < 2:
            raise ValueError("dct type 1 needs at least 2 points")
        m = 2 * torch.cos(math.pi * k * j / (n - 1))
        m[:, 0] = 1.0
        m[:, -1] = (-1.0) ** torch.arange(n, dtype=torch.float64)
        if norm == "ortho":
            raise NotImplementedError("dct type 1 with norm='ortho' is not provided")
    else:
        raise ValueError("dct type must be 1, 2, 3 or 4, but got %r" % (kind,))
    return m


def _apply(x, kind, n, axis, norm):
    t = x.as_subclass(torch.Tensor) if isinstance(x, torch.Tensor) else torch.as_tensor(x)
    if not t.is_floating_point():
        t = t.float()
    t = t.movedim(axis, -1)
    size = t.shape[-1] if n is None else int(n)
    if size > t.shape[-1]:
        t = torch.nn.functional.pad(t, (0, size - t.shape[-1]))
    t = t[..., :size]
    out = (t.double() @ _matrix(size, kind, norm).t()).to(t.dtype)
    return _wrap_out(out.movedim(-1, axis))


def dct(x, type=2, n=None, axis=-1, norm=None):  # noqa: A002
    return _apply(x, type, n, axis, norm)


def idct(x, type=2, n=None, axis=-1, norm=None):  # noqa: A002
    inv = {1: 1, 2: 3, 3: 2, 4: 4}[type]
    out = _apply(x, inv, n, axis, norm)
    if norm == "ortho":
        return out
    size = out.shape[axis]
    return _wrap_out(out.as_subclass(torch.Tensor) / (2 * (size - 1) if type == 1 else 2 * size))
