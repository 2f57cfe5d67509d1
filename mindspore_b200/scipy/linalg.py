"""Dense linear algebra (python/mindspore/scipy/linalg.py: block_diag, inv, cho_factor, cholesky, cho_solve,
solve_triangular, eigh, lu_factor, lu, det)."""
from __future__ import annotations

import torch

from ..ops.primitive import _wrap_out

__all__ = ["block_diag", "solve_triangular", "inv", "cho_factor", "cholesky", "cho_solve", "eigh", "lu_factor", "lu",
           "det"]


def _t(x):
    return x if isinstance(x, torch.Tensor) else torch.as_tensor(x)


def block_diag(*arrs):
    mats = [_t(a).reshape(1, -1) if _t(a).dim() < 2 else _t(a) for a in arrs]
    return _wrap_out(torch.block_diag(*mats))


def solve_triangular(a, b, trans=0, lower=False, unit_diagonal=False, overwrite_b=False, debug=None, check_finite=True):
    a, b = _t(a), _t(b)
    if trans in (1, "T"):
        a, lower = a.transpose(-1, -2), not lower
    elif trans in (2, "C"):
        a, lower = a.conj().transpose(-1, -2), not lower
    vec = b.dim() == a.dim() - 1
    rhs = b.unsqueeze(-1) if vec else b
    x = torch.linalg.solve_triangular(a, rhs, upper=not lower, unitriangular=unit_diagonal)
    return _wrap_out(x.squeeze(-1) if vec else x)


def inv(a, overwrite_a=False, check_finite=True):
    return _wrap_out(torch.linalg.inv(_t(a)))


def cho_factor(a, lower=False, overwrite_a=False, check_finite=True):
    return _wrap_out(torch.linalg.cholesky(_t(a), upper=not lower)), lower


def cholesky(a, lower=False, overwrite_a=False, check_finite=True):
    return _wrap_out(torch.linalg.cholesky(_t(a), upper=not lower))


def cho_solve(c_and_lower, b, overwrite_b=False, check_finite=True):
    c, lower = c_and_lower
    b = _t(b)
    vec = b.dim() == 1
    x = torch.cholesky_solve(b.unsqueeze(-1) if vec else b, _t(c), upper=not lower)
    return _wrap_out(x.squeeze(-1) if vec else x)


def eigh(a, b=None, lower=True, eigvals_only=False, overwrite_a=False, overwrite_b=False, turbo=True, eigvals=None,
         _type=1, check_finite=True):
    if b is not None:
        raise NotImplementedError("generalised eigenproblems are not supported")
    w, v = torch.linalg.eigh(_t(a), UPLO="L" if lower else "U")
    if eigvals is not None:
        lo, hi = eigvals
        w, v = w[..., lo:hi + 1], v[..., lo:hi + 1]
    return _wrap_out(w) if eigvals_only else (_wrap_out(w), _wrap_out(v))


def lu_factor(a, overwrite_a=False, check_finite=True):
    lu_, piv = torch.linalg.lu_factor(_t(a))
    return _wrap_out(lu_), _wrap_out(piv - 1)


def lu(a, permute_l=False, overwrite_a=False, check_finite=True):
    p, l, u = torch.linalg.lu(_t(a))
    if permute_l:
        return _wrap_out(p @ l), _wrap_out(u)
    return _wrap_out(p), _wrap_out(l), _wrap_out(u)


def det(a, overwrite_a=False, check_finite=True):
    return _wrap_out(torch.linalg.det(_t(a)))
