"""Iterative solvers ``sparse.linalg.cg`` / ``gmres`` / ``bicgstab`` for ``A x = b`` with ``A`` a dense tensor, a
``CSRTensor`` or a function computing ``A @ v`` (python/mindspore/scipy/sparse/linalg.py)."""
from __future__ import annotations

import types

import torch

from ..ops.primitive import _wrap_out

__all__ = ["linalg"]


def _matvec(A):
    if callable(A) and not isinstance(A, torch.Tensor):
        return lambda v: torch.as_tensor(A(v))
    if hasattr(A, "mv") and hasattr(A, "indptr"):
        return lambda v: torch.as_tensor(A.mv(v)).reshape(-1)
    M = torch.as_tensor(A)
    return lambda v: M @ v


def cg(A, b, x0=None, tol=1e-5, atol=0.0, maxiter=None, M=None, callback=None):
    mv, pre = _matvec(A), (_matvec(M) if M is not None else (lambda v: v))
    b = torch.as_tensor(b).float().reshape(-1)
    x = torch.zeros_like(b) if x0 is None else torch.as_tensor(x0).float().reshape(-1).clone()
    r = b - mv(x)
    z = pre(r)
    p = z.clone()
    rz = torch.dot(r, z)
    limit = max(float(tol) * float(b.norm()), float(atol))
    maxiter = maxiter or 10 * b.numel()
    info = maxiter
    for k in range(maxiter):
        if float(r.norm()) <= limit:
            info = 0
            break
        Ap = mv(p)
        alpha = rz / torch.dot(p, Ap)
        x = x + alpha * p
        r = r - alpha * Ap
        z = pre(r)
        rz_new = torch.dot(r, z)
        p = z + (rz_new / rz) * p
        rz = rz_new
        if callback is not None:
            callback(_wrap_out(x))
    else:
        info = 0 if float(r.norm()) <= limit else maxiter
    return _wrap_out(x), info


def bicgstab(A, b, x0=None, tol=1e-5, atol=0.0, maxiter=None, M=None, callback=None):
    mv, pre = _matvec(A), (_matvec(M) if M is not None else (lambda v: v))
    b = torch.as_tensor(b).float().reshape(-1)
    x = torch.zeros_like(b) if x0 is None else torch.as_tensor(x0).float().reshape(-1).clone()
    r = b - mv(x)
    r0 = r.clone()
    rho = alpha = omega = torch.tensor(1.0)
    v = p = torch.zeros_like(b)
    limit = max(float(tol) * float(b.norm()), float(atol))
    maxiter = maxiter or 10 * b.numel()
    for _ in range(maxiter):
        if float(r.norm()) <= limit:
            return _wrap_out(x), 0
        rho_new = torch.dot(r0, r)
        beta = (rho_new / rho) * (alpha / omega)
        p = r + beta * (p - omega * v)
        ph = pre(p)
        v = mv(ph)
        alpha = rho_new / torch.dot(r0, v)
        s = r - alpha * v
        if float(s.norm()) <= limit:
            return _wrap_out(x + alpha * ph), 0
        sh = pre(s)
        t = mv(sh)
        omega = torch.dot(t, s) / torch.dot(t, t)
        x = x + alpha * ph + omega * sh
        r = s - omega * t
        rho = rho_new
        if callback is not None:
            callback(_wrap_out(x))
    return _wrap_out(x), 0 if float(r.norm()) <= limit else maxiter


def gmres(A, b, x0=None, tol=1e-5, atol=0.0, restart=20, maxiter=None, M=None, callback=None, solve_method="batched"):
    mv, pre = _matvec(A), (_matvec(M) if M is not None else (lambda v: v))
    b = torch.as_tensor(b).float().reshape(-1)
    n = b.numel()
    x = torch.zeros_like(b) if x0 is None else torch.as_tensor(x0).float().reshape(-1).clone()
    restart = min(int(restart), n)
    limit = max(float(tol) * float(b.norm()), float(atol))
    maxiter = maxiter or 10 * n
    for _ in range(maxiter):
        r = pre(b - mv(x))
        beta = r.norm()
        if float((b - mv(x)).norm()) <= limit:
            return _wrap_out(x), 0
        Q = torch.zeros(n, restart + 1)
        Hm = torch.zeros(restart + 1, restart)
        Q[:, 0] = r / beta
        k_used = restart
        for k in range(restart):
            w = pre(mv(Q[:, k]))
            for j in range(k + 1):
                Hm[j, k] = torch.dot(Q[:, j], w)
                w = w - Hm[j, k] * Q[:, j]
            Hm[k + 1, k] = w.norm()
            if float(Hm[k + 1, k]) < 1e-12:
                k_used = k + 1
                break
            Q[:, k + 1] = w / Hm[k + 1, k]
        e1 = torch.zeros(k_used + 1)
        e1[0] = beta
        y = torch.linalg.lstsq(Hm[:k_used + 1, :k_used], e1.unsqueeze(-1)).solution.squeeze(-1)
        x = x + Q[:, :k_used] @ y
        if callback is not None:
            callback(_wrap_out(x))
    return _wrap_out(x), 0 if float((b - mv(x)).norm()) <= limit else maxiter


linalg = types.SimpleNamespace(cg=cg, gmres=gmres, bicgstab=bicgstab)
