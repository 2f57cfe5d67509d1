"""``minimize`` (BFGS / L-BFGS with a backtracking Armijo line search) and ``line_search``
(python/mindspore/scipy/optimize/{minimize.py, _bfgs.py, _lbfgs.py, line_search.py})."""
from __future__ import annotations

from collections import namedtuple

import torch

from ..ops.primitive import _wrap_out

__all__ = ["minimize", "line_search", "OptimizeResults", "linear_sum_assignment"]

OptimizeResults = namedtuple("OptimizeResults", "x success status fun jac hess_inv nfev njev nit")
LineSearchResults = namedtuple("LineSearchResults", "a_k f_k g_k nfev ngev failed")


def _value_and_grad(fun, x, args):
    x = x.detach().clone().requires_grad_(True)
    with torch.enable_grad():
        f = fun(x, *args)
        f = f if isinstance(f, torch.Tensor) else torch.as_tensor(f)
        (g,) = torch.autograd.grad(f, x)
    return f.detach(), g.detach()


def line_search(f, xk, pk, jac=None, gfk=None, old_fval=None, old_old_fval=None, c1=1e-4, c2=0.9, maxiter=20, args=()):
    """Step length along ``pk`` satisfying the Armijo condition (and the curvature condition when reachable)."""
    xk, pk = torch.as_tensor(xk).float(), torch.as_tensor(pk).float()
    f0, g0 = _value_and_grad(f, xk, args) if old_fval is None or gfk is None else (torch.as_tensor(old_fval), torch.as_tensor(gfk))
    slope = torch.dot(g0.reshape(-1), pk.reshape(-1))
    a, nfev = 1.0, 0
    best = None
    for _ in range(maxiter):
        fa, ga = _value_and_grad(f, xk + a * pk, args)
        nfev += 1
        if fa <= f0 + c1 * a * slope:
            best = (a, fa, ga)
            if torch.dot(ga.reshape(-1), pk.reshape(-1)).abs() <= c2 * slope.abs():
                break
            if best is not None:
                break
        a *= 0.5
    if best is None:
        return LineSearchResults(_wrap_out(torch.tensor(0.0)), _wrap_out(f0), _wrap_out(g0), nfev, nfev, True)
    return LineSearchResults(_wrap_out(torch.tensor(best[0])), _wrap_out(best[1]), _wrap_out(best[2]), nfev, nfev, False)


def minimize(func, x0, args=(), method="BFGS", jac=None, hess=None, hessp=None, bounds=None, constraints=(), tol=None,
             callback=None, options=None):
    if method is None:
        method = "BFGS"
    m = method.upper().replace("-", "")
    if m not in ("BFGS", "LBFGS"):
        raise ValueError("Method %s not recognized" % method)
    opt = dict(options or {})
    maxiter = int(opt.get("maxiter", 200 * max(1, torch.as_tensor(x0).numel())))
    gtol = float(opt.get("gtol", tol if tol is not None else 1e-5))
    history = int(opt.get("history_size", 10))
    x = torch.as_tensor(x0).detach().float().clone()
    shape = x.shape
    f, g = _value_and_grad(func, x, args)
    n = x.numel()
    H = torch.eye(n)
    s_hist, y_hist = [], []
    nfev, nit, status = 1, 0, 0
    while nit < maxiter:
        if float(g.abs().max()) <= gtol:
            break
        gv = g.reshape(-1)
        if m == "BFGS":
            p = -(H @ gv)
        else:                                            # two-loop recursion
            q, alphas = gv.clone(), []
            for s, y in reversed(list(zip(s_hist, y_hist))):
                a = torch.dot(s, q) / torch.dot(y, s)
                alphas.append(a)
                q = q - a * y
            if s_hist:
                q = q * (torch.dot(s_hist[-1], y_hist[-1]) / torch.dot(y_hist[-1], y_hist[-1]))
            for (s, y), a in zip(zip(s_hist, y_hist), reversed(alphas)):
                b = torch.dot(y, q) / torch.dot(y, s)
                q = q + (a - b) * s
            p = -q
        step, slope, ok = 1.0, float(torch.dot(gv, p)), False
        if slope >= 0:                                    # not a descent direction: restart from steepest descent
            p, H, s_hist, y_hist = -gv, torch.eye(n), [], []
            slope = float(torch.dot(gv, p))
        for _ in range(40):
            f_new, g_new = _value_and_grad(func, (x.reshape(-1) + step * p).reshape(shape), args)
            nfev += 1
            if float(f_new) <= float(f) + 1e-4 * step * slope:
                ok = True
                break
            step *= 0.5
        if not ok:
            status = 3
            break
        if step == 1.0:                                   # a full step was accepted at once: see whether a longer one is better
            for _ in range(10):
                f_try, g_try = _value_and_grad(func, (x.reshape(-1) + 2 * step * p).reshape(shape), args)
                nfev += 1
                if float(f_try) < float(f_new) and float(f_try) <= float(f) + 1e-4 * 2 * step * slope:
                    step, f_new, g_new = 2 * step, f_try, g_try
                else:
                    break
        s = step * p
        y = g_new.reshape(-1) - gv
        sy = float(torch.dot(s, y))
        if sy > 1e-12:
            if m == "BFGS":
                rho = 1.0 / sy
                I = torch.eye(n)
                H = (I - rho * torch.outer(s, y)) @ H @ (I - rho * torch.outer(y, s)) + rho * torch.outer(s, s)
            else:
                s_hist.append(s)
                y_hist.append(y)
                if len(s_hist) > history:
                    s_hist.pop(0)
                    y_hist.pop(0)
        x, f, g = (x.reshape(-1) + s).reshape(shape), f_new, g_new
        nit += 1
        if callback is not None:
            callback(_wrap_out(x))
    else:
        status = 1
    success = status == 0 and float(g.abs().max()) <= gtol
    return OptimizeResults(_wrap_out(x), success, status, _wrap_out(f), _wrap_out(g),
                           _wrap_out(H) if m == "BFGS" else None, nfev, nfev, nit)


def linear_sum_assignment(cost_matrix, maximize, dimension_limit=None):
    """Rows and columns of the minimum- (or maximum-) cost assignment of a rectangular cost matrix;
    ``dimension_limit`` restricts the problem to the first columns.  Solved on the host (Jonker-Volgenant, SciPy)."""
    import scipy.optimize as _so
    c = cost_matrix.detach().as_subclass(torch.Tensor).cpu() if isinstance(cost_matrix, torch.Tensor) else \
        torch.as_tensor(cost_matrix)
    if dimension_limit is not None:
        lim = int(dimension_limit)
        if lim > c.shape[1]:
            raise ValueError("dimension_limit %d exceeds the %d columns of the cost matrix" % (lim, c.shape[1]))
        c = c[:, :lim]
    mx = bool(maximize) if not isinstance(maximize, torch.Tensor) else bool(maximize.item())
    rows, cols = _so.linear_sum_assignment(c.numpy(), maximize=mx)
    return _wrap_out(torch.as_tensor(rows, dtype=torch.int64)), _wrap_out(torch.as_tensor(cols, dtype=torch.int64))
