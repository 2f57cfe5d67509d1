"""Optimizers beyond the first-order dense family: ``LazyAdam`` (sparse rows), ``AdamOffload`` (state in pinned host
memory), ``THOR`` (Kronecker-factored second order) and the AdaSum wrappers.

Parity: python/mindspore/nn/optim/{lazyadam.py, adam.py (AdamOffload :1180), thor.py, adasum.py}."""
from __future__ import annotations

import math

import torch

from ..ops.primitive import _wrap_out
from .cell import Cell
from .optim import Adam, Momentum, Optimizer, _to_plain

__all__ = ["opt_init_args_register", "ConvertNetUtils", "ConvertModelUtils", "LazyAdam", "AdamOffload", "THOR", "thor", "AdaSumByGradWrapCell", "AdaSumByDeltaWeightWrapCell"]


class LazyAdam(Adam):
    """Adam that, for a gradient with few non-zero rows (embedding tables), updates only those rows' moments and
    weights; dense gradients take the ordinary path."""

    def construct(self, gradients):
        gradients = self._prep(gradients)
        lrs = self._lrs()
        t = self._step() + 1
        lr_scale = math.sqrt(1 - self.beta2 ** t) / (1 - self.beta1 ** t)
        with torch.no_grad():
            for p, g, m, v, lr in zip(self._parameters, gradients, self.moment1, self.moment2, lrs):
                pt, mt, vt, gt = _to_plain(p), _to_plain(m), _to_plain(v), _to_plain(g).to(m.dtype)
                rows = None
                if gt.dim() >= 2:
                    nz = gt.reshape(gt.shape[0], -1).ne(0).any(1)
                    if int(nz.sum()) * 4 < gt.shape[0]:
                        rows = nz.nonzero().squeeze(1)
                if rows is None:
                    mt.mul_(self.beta1).add_(gt, alpha=1 - self.beta1)
                    vt.mul_(self.beta2).addcmul_(gt, gt, value=1 - self.beta2)
                    pt.sub_((lr * lr_scale * mt / (vt.sqrt() + self.eps)).to(pt.dtype))
                else:
                    gr = gt[rows]
                    mr = mt[rows] * self.beta1 + gr * (1 - self.beta1)
                    vr = vt[rows] * self.beta2 + gr * gr * (1 - self.beta2)
                    mt[rows], vt[rows] = mr, vr
                    pt[rows] = pt[rows] - (lr * lr_scale * mr / (vr.sqrt() + self.eps)).to(pt.dtype)
        self._advance()
        return True


class AdamOffload(Adam):
    """Adam whose moments live in (pinned) host memory: the gradient is copied down, the moments are updated on the
    CPU, and only the weight update travels back.  Trades step time for 8 bytes per parameter of device memory."""

    def __init__(self, params, learning_rate=1e-3, beta1=0.9, beta2=0.999, eps=1e-8, use_locking=False,
                 use_nesterov=False, weight_decay=0.0, loss_scale=1.0):
        super().__init__(params, learning_rate, beta1, beta2, eps, use_locking, use_nesterov, weight_decay, loss_scale)
        pin = torch.cuda.is_available()
        self._host_m = [torch.zeros(p.shape, dtype=torch.float32, pin_memory=pin) for p in self._parameters]
        self._host_v = [torch.zeros(p.shape, dtype=torch.float32, pin_memory=pin) for p in self._parameters]
        self.moment1 = self.moment2 = None           # no device-side state

    def construct(self, gradients):
        gradients = self._prep(gradients)
        lrs = self._lrs()
        t = self._step() + 1
        lr_scale = math.sqrt(1 - self.beta2 ** t) / (1 - self.beta1 ** t)
        with torch.no_grad():
            for p, g, m, v, lr in zip(self._parameters, gradients, self._host_m, self._host_v, lrs):
                pt = _to_plain(p)
                gh = _to_plain(g).detach().to("cpu", torch.float32)
                m.mul_(self.beta1).add_(gh, alpha=1 - self.beta1)
                v.mul_(self.beta2).addcmul_(gh, gh, value=1 - self.beta2)
                num = (self.beta1 * m + (1 - self.beta1) * gh) if self.use_nesterov else m
                upd = lr * lr_scale * num / (v.sqrt() + self.eps)
                pt.sub_(upd.to(pt.device, pt.dtype, non_blocking=True))
        self._advance()
        return True


class THOR(Momentum):
    """Second-order optimizer with Kronecker-factored curvature for ``nn.Dense`` layers: for y = x W^T the Fisher
    block is approximated by A (x) G with A = E[x x^T], G = E[dy dy^T]; the weight gradient is preconditioned as
    (G + sqrt(damping) I)^-1 dW (A + sqrt(damping) I)^-1 and handed to Momentum.  The factors are refreshed every
    ``frequency`` steps from activations / output gradients captured by hooks; other parameters get plain Momentum."""

    def __init__(self, net, learning_rate, damping, momentum, weight_decay=0.0, loss_scale=1.0, batch_size=32,
                 use_nesterov=False, decay_filter=None, split_indices=None, enable_clip_grad=False, frequency=100):
        super().__init__(net.trainable_params(), learning_rate, momentum, weight_decay, loss_scale, use_nesterov)
        from .layer import Dense
        self.damping, self.frequency, self.enable_clip_grad = damping, max(1, int(frequency)), enable_clip_grad
        self._layers = []
        index = {id(p): i for i, p in enumerate(self._parameters)}
        for _, cell in net.cells_and_names():
            if isinstance(cell, Dense) and id(cell.weight) in index:
                rec = {"idx": index[id(cell.weight)], "A": None, "G": None, "Ainv": None, "Ginv": None}
                cell.register_forward_pre_hook(self._make_fwd(rec))
                cell.register_backward_hook(self._make_bwd(rec))
                self._layers.append(rec)

    def _refresh(self):
        return self._step_host % self.frequency == 0

    def _make_fwd(self, rec):
        def hook(cell, inputs):
            if cell.training and self._refresh():
                x = _to_plain(inputs[0]).detach().float().reshape(-1, inputs[0].shape[-1])
                rec["A"] = x.t() @ x / x.shape[0]
        return hook

    def _make_bwd(self, rec):
        def hook(cell, grad_in, grad_out):
            if self._refresh():
                g = _to_plain(grad_out).detach().float().reshape(-1, grad_out.shape[-1])
                rec["G"] = g.t() @ g * g.shape[0]          # undo the 1/batch of a mean loss
        return hook

    def _damp(self, step):
        d = self.damping
        if callable(d):
            return float(d(step))
        if isinstance(d, torch.Tensor) and d.numel() > 1:
            return float(d.reshape(-1)[min(step, d.numel() - 1)])
        return float(d)

    def construct(self, gradients=None):
        if gradients is not None and self._layers:
            gradients = list(gradients)
            lam = math.sqrt(self._damp(self._step_host))
            for rec in self._layers:
                if rec["A"] is not None and rec["G"] is not None and (self._refresh() or rec["Ainv"] is None):
                    eye_a = torch.eye(rec["A"].shape[0], device=rec["A"].device)
                    eye_g = torch.eye(rec["G"].shape[0], device=rec["G"].device)
                    rec["Ainv"] = torch.linalg.inv(rec["A"] + lam * eye_a)
                    rec["Ginv"] = torch.linalg.inv(rec["G"] + lam * eye_g)
                if rec["Ainv"] is None:
                    continue
                g = _to_plain(gradients[rec["idx"]])
                pre = rec["Ginv"] @ g.float() @ rec["Ainv"]
                if self.enable_clip_grad:
                    pre = pre * min(1.0, 1.0 / (float(pre.norm()) + 1e-12))
                gradients[rec["idx"]] = _wrap_out(pre.to(g.dtype))
            gradients = tuple(gradients)
        return super().construct(gradients)


def thor(net, learning_rate, damping, momentum, weight_decay=0.0, loss_scale=1.0, batch_size=32, use_nesterov=False,
         decay_filter=None, split_indices=None, enable_clip_grad=False, frequency=100):
    return THOR(net, learning_rate, damping, momentum, weight_decay, loss_scale, batch_size, use_nesterov, decay_filter,
                split_indices, enable_clip_grad, frequency)


# ------------------------------------------------------------------------------------------------ AdaSum
def _adasum_pair(a, b):
    """AdaSum of two vectors: a (1 - a.b / 2|a|^2) + b (1 - a.b / 2|b|^2) - orthogonal parts add, parallel parts
    average."""
    dot = torch.sum(a.float() * b.float())
    na, nb = torch.sum(a.float() ** 2).clamp_min(1e-30), torch.sum(b.float() ** 2).clamp_min(1e-30)
    return (a.float() * (1 - dot / (2 * na)) + b.float() * (1 - dot / (2 * nb))).to(a.dtype)


def _adasum_allreduce(t, group_ranks, rank):
    """Recursive-halving AdaSum across ``group_ranks`` (size a power of two): log2(n) exchanges with the partner at
    distance 1, 2, 4, ..; after the last round every rank holds the same combination."""
    import torch.distributed as dist
    n = len(group_ranks)
    me = group_ranks.index(rank)
    out = t.clone()
    d = 1
    while d < n:
        partner = group_ranks[me ^ d]
        other = torch.empty_like(out)
        ops = [dist.P2POp(dist.isend, out.contiguous(), partner), dist.P2POp(dist.irecv, other, partner)]
        for w in dist.batch_isend_irecv(ops):
            w.wait()
        first, second = (out, other) if (me & d) == 0 else (other, out)
        out = _adasum_pair(first, second)
        d *= 2
    return out


class _AdaSumWrap(Cell):
    _by_delta = False

    def __init__(self, optimizer):
        super().__init__(auto_prefix=False)
        if not isinstance(optimizer, Optimizer):
            raise TypeError("AdaSum wrappers take an Optimizer, got %s" % type(optimizer).__name__)
        self.optimizer = optimizer
        from ..communication import management as M
        self._world = M.get_group_size() if M.GlobalComm.INITED else 1
        self._rank = M.get_rank() if M.GlobalComm.INITED else 0
        if self._world & (self._world - 1):
            raise RuntimeError("AdaSum needs a power-of-two number of devices, got %d" % self._world)

    def _combine(self, t):
        if self._world == 1:
            return t
        return _adasum_allreduce(_to_plain(t), list(range(self._world)), self._rank)

    def construct(self, grads):
        if not self._by_delta:
            grads = tuple(_wrap_out(self._combine(g)) for g in grads)
            return self.optimizer(grads)
        params = self.optimizer._parameters
        before = [_to_plain(p).detach().clone() for p in params]
        res = self.optimizer(grads)
        with torch.no_grad():
            for p, old in zip(params, before):
                delta = self._combine(_to_plain(p) - old)
                _to_plain(p).copy_(old + delta)
        return res


class AdaSumByGradWrapCell(_AdaSumWrap):
    """Combines the gradients of the data-parallel ranks with AdaSum (instead of the mean) before the update."""
    _by_delta = False


class AdaSumByDeltaWeightWrapCell(_AdaSumWrap):
    """Runs the local update first and combines the resulting weight deltas with AdaSum."""
    _by_delta = True


class ConvertNetUtils:
    """Prepares a network for THOR.  The reference swaps Dense / Conv2d / Embedding cells for variants that record
    the Kronecker factors; here ``THOR`` attaches hooks to the ordinary cells, so the network is returned as is."""

    def convert_to_thor_net(self, net):
        return net


class ConvertModelUtils:
    @staticmethod
    def convert_to_thor_model(model, network, loss_fn=None, optimizer=None, metrics=None, amp_level="O0",
                              loss_scale_manager=None, keep_batchnorm_fp32=False):
        """Rebuilds ``model`` around ``network`` / ``optimizer`` (a ``THOR`` instance); other optimizers pass through."""
        from ..train.model import Model
        if not isinstance(optimizer, THOR):
            return model
        return Model(network, loss_fn, optimizer, metrics, amp_level=amp_level, loss_scale_manager=loss_scale_manager)


def opt_init_args_register(fn):
    """Decorator for an optimizer's ``__init__``: records the constructor arguments (tensors and parameter lists
    left out) as ``self.init_args``, which checkpoint tools and ``boost`` read back.  Parity:
    nn/optim/optimizer.py (opt_init_args_register)."""
    import functools
    import inspect

    @functools.wraps(fn)
    def deco(self, *args, **kwargs):
        bound = inspect.signature(fn).bind(self, *args, **kwargs)
        bound.apply_defaults()
        keep = {}
        for k, v in list(bound.arguments.items())[1:]:
            if k in ("params", "parameters") or isinstance(v, torch.Tensor):
                continue
            keep[k] = v
        object.__setattr__(self, "init_args", keep)
        return fn(self, *args, **kwargs)
    return deco
