"""Loss cells.  Parity: mindspore/python/mindspore/nn/loss/loss.py (LossBase and the common losses)."""
from __future__ import annotations

import torch
import torch.nn.functional as F

from ..ops import fused
from ..ops.primitive import _wrap_out
from .cell import Cell


class LossBase(Cell):
    def __init__(self, reduction="mean"):
        super().__init__()
        if reduction not in ("mean", "sum", "none"):
            raise ValueError("For '%s', the 'reduction' must be in ['mean', 'sum', 'none'], but got %r."
                             % (self.cls_name if hasattr(self, "cls_name") else type(self).__name__, reduction))
        self.reduction = reduction

    def get_loss(self, x, weights=1.0):
        x = x.float() * weights
        if self.reduction == "mean":
            return _wrap_out(x.mean())
        if self.reduction == "sum":
            return _wrap_out(x.sum())
        return _wrap_out(x)

    def construct(self, logits, labels):
        raise NotImplementedError


_Loss = LossBase


class SoftmaxCrossEntropyWithLogits(LossBase):
    def __init__(self, sparse=False, reduction="none"):
        super().__init__(reduction)
        self.sparse = sparse

    def construct(self, logits, labels):
        if self.sparse:
            if self.reduction == "mean" and logits.is_cuda and logits.dim() == 2:
                return _wrap_out(fused.softmax_cross_entropy(logits, labels))
            loss = F.cross_entropy(logits.float(), labels.long(), reduction="none")
        else:
            loss = -(labels.float() * torch.log_softmax(logits.float(), -1)).sum(-1)
        return self.get_loss(loss)


class CrossEntropyLoss(LossBase):
    def __init__(self, weight=None, ignore_index=-100, reduction="mean", label_smoothing=0.0):
        super().__init__(reduction)
        if label_smoothing < 0 or label_smoothing > 1:
            raise ValueError("label_smoothing must be in [0, 1]")
        self.weight, self.ignore_index, self.label_smoothing = weight, ignore_index, label_smoothing

    def construct(self, logits, labels):
        if self.weight is None and self.reduction == "mean" and self.label_smoothing == 0.0 and logits.is_cuda \
                and not labels.is_floating_point() and logits.dim() == 2:
            return _wrap_out(fused.softmax_cross_entropy(logits, labels, self.ignore_index))
        tgt = labels if labels.is_floating_point() else labels.long()
        return _wrap_out(F.cross_entropy(logits.float(), tgt, self.weight, ignore_index=self.ignore_index,
                                         reduction=self.reduction, label_smoothing=self.label_smoothing))


class NLLLoss(LossBase):
    def __init__(self, weight=None, ignore_index=-100, reduction="mean"):
        super().__init__(reduction)
        self.weight, self.ignore_index = weight, ignore_index

    def construct(self, logits, labels):
        return _wrap_out(F.nll_loss(logits, labels.long(), self.weight, ignore_index=self.ignore_index,
                                    reduction=self.reduction))


class MSELoss(LossBase):
    def construct(self, logits, labels):
        return self.get_loss((logits - labels) ** 2)


class L1Loss(LossBase):
    def construct(self, logits, labels):
        return self.get_loss((logits - labels).abs())


MAELoss = L1Loss


class RMSELoss(LossBase):
    def construct(self, logits, labels):
        return _wrap_out(torch.sqrt(((logits - labels) ** 2).float().mean()))


class SmoothL1Loss(LossBase):
    def __init__(self, beta=1.0, reduction="none"):
        super().__init__(reduction)
        self.beta = beta

    def construct(self, logits, labels):
        return _wrap_out(F.smooth_l1_loss(logits, labels, beta=self.beta, reduction=self.reduction))


class HuberLoss(LossBase):
    def __init__(self, reduction="mean", delta=1.0):
        super().__init__(reduction)
        self.delta = delta

    def construct(self, logits, labels):
        return _wrap_out(F.huber_loss(logits, labels, delta=self.delta, reduction=self.reduction))


class BCELoss(LossBase):
    def __init__(self, weight=None, reduction="mean"):
        super().__init__(reduction)
        self.weight = weight

    def construct(self, logits, labels):
        return _wrap_out(F.binary_cross_entropy(logits, labels, self.weight, reduction=self.reduction))


class BCEWithLogitsLoss(LossBase):
    def __init__(self, reduction="mean", weight=None, pos_weight=None):
        super().__init__(reduction)
        self.weight, self.pos_weight = weight, pos_weight

    def construct(self, logits, labels):
        return _wrap_out(F.binary_cross_entropy_with_logits(logits, labels, self.weight, pos_weight=self.pos_weight,
                                                            reduction=self.reduction))


class KLDivLoss(LossBase):
    def construct(self, logits, labels):
        red = self.reduction
        return _wrap_out(F.kl_div(logits, labels, reduction=red if red != "mean" else "mean"))


class CosineEmbeddingLoss(LossBase):
    def __init__(self, margin=0.0, reduction="mean"):
        super().__init__(reduction)
        self.margin = margin

    def construct(self, x1, x2, y):
        return _wrap_out(F.cosine_embedding_loss(x1, x2, y, self.margin, reduction=self.reduction))


class FocalLoss(LossBase):
    def __init__(self, weight=None, gamma=2.0, reduction="mean"):
        super().__init__(reduction)
        self.gamma, self.weight = gamma, weight

    def construct(self, logits, labels):
        logp = torch.log_softmax(logits.float(), 1)
        if labels.dim() == logits.dim() and labels.shape[1] == 1:
            labels = labels.squeeze(1)
        lp = logp.gather(1, labels.long().unsqueeze(1)).squeeze(1)
        loss = -((1 - lp.exp()) ** self.gamma) * lp
        if self.weight is not None:
            loss = loss * self.weight[labels.long()]
        return self.get_loss(loss)


class DiceLoss(LossBase):
    def __init__(self, smooth=1e-5):
        super().__init__()
        self.smooth = smooth

    def construct(self, logits, labels):
        inter = (logits * labels).sum()
        union = (logits * logits).sum() + (labels * labels).sum()
        return _wrap_out(1 - (2 * inter + self.smooth) / (union + self.smooth))


class CTCLoss(LossBase):
    def __init__(self, blank=0, reduction="mean", zero_infinity=False):
        super().__init__(reduction)
        self.blank, self.zero_infinity = blank, zero_infinity

    def construct(self, log_probs, targets, input_lengths, target_lengths):
        return _wrap_out(F.ctc_loss(log_probs, targets, input_lengths, target_lengths, self.blank, self.reduction,
                                    self.zero_infinity))


class MarginRankingLoss(LossBase):
    def __init__(self, margin=0.0, reduction="mean"):
        super().__init__(reduction)
        self.margin = margin

    def construct(self, x1, x2, y):
        return _wrap_out(F.margin_ranking_loss(x1, x2, y, self.margin, reduction=self.reduction))


class TripletMarginLoss(LossBase):
    def __init__(self, p=2, swap=False, eps=1e-6, reduction="mean", margin=1.0):
        super().__init__(reduction)
        self.p, self.swap, self.eps, self.margin = p, swap, eps, margin

    def construct(self, a, pos, neg):
        return _wrap_out(F.triplet_margin_loss(a, pos, neg, self.margin, self.p, self.eps, self.swap,
                                               reduction=self.reduction))


# ------------------------------------------------------------------------------------------------ further losses
class SoftMarginLoss(LossBase):
    def construct(self, logits, labels):
        return self.get_loss(torch.log1p(torch.exp(-labels.float() * logits.float())))


class HingeEmbeddingLoss(LossBase):
    def __init__(self, margin=1.0, reduction="mean"):
        super().__init__(reduction)
        self.margin = float(margin)

    def construct(self, logits, labels):
        x, y = logits.float(), labels.float()
        return self.get_loss(torch.where(y > 0, x, (self.margin - x).clamp_min(0)))


class PoissonNLLLoss(LossBase):
    def __init__(self, log_input=True, full=False, eps=1e-8, reduction="mean"):
        super().__init__(reduction)
        self.log_input, self.full, self.eps = log_input, full, eps

    def construct(self, input, target):      # noqa: A002
        return self.get_loss(torch.nn.functional.poisson_nll_loss(input.float(), target.float(), self.log_input,
                                                                   self.full, eps=self.eps, reduction="none"))


class GaussianNLLLoss(LossBase):
    def __init__(self, full=False, eps=1e-6, reduction="mean"):
        super().__init__(reduction)
        self.full, self.eps = full, eps

    def construct(self, logits, labels, var):
        return self.get_loss(torch.nn.functional.gaussian_nll_loss(logits.float(), labels.float(), var.float(),
                                                                    self.full, self.eps, reduction="none"))


class MultiLabelSoftMarginLoss(LossBase):
    def __init__(self, weight=None, reduction="mean"):
        super().__init__(reduction)
        self.weight = weight

    def construct(self, x, target):
        x, t = x.float(), target.float()
        loss = -(t * torch.nn.functional.logsigmoid(x) + (1 - t) * torch.nn.functional.logsigmoid(-x))
        if self.weight is not None:
            loss = loss * self.weight
        return self.get_loss(loss.mean(-1))


class MultilabelMarginLoss(LossBase):
    def construct(self, x, target):
        loss = torch.nn.functional.multilabel_margin_loss(x.float(), target.long(), reduction="none")
        return self.get_loss(loss)


class MultiMarginLoss(LossBase):
    def __init__(self, p=1, margin=1.0, reduction="mean", weight=None):
        super().__init__(reduction)
        self.p, self.margin, self.weight = p, margin, weight

    def construct(self, x, target, weight=None):
        w = weight if weight is not None else self.weight
        loss = torch.nn.functional.multi_margin_loss(x.float(), target.long(), self.p, self.margin,
                                                     w.float() if w is not None else None, reduction="none")
        return self.get_loss(loss)


class MultiClassDiceLoss(LossBase):
    def __init__(self, weights=None, ignore_indiex=None, activation="softmax"):
        super().__init__("mean")
        self.weights, self.ignore = weights, ignore_indiex
        self.activation = {"softmax": lambda t: torch.softmax(t, 1), "sigmoid": torch.sigmoid, "relu": torch.relu,
                           "tanh": torch.tanh, None: lambda t: t}[activation]
        self.smooth = 1e-5

    def construct(self, logits, label):
        p, y = self.activation(logits.float()), label.float()
        total = 0.0
        for c in range(y.shape[1]):
            if c == self.ignore:
                continue
            pc, yc = p[:, c].reshape(-1), y[:, c].reshape(-1)
            dice = 1 - (2 * (pc * yc).sum() + self.smooth) / ((pc * pc).sum() + (yc * yc).sum() + self.smooth)
            if self.weights is not None:
                dice = dice * self.weights[c]
            total = total + dice
        return _wrap_out(total / y.shape[1])


class SampledSoftmaxLoss(LossBase):
    """Softmax cross entropy over the true class and ``num_sampled`` uniformly sampled negatives (with the
    log-expected-count correction), for very large output vocabularies."""

    def __init__(self, num_sampled, num_classes, num_true=1, sampled_values=None, remove_accidental_hits=True, seed=0,
                 reduction="none"):
        super().__init__(reduction)
        self.num_sampled, self.num_classes, self.num_true = num_sampled, num_classes, num_true
        self.sampled_values, self.remove_accidental_hits = sampled_values, remove_accidental_hits
        self._gen = torch.Generator().manual_seed(seed)

    def construct(self, weights, biases, labels, logits):
        labels = labels.reshape(-1, self.num_true).long()
        dev = logits.device
        if self.sampled_values is not None:
            sampled = torch.as_tensor(self.sampled_values[0]).long().to(dev)
        else:
            sampled = torch.randint(0, self.num_classes, (self.num_sampled,), generator=self._gen).to(dev)
        q = self.num_sampled / self.num_classes
        true_w, true_b = weights[labels], biases[labels]                                   # [B, T, D], [B, T]
        true_logit = (logits.unsqueeze(1) * true_w).sum(-1) + true_b - torch.log(torch.tensor(q, device=dev))
        samp_logit = logits @ weights[sampled].t() + biases[sampled] - torch.log(torch.tensor(q, device=dev))
        if self.remove_accidental_hits:
            hit = (sampled.reshape(1, 1, -1) == labels.unsqueeze(-1)).any(1)
            samp_logit = samp_logit.masked_fill(hit, -1e9)
        all_logits = torch.cat([true_logit, samp_logit], 1).float()
        target = torch.cat([torch.full_like(true_logit, 1.0 / self.num_true), torch.zeros_like(samp_logit)], 1).float()
        return self.get_loss(-(target * torch.log_softmax(all_logits, -1)).sum(-1))


class TripletMarginWithDistanceLoss(LossBase):
    """max(d(a, p) - d(a, n) + margin, 0) with a caller-supplied distance (pairwise L2 by default); ``swap`` uses
    min(d(a, n), d(p, n)) as the negative distance.  Parity: nn/loss/loss.py (TripletMarginWithDistanceLoss)."""

    def __init__(self, distance_function=None, swap=False, reduction="mean", margin=1.0):
        super().__init__(reduction)
        self.distance_function, self.swap, self.margin = distance_function, swap, margin

    def construct(self, x, positive, negative):
        d = self.distance_function or (lambda a, b: _wrap_out(F.pairwise_distance(a, b)))
        dp, dn = d(x, positive), d(x, negative)
        if self.swap:
            dn = torch.minimum(dn, d(positive, negative))
        return self.get_loss(_wrap_out(torch.clamp(dp - dn + self.margin, min=0)))
