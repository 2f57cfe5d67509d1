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
