"""Evaluation metrics.  Parity: mindspore/python/mindspore/train/metrics/*.py (Metric base, Accuracy, Top1/Top5,
Loss, MAE, MSE, Precision, Recall, F1/Fbeta, ConfusionMatrix, Perplexity, Dice, names() / get_metric_fn())."""
import numpy as np
import torch


def _np(x):
    if isinstance(x, torch.Tensor):
        x = x.detach()
        if x.dtype == torch.bfloat16:
            x = x.float()
        return x.cpu().numpy()
    return np.asarray(x)


class Metric:
    def __init__(self):
        self._indexes = None

    def set_indexes(self, indexes):
        if not isinstance(indexes, list) or not all(isinstance(i, int) and not isinstance(i, bool) for i in indexes):
            raise ValueError("For 'set_indexes', the argument 'indexes' must be a list of int")
        self._indexes = indexes
        return self

    @property
    def indexes(self):
        return self._indexes

    def __call__(self, *inputs):
        self.clear()
        self.update(*inputs)
        return self.eval()

    def clear(self): raise NotImplementedError
    def update(self, *inputs): raise NotImplementedError
    def eval(self): raise NotImplementedError


class Accuracy(Metric):
    def __init__(self, eval_type="classification"):
        super().__init__()
        if eval_type not in ("classification", "multilabel"):
            raise ValueError("eval_type must be classification or multilabel")
        self._type = eval_type
        self.clear()

    def clear(self):
        self._correct, self._total = 0, 0

    def update(self, *inputs):
        if len(inputs) != 2:
            raise ValueError("For 'Accuracy.update', it needs 2 inputs (predicted value, true value)")
        y_pred, y = _np(inputs[0]), _np(inputs[1])
        if self._type == "classification":
            if y_pred.ndim == y.ndim and y_pred.shape == y.shape and y_pred.ndim > 1:
                y = y.argmax(1)
            idx = y_pred.argmax(1)
            self._correct += int((idx == y.reshape(idx.shape)).sum())
        else:
            self._correct += int((y_pred.round() == y).all(1).sum())
        self._total += y_pred.shape[0]

    def eval(self):
        if self._total == 0:
            raise RuntimeError("The 'Accuracy' can not be calculated, because the number of samples is 0")
        return self._correct / self._total


class TopKCategoricalAccuracy(Metric):
    def __init__(self, k):
        super().__init__()
        if not isinstance(k, int) or k <= 0:
            raise ValueError("k must be a positive int")
        self.k = k
        self.clear()

    def clear(self):
        self._correct, self._total = 0, 0

    def update(self, *inputs):
        y_pred, y = _np(inputs[0]), _np(inputs[1])
        if y.ndim == y_pred.ndim:
            y = y.argmax(1)
        top = np.argsort(-y_pred, axis=1)[:, :self.k]
        self._correct += int((top == y.reshape(-1, 1)).any(1).sum())
        self._total += y_pred.shape[0]

    def eval(self):
        if self._total == 0:
            raise RuntimeError("The number of samples is 0")
        return self._correct / self._total


class Top1CategoricalAccuracy(TopKCategoricalAccuracy):
    def __init__(self):
        super().__init__(1)


class Top5CategoricalAccuracy(TopKCategoricalAccuracy):
    def __init__(self):
        super().__init__(5)


class Loss(Metric):
    def __init__(self):
        super().__init__()
        self.clear()

    def clear(self):
        self._sum, self._n = 0.0, 0

    def update(self, *inputs):
        if len(inputs) != 1:
            raise ValueError("For 'Loss.update', it needs 1 input (loss)")
        v = _np(inputs[0])
        if v.ndim > 1:
            raise ValueError("the dimension of loss must be 0 or 1")
        self._sum += float(v.mean())
        self._n += 1

    def eval(self):
        if self._n == 0:
            raise RuntimeError("The total number can not be 0")
        return self._sum / self._n


class MAE(Metric):
    def __init__(self):
        super().__init__()
        self.clear()

    def clear(self):
        self._sum, self._n = 0.0, 0

    def update(self, *inputs):
        a, b = _np(inputs[0]), _np(inputs[1])
        self._sum += float(np.abs(a.reshape(b.shape) - b).mean())
        self._n += 1

    def eval(self):
        if self._n == 0:
            raise RuntimeError("The number of input samples must not be 0")
        return self._sum / self._n


class MSE(MAE):
    def update(self, *inputs):
        a, b = _np(inputs[0]), _np(inputs[1])
        self._sum += float(((a.reshape(b.shape) - b) ** 2).mean())
        self._n += 1


class ConfusionMatrix(Metric):
    def __init__(self, num_classes, normalize="no_norm", threshold=0.5):
        super().__init__()
        self.num_classes, self.normalize = num_classes, normalize
        self.clear()

    def clear(self):
        self.cm = np.zeros((self.num_classes, self.num_classes))

    def update(self, *inputs):
        y_pred, y = _np(inputs[0]), _np(inputs[1]).astype(int).reshape(-1)
        if y_pred.ndim > 1:
            y_pred = y_pred.argmax(1)
        np.add.at(self.cm, (y, y_pred.astype(int).reshape(-1)), 1)

    def eval(self):
        cm = self.cm.copy()
        if self.normalize == "target":
            cm = cm / np.maximum(cm.sum(1, keepdims=True), 1)
        elif self.normalize == "prediction":
            cm = cm / np.maximum(cm.sum(0, keepdims=True), 1)
        elif self.normalize == "all":
            cm = cm / max(cm.sum(), 1)
        return cm


class _PRBase(Metric):
    def __init__(self, eval_type="classification"):
        super().__init__()
        self.clear()

    def clear(self):
        self.tp = self.fp = self.fn = None

    def update(self, *inputs):
        y_pred, y = _np(inputs[0]), _np(inputs[1])
        c = y_pred.shape[1]
        pred = np.eye(c)[y_pred.argmax(1)]
        if y.ndim == 1 or y.shape != pred.shape:
            y = np.eye(c)[y.astype(int).reshape(-1)]
        tp, fp, fn = (pred * y).sum(0), (pred * (1 - y)).sum(0), ((1 - pred) * y).sum(0)
        if self.tp is None:
            self.tp, self.fp, self.fn = tp, fp, fn
        else:
            self.tp, self.fp, self.fn = self.tp + tp, self.fp + fp, self.fn + fn


class Precision(_PRBase):
    def eval(self, average=False):
        v = self.tp / np.maximum(self.tp + self.fp, 1e-12)
        return v.mean() if average else v


class Recall(_PRBase):
    def eval(self, average=False):
        v = self.tp / np.maximum(self.tp + self.fn, 1e-12)
        return v.mean() if average else v


class Fbeta(_PRBase):
    def __init__(self, beta):
        super().__init__()
        self.beta = beta

    def eval(self, average=False):
        b2 = self.beta ** 2
        v = (1 + b2) * self.tp / np.maximum((1 + b2) * self.tp + b2 * self.fn + self.fp, 1e-12)
        return v.mean() if average else v


class F1(Fbeta):
    def __init__(self):
        super().__init__(1.0)


class Perplexity(Metric):
    def __init__(self, ignore_label=None):
        super().__init__()
        self.ignore = ignore_label
        self.clear()

    def clear(self):
        self._sum, self._n = 0.0, 0

    def update(self, *inputs):
        probs, labels = _np(inputs[0]), _np(inputs[1]).astype(int).reshape(-1)
        p = probs.reshape(-1, probs.shape[-1])[np.arange(labels.size), labels]
        if self.ignore is not None:
            keep = labels != self.ignore
            p = p[keep]
        self._sum += float(-np.log(np.maximum(p, 1e-10)).sum())
        self._n += p.size

    def eval(self):
        if self._n == 0:
            raise RuntimeError("The 'Perplexity' can not be calculated, because the number of samples is 0")
        return float(np.exp(self._sum / self._n))


class Dice(Metric):
    def __init__(self, smooth=1e-5):
        super().__init__()
        self.smooth = smooth
        self.clear()

    def clear(self):
        self._sum, self._n = 0.0, 0

    def update(self, *inputs):
        a, b = _np(inputs[0]), _np(inputs[1])
        inter = (a * b).sum()
        self._sum += float((2 * inter + self.smooth) / ((a * a).sum() + (b * b).sum() + self.smooth))
        self._n += 1

    def eval(self):
        if self._n == 0:
            raise RuntimeError("The 'Dice' can not be calculated, because the number of samples is 0")
        return self._sum / self._n


_METRICS = {"acc": Accuracy, "accuracy": Accuracy, "loss": Loss, "mae": MAE, "mse": MSE, "precision": Precision,
            "recall": Recall, "f1_score": F1, "F1": F1, "top_1_accuracy": Top1CategoricalAccuracy,
            "top_5_accuracy": Top5CategoricalAccuracy, "perplexity": Perplexity, "dice": Dice}


def names():
    return list(_METRICS)


def get_metric_fn(name, *args, **kwargs):
    if name not in _METRICS:
        raise KeyError("Metric %r is not supported; supported: %s" % (name, names()))
    return _METRICS[name](*args, **kwargs)


def get_metrics(metrics):
    if metrics is None:
        return {}
    if isinstance(metrics, dict):
        for k, v in metrics.items():
            if not isinstance(k, str) or not isinstance(v, Metric):
                raise TypeError("Metrics format error: dict of str -> Metric expected")
        return dict(metrics)
    if isinstance(metrics, (set, list, tuple)):
        return {m: get_metric_fn(m) for m in metrics}
    raise TypeError("Metrics should be None, dict or set, but got %s" % type(metrics))


# ------------------------------------------------------------------------------------------------ further metrics
def _np(x):
    import numpy as np
    if hasattr(x, "detach"):
        x = x.detach().float().cpu().numpy() if x.dtype.is_floating_point else x.detach().cpu().numpy()
    return np.asarray(x)


class ROC(Metric):
    """(fpr, tpr, thresholds) of a binary (``pos_label``) or multi-class (``class_num``) problem."""

    def __init__(self, class_num=None, pos_label=None):
        super().__init__()
        self.class_num, self.pos_label = class_num, pos_label
        self.clear()

    def clear(self):
        self._pred, self._true = [], []

    def update(self, y_pred, y):
        self._pred.append(_np(y_pred))
        self._true.append(_np(y))

    @staticmethod
    def _curve(score, pos):
        import numpy as np
        order = np.argsort(-score, kind="stable")
        score, pos = score[order], pos[order]
        distinct = np.where(np.diff(score))[0]
        idx = np.r_[distinct, pos.size - 1]
        tps = np.cumsum(pos)[idx]
        fps = 1 + idx - tps
        tps, fps = np.r_[0, tps], np.r_[0, fps]
        thr = np.r_[score[idx[0]] + 1, score[idx]]
        return fps / max(fps[-1], 1), tps / max(tps[-1], 1), thr

    def eval(self):
        import numpy as np
        if not self._pred:
            raise RuntimeError("ROC: update must be called before eval")
        pred, true = np.concatenate(self._pred), np.concatenate(self._true)
        if pred.ndim == 1 or (self.class_num in (None, 1)):
            pos = 1 if self.pos_label is None else self.pos_label
            return self._curve(pred.reshape(-1), (true.reshape(-1) == pos).astype(np.float64))
        res = [self._curve(pred[:, c], (true == c).astype(np.float64)) for c in range(pred.shape[1])]
        return [r[0] for r in res], [r[1] for r in res], [r[2] for r in res]


def auc(x, y, reorder=False):
    """Area under the curve (x, y) by the trapezoidal rule."""
    import numpy as np
    x, y = _np(x).astype(np.float64), _np(y).astype(np.float64)
    if x.size < 2:
        raise ValueError("For 'auc', at least 2 points are needed")
    if reorder:
        o = np.lexsort((y, x))
        x, y = x[o], y[o]
    direction = 1
    d = np.diff(x)
    if np.any(d < 0):
        if np.all(d <= 0):
            direction = -1
        else:
            raise ValueError("The 'x' array is neither increasing nor decreasing")
    return float(direction * np.sum((y[1:] + y[:-1]) * d / 2.0))


class BleuScore(Metric):
    def __init__(self, n_gram=4, smooth=False):
        super().__init__()
        self.n_gram, self.smooth = int(n_gram), smooth
        self.clear()

    def clear(self):
        self._num = [0.0] * self.n_gram
        self._den = [0.0] * self.n_gram
        self._c = self._r = 0

    @staticmethod
    def _counts(tokens, n):
        from collections import Counter
        c = Counter()
        for k in range(1, n + 1):
            for i in range(len(tokens) - k + 1):
                c[tuple(tokens[i:i + k])] += 1
        return c

    def update(self, candidate_corpus, reference_corpus):
        for cand, refs in zip(candidate_corpus, reference_corpus):
            self._c += len(cand)
            self._r += min((len(r) for r in refs), key=lambda L: (abs(L - len(cand)), L))
            cc = self._counts(cand, self.n_gram)
            from collections import Counter
            best = Counter()
            for r in refs:
                best |= self._counts(r, self.n_gram)
            clipped = cc & best
            for g, v in clipped.items():
                self._num[len(g) - 1] += v
            for g, v in cc.items():
                self._den[len(g) - 1] += v

    def eval(self):
        import math
        if self._c == 0:
            raise RuntimeError("BleuScore: update must be called before eval")
        if min(self._num) == 0 and not self.smooth:
            return 0.0
        if self.smooth:
            prec = [(n + 1) / (d + 1) for n, d in zip(self._num, self._den)]
        else:
            prec = [n / d for n, d in zip(self._num, self._den)]
        geo = math.exp(sum(math.log(p) for p in prec) / self.n_gram)
        bp = 1.0 if self._c > self._r else math.exp(1 - self._r / self._c)
        return bp * geo


class CosineSimilarity(Metric):
    def __init__(self, similarity="cosine", reduction="none", zero_diagonal=True):
        super().__init__()
        self.similarity, self.reduction, self.zero_diagonal = similarity, reduction, zero_diagonal
        self.clear()

    def clear(self):
        self._m = None

    def update(self, inputs):
        import numpy as np
        m = _np(inputs).astype(np.float64)
        if self.similarity == "cosine":
            m = m / np.linalg.norm(m, axis=1, keepdims=True)
        s = m @ m.T
        if self.zero_diagonal:
            np.fill_diagonal(s, 0)
        self._m = s

    def eval(self):
        if self._m is None:
            raise RuntimeError("CosineSimilarity: update must be called before eval")
        if self.reduction == "mean":
            return self._m.mean(-1)
        if self.reduction == "sum":
            return self._m.sum(-1)
        return self._m


class ConfusionMatrixMetric(Metric):
    """Metrics derived from the binary confusion matrix per class: sensitivity / recall / tpr, specificity / tnr,
    precision / ppv, npv, fnr, fpr, accuracy, f1 score, threat score (one-hot or thresholded predictions)."""

    _ALIASES = {"sensitivity": "tpr", "recall": "tpr", "hit_rate": "tpr", "true_positive_rate": "tpr", "tpr": "tpr",
                "specificity": "tnr", "selectivity": "tnr", "true_negative_rate": "tnr", "tnr": "tnr",
                "precision": "ppv", "positive_predictive_value": "ppv", "ppv": "ppv",
                "negative_predictive_value": "npv", "npv": "npv", "miss_rate": "fnr", "false_negative_rate": "fnr",
                "fnr": "fnr", "fall_out": "fpr", "false_positive_rate": "fpr", "fpr": "fpr", "accuracy": "acc",
                "acc": "acc", "f1_score": "f1", "f1": "f1", "threat_score": "ts", "critical_success_index": "ts",
                "ts": "ts", "csi": "ts"}

    def __init__(self, skip_channel=True, metric_name="sensitivity", calculation_method=False, decrease="mean"):
        super().__init__()
        key = metric_name.replace(" ", "_").lower()
        if key not in self._ALIASES:
            raise NotImplementedError("The metric is not implemented: %s" % metric_name)
        self.kind, self.skip_channel, self.decrease = self._ALIASES[key], skip_channel, decrease
        self.calculation_method = calculation_method
        self.clear()

    def clear(self):
        self._cm = None

    def update(self, y_pred, y):
        import numpy as np
        p, t = _np(y_pred) > 0.5, _np(y) > 0.5
        if self.skip_channel and p.shape[1] > 1:
            p, t = p[:, 1:], t[:, 1:]
        p = p.reshape(p.shape[0], p.shape[1], -1)
        t = t.reshape(t.shape[0], t.shape[1], -1)
        tp = (p & t).sum(-1); fp = (p & ~t).sum(-1); tn = (~p & ~t).sum(-1); fn = (~p & t).sum(-1)
        cm = np.stack([tp, fp, tn, fn], -1).astype(np.float64)            # [B, C, 4]
        self._cm = cm if self._cm is None else np.concatenate([self._cm, cm], 0)

    def eval(self):
        import numpy as np
        if self._cm is None:
            raise RuntimeError("ConfusionMatrixMetric: update must be called before eval")
        cm = self._cm.sum(0) if self.calculation_method else self._cm
        tp, fp, tn, fn = (cm[..., i] for i in range(4))
        with np.errstate(divide="ignore", invalid="ignore"):
            v = {"tpr": tp / (tp + fn), "tnr": tn / (tn + fp), "ppv": tp / (tp + fp), "npv": tn / (tn + fn),
                 "fnr": fn / (fn + tp), "fpr": fp / (fp + tn), "acc": (tp + tn) / (tp + fp + tn + fn),
                 "f1": 2 * tp / (2 * tp + fp + fn), "ts": tp / (tp + fn + fp)}[self.kind]
        return float(np.nanmean(v)) if self.decrease == "mean" else np.nan_to_num(v)


def _surface(mask):
    import numpy as np
    from scipy import ndimage
    m = mask.astype(bool)
    return m & ~ndimage.binary_erosion(m)


class _SurfaceDistance(Metric):
    def __init__(self, symmetric=False, distance_metric="euclidean"):
        super().__init__()
        self.symmetric, self.distance_metric = symmetric, distance_metric
        self.clear()

    def clear(self):
        self._d = None

    def _dist(self, a, b):
        from scipy import ndimage
        sa, sb = _surface(a), _surface(b)
        if not sb.any() or not sa.any():
            import numpy as np
            return np.array([np.inf])
        dt = ndimage.distance_transform_edt(~sb) if self.distance_metric == "euclidean" else \
            ndimage.distance_transform_cdt(~sb, metric="taxicab" if self.distance_metric == "taxicab" else "chessboard")
        return dt[sa]

    def update(self, y_pred, y, label_idx=1):
        import numpy as np
        a, b = _np(y_pred) == label_idx, _np(y) == label_idx
        d = self._dist(a, b)
        if self.symmetric:
            d = np.concatenate([d, self._dist(b, a)])
        self._d = d

    def _reduce(self, d):
        raise NotImplementedError

    def eval(self):
        if self._d is None:
            raise RuntimeError("update must be called before eval")
        return float(self._reduce(self._d))


class MeanSurfaceDistance(_SurfaceDistance):
    def _reduce(self, d):
        return d.mean()


class RootMeanSquareDistance(_SurfaceDistance):
    def _reduce(self, d):
        import numpy as np
        return np.sqrt((d ** 2).mean())


class HausdorffDistance(_SurfaceDistance):
    def __init__(self, distance_metric="euclidean", percentile=None, directed=False, crop=True):
        super().__init__(symmetric=not directed, distance_metric=distance_metric)
        self.percentile = percentile

    def _reduce(self, d):
        import numpy as np
        return d.max() if self.percentile is None else np.percentile(d, self.percentile)


class OcclusionSensitivity(Metric):
    """Drop in the score of class ``label`` when a ``mask_size`` window of the input is replaced by ``pad_val``,
    for every window position (stride ``stride``): a map of which regions the model relies on."""

    def __init__(self, pad_val=0.0, margin=2, n_batch=128, b_box=None):
        super().__init__()
        self.pad_val, self.margin, self.n_batch, self.b_box = pad_val, margin, n_batch, b_box
        self.clear()

    def clear(self):
        self._map = None

    def update(self, model, y_pred, label):
        import numpy as np
        import torch
        x = y_pred if isinstance(y_pred, torch.Tensor) else torch.as_tensor(_np(y_pred))
        lab = int(_np(label).reshape(-1)[0])
        with torch.no_grad():
            base = float(model(x)[0, lab])
            spatial = x.shape[2:]
            out = np.zeros(spatial, dtype=np.float64)
            m = self.margin
            for idx in np.ndindex(*spatial):
                occ = x.clone()
                sl = (slice(None), slice(None)) + tuple(slice(max(i - m, 0), i + m + 1) for i in idx)
                occ[sl] = self.pad_val
                out[idx] = base - float(model(occ)[0, lab])
        self._map = out

    def eval(self):
        if self._map is None:
            raise RuntimeError("OcclusionSensitivity: update must be called before eval")
        return self._map


def rearrange_inputs(func):
    """Decorator for ``update``: reorders the inputs by ``set_indexes`` before the metric sees them."""
    import functools

    @functools.wraps(func)
    def wrapper(self, *inputs):
        idx = self._indexes
        return func(self, *(inputs if idx is None else [inputs[i] for i in idx]))
    return wrapper


EvaluationBase = Metric
_METRICS.update({"roc": ROC, "bleu_score": BleuScore, "cosine_similarity": CosineSimilarity,
                 "confusion_matrix_metric": ConfusionMatrixMetric, "hausdorff_distance": HausdorffDistance,
                 "mean_surface_distance": MeanSurfaceDistance, "root_mean_square_distance": RootMeanSquareDistance,
                 "occlusion_sensitivity": OcclusionSensitivity})
