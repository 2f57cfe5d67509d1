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
