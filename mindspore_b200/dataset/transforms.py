"""Column transforms usable in ``Dataset.map`` (python/mindspore/dataset/transforms/transforms.py)."""
import numpy as np


class Compose:
    def __init__(self, transforms):
        self.transforms = list(transforms)

    def __call__(self, *x):
        for t in self.transforms:
            x = t(*x)
            if not isinstance(x, tuple):
                x = (x,)
        return x if len(x) > 1 else x[0]


class TypeCast:
    def __init__(self, data_type):
        import torch
        self.dtype = {torch.float32: np.float32, torch.int32: np.int32, torch.int64: np.int64,
                      torch.float16: np.float16, torch.uint8: np.uint8}.get(data_type, data_type)

    def __call__(self, x):
        return np.asarray(x).astype(self.dtype)


class OneHot:
    def __init__(self, num_classes, smoothing_rate=0.0):
        self.n, self.s = num_classes, smoothing_rate

    def __call__(self, x):
        out = np.full((self.n,), self.s / self.n, dtype=np.float32)
        out[int(x)] += 1.0 - self.s
        return out
