"""Image transforms on HWC numpy arrays (python/mindspore/dataset/vision/transforms.py subset)."""
import numpy as np


class Rescale:
    def __init__(self, rescale, shift):
        self.r, self.s = rescale, shift

    def __call__(self, img):
        return np.asarray(img, dtype=np.float32) * self.r + self.s


class Normalize:
    def __init__(self, mean, std, is_hwc=True):
        self.mean, self.std, self.hwc = np.asarray(mean, np.float32), np.asarray(std, np.float32), is_hwc

    def __call__(self, img):
        img = np.asarray(img, dtype=np.float32)
        if self.hwc:
            return (img - self.mean) / self.std
        return (img - self.mean[:, None, None]) / self.std[:, None, None]


class HWC2CHW:
    def __call__(self, img):
        return np.ascontiguousarray(np.transpose(img, (2, 0, 1)))


class RandomHorizontalFlip:
    def __init__(self, prob=0.5):
        self.p = prob

    def __call__(self, img):
        return img[:, ::-1].copy() if np.random.random() < self.p else img


class RandomCrop:
    def __init__(self, size, padding=0):
        self.size = (size, size) if isinstance(size, int) else tuple(size)
        self.pad = padding

    def __call__(self, img):
        if self.pad:
            img = np.pad(img, ((self.pad, self.pad), (self.pad, self.pad), (0, 0)))
        h, w = img.shape[:2]
        th, tw = self.size
        i, j = np.random.randint(0, h - th + 1), np.random.randint(0, w - tw + 1)
        return img[i:i + th, j:j + tw]


class CenterCrop:
    def __init__(self, size):
        self.size = (size, size) if isinstance(size, int) else tuple(size)

    def __call__(self, img):
        h, w = img.shape[:2]
        th, tw = self.size
        i, j = (h - th) // 2, (w - tw) // 2
        return img[i:i + th, j:j + tw]


class Resize:
    """Nearest / bilinear resize of an HWC array."""

    def __init__(self, size, interpolation="bilinear"):
        self.size = (size, size) if isinstance(size, int) else tuple(size)
        self.mode = interpolation

    def __call__(self, img):
        import torch
        t = torch.from_numpy(np.ascontiguousarray(img)).float().permute(2, 0, 1)[None]
        mode = "nearest" if str(self.mode).lower().startswith("nearest") else "bilinear"
        out = torch.nn.functional.interpolate(t, size=self.size, mode=mode,
                                              **({} if mode == "nearest" else {"align_corners": False}))
        return out[0].permute(1, 2, 0).numpy().astype(img.dtype if img.dtype != np.uint8 else np.float32)
