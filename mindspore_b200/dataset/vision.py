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


# ------------------------------------------------------------------------------------------------ further operations
import enum as _enum
import io as _io


class Inter(_enum.IntEnum):
    NEAREST = 0
    LINEAR = 2
    BILINEAR = 2
    CUBIC = 3
    BICUBIC = 3
    AREA = 4
    PILCUBIC = 5
    ANTIALIAS = 1


class Border(str, _enum.Enum):
    CONSTANT = "constant"
    EDGE = "edge"
    REFLECT = "reflect"
    SYMMETRIC = "symmetric"


def _pil(img):
    from PIL import Image
    if isinstance(img, Image.Image):
        return img
    a = np.asarray(img)
    if a.ndim == 3 and a.shape[2] == 1:
        a = a[..., 0]
    if a.dtype != np.uint8:
        a = np.clip(a, 0, 255).astype(np.uint8)
    return Image.fromarray(a)


def _np_img(pil, like=None):
    a = np.asarray(pil)
    if a.ndim == 2 and like is not None and np.asarray(like).ndim == 3:
        a = a[..., None]
    return a


def _resample(interp):
    from PIL import Image
    return {Inter.NEAREST: Image.NEAREST, Inter.LINEAR: Image.BILINEAR, Inter.CUBIC: Image.BICUBIC,
            Inter.AREA: Image.BOX, Inter.ANTIALIAS: Image.LANCZOS, Inter.PILCUBIC: Image.BICUBIC}[Inter(interp)]


def _pair(v):
    return (v, v) if isinstance(v, int) else tuple(v)


class Decode:
    """Encoded image bytes (uint8 1-D array or bytes) -> HWC uint8 RGB."""

    def __init__(self, to_pil=False):
        self.to_pil = to_pil

    def __call__(self, img):
        from PIL import Image
        raw = img.tobytes() if isinstance(img, np.ndarray) else bytes(img)
        im = Image.open(_io.BytesIO(raw)).convert("RGB")
        return im if self.to_pil else np.asarray(im)


class ToPIL:
    def __call__(self, img):
        return _pil(img)


class ToTensor:
    """HWC [0, 255] -> CHW float in [0, 1]."""

    def __init__(self, output_type=np.float32):
        self.dtype = output_type

    def __call__(self, img):
        a = np.asarray(img)
        if a.ndim == 2:
            a = a[..., None]
        return np.ascontiguousarray(a.transpose(2, 0, 1)).astype(self.dtype) / 255.0


class ToType:
    def __init__(self, data_type):
        self.dtype = data_type

    def __call__(self, img):
        return np.asarray(img).astype(self.dtype)


class Pad:
    def __init__(self, padding, fill_value=0, padding_mode=Border.CONSTANT):
        p = (padding,) * 4 if isinstance(padding, int) else tuple(padding)
        self.p = p * 2 if len(p) == 2 else p                    # left, top, right, bottom
        self.fill, self.mode = fill_value, Border(padding_mode)

    def __call__(self, img):
        l, t, r, b = self.p
        a = np.asarray(img)
        widths = ((t, b), (l, r)) + ((0, 0),) * (a.ndim - 2)
        if self.mode is Border.CONSTANT:
            return np.pad(a, widths, constant_values=self.fill)
        return np.pad(a, widths, mode=self.mode.value)


class Crop:
    def __init__(self, coordinates, size):
        self.c, self.s = tuple(coordinates), _pair(size)

    def __call__(self, img):
        return np.asarray(img)[self.c[0]:self.c[0] + self.s[0], self.c[1]:self.c[1] + self.s[1]]


class HorizontalFlip:
    def __call__(self, img):
        return np.asarray(img)[:, ::-1].copy()


class VerticalFlip:
    def __call__(self, img):
        return np.asarray(img)[::-1].copy()


class RandomVerticalFlip:
    def __init__(self, prob=0.5):
        self.p = prob

    def __call__(self, img):
        return np.asarray(img)[::-1].copy() if np.random.random() < self.p else img


class Rotate:
    def __init__(self, degrees, resample=Inter.NEAREST, expand=False, center=None, fill_value=0):
        self.deg, self.rs, self.expand, self.center, self.fill = degrees, resample, expand, center, fill_value

    def __call__(self, img):
        return _np_img(_pil(img).rotate(self.deg, _resample(self.rs), self.expand, self.center,
                                        fillcolor=self.fill), img)


class RandomRotation(Rotate):
    def __init__(self, degrees, resample=Inter.NEAREST, expand=False, center=None, fill_value=0):
        lo, hi = (-degrees, degrees) if isinstance(degrees, (int, float)) else degrees
        super().__init__(0, resample, expand, center, fill_value)
        self.range = (lo, hi)

    def __call__(self, img):
        self.deg = np.random.uniform(*self.range)
        return super().__call__(img)


class RandomResizedCrop:
    def __init__(self, size, scale=(0.08, 1.0), ratio=(3 / 4, 4 / 3), interpolation=Inter.BILINEAR, max_attempts=10):
        self.size, self.scale, self.ratio, self.interp, self.attempts = _pair(size), scale, ratio, interpolation, max_attempts

    def _box(self, h, w):
        area = h * w
        for _ in range(self.attempts):
            target = area * np.random.uniform(*self.scale)
            ar = np.exp(np.random.uniform(np.log(self.ratio[0]), np.log(self.ratio[1])))
            cw, ch = int(round(np.sqrt(target * ar))), int(round(np.sqrt(target / ar)))
            if 0 < cw <= w and 0 < ch <= h:
                return np.random.randint(0, h - ch + 1), np.random.randint(0, w - cw + 1), ch, cw
        s = min(h, w)
        return (h - s) // 2, (w - s) // 2, s, s

    def __call__(self, img):
        a = np.asarray(img)
        i, j, ch, cw = self._box(*a.shape[:2])
        crop = a[i:i + ch, j:j + cw]
        return _np_img(_pil(crop).resize((self.size[1], self.size[0]), _resample(self.interp)), img)


class RandomCropDecodeResize(RandomResizedCrop):
    def __call__(self, img):
        return super().__call__(Decode()(img))


def _enhance(kind, img, factor):
    from PIL import ImageEnhance
    return _np_img(getattr(ImageEnhance, kind)(_pil(img)).enhance(factor), img)


class AdjustBrightness:
    def __init__(self, brightness_factor):
        self.f = brightness_factor

    def __call__(self, img):
        return _enhance("Brightness", img, self.f)


class AdjustContrast:
    def __init__(self, contrast_factor):
        self.f = contrast_factor

    def __call__(self, img):
        return _enhance("Contrast", img, self.f)


class AdjustSaturation:
    def __init__(self, saturation_factor):
        self.f = saturation_factor

    def __call__(self, img):
        return _enhance("Color", img, self.f)


class AdjustHue:
    def __init__(self, hue_factor):
        if not -0.5 <= hue_factor <= 0.5:
            raise ValueError("hue_factor must be in [-0.5, 0.5], got %r" % (hue_factor,))
        self.f = hue_factor

    def __call__(self, img):
        hsv = np.array(_pil(img).convert("HSV"))
        hsv[..., 0] = (hsv[..., 0].astype(np.int32) + int(self.f * 255)) % 256
        from PIL import Image
        return np.asarray(Image.fromarray(hsv, "HSV").convert("RGB"))


class RandomSharpness:
    def __init__(self, degrees=(0.1, 1.9)):
        self.d = degrees

    def __call__(self, img):
        return _enhance("Sharpness", img, np.random.uniform(*self.d))


class RandomColorAdjust:
    def __init__(self, brightness=(1, 1), contrast=(1, 1), saturation=(1, 1), hue=(0, 0)):
        def rng(v, center):
            return (max(center - v, 0), center + v) if isinstance(v, (int, float)) else tuple(v)
        self.b, self.c, self.s = rng(brightness, 1), rng(contrast, 1), rng(saturation, 1)
        self.h = (-hue, hue) if isinstance(hue, (int, float)) else tuple(hue)

    def __call__(self, img):
        ops = [AdjustBrightness(np.random.uniform(*self.b)), AdjustContrast(np.random.uniform(*self.c)),
               AdjustSaturation(np.random.uniform(*self.s))]
        if self.h != (0, 0):
            ops.append(AdjustHue(np.random.uniform(*self.h)))
        for k in np.random.permutation(len(ops)):
            img = ops[k](img)
        return img


class Grayscale:
    def __init__(self, num_output_channels=1):
        self.n = num_output_channels

    def __call__(self, img):
        g = np.asarray(_pil(img).convert("L"))
        return np.repeat(g[..., None], self.n, 2)


class RandomGrayscale:
    def __init__(self, prob=0.1):
        self.p = prob

    def __call__(self, img):
        return Grayscale(np.asarray(img).shape[2])(img) if np.random.random() < self.p else img


class AutoContrast:
    def __init__(self, cutoff=0.0, ignore=None):
        self.cutoff, self.ignore = cutoff, ignore

    def __call__(self, img):
        from PIL import ImageOps
        return _np_img(ImageOps.autocontrast(_pil(img), self.cutoff, self.ignore), img)


class Equalize:
    def __call__(self, img):
        from PIL import ImageOps
        return _np_img(ImageOps.equalize(_pil(img)), img)


class Invert:
    def __call__(self, img):
        return 255 - np.asarray(img)


class GaussianBlur:
    def __init__(self, kernel_size, sigma=None):
        k = _pair(kernel_size)
        self.k = k
        self.sigma = _pair(sigma) if sigma is not None else tuple(0.3 * ((x - 1) * 0.5 - 1) + 0.8 for x in k)

    def __call__(self, img):
        a = np.asarray(img).astype(np.float32)
        for axis, (k, s) in enumerate(zip(self.k, self.sigma)):
            x = np.arange(k) - (k - 1) / 2
            w = np.exp(-x * x / (2 * s * s))
            w /= w.sum()
            pad = [(0, 0)] * a.ndim
            pad[axis] = (k // 2, k // 2)
            ap = np.pad(a, pad, mode="reflect")
            a = sum(w[i] * np.take(ap, np.arange(i, i + a.shape[axis]), axis=axis) for i in range(k))
        return a.astype(np.asarray(img).dtype) if np.asarray(img).dtype == np.uint8 else a


class RandomErasing:
    """CHW or HWC array: a random rectangle is set to ``value`` with probability ``prob``."""

    def __init__(self, prob=0.5, scale=(0.02, 0.33), ratio=(0.3, 3.3), value=0, inplace=False, max_attempts=10):
        self.p, self.scale, self.ratio, self.value, self.attempts = prob, scale, ratio, value, max_attempts

    def __call__(self, img):
        a = np.array(img)
        if np.random.random() >= self.p:
            return a
        chw = a.ndim == 3 and a.shape[0] <= 4 < a.shape[2]
        h, w = (a.shape[1], a.shape[2]) if chw else a.shape[:2]
        for _ in range(self.attempts):
            target = h * w * np.random.uniform(*self.scale)
            ar = np.exp(np.random.uniform(np.log(self.ratio[0]), np.log(self.ratio[1])))
            eh, ew = int(round(np.sqrt(target * ar))), int(round(np.sqrt(target / ar)))
            if 0 < eh < h and 0 < ew < w:
                i, j = np.random.randint(0, h - eh + 1), np.random.randint(0, w - ew + 1)
                if chw:
                    a[:, i:i + eh, j:j + ew] = self.value
                else:
                    a[i:i + eh, j:j + ew] = self.value
                break
        return a


class MixUpBatch:
    """Batch operation (use after ``batch`` with one-hot labels): convex combination of the batch with a permutation."""

    def __init__(self, alpha=1.0):
        self.alpha = alpha

    def __call__(self, images, labels):
        lam = np.random.beta(self.alpha, self.alpha)
        perm = np.random.permutation(len(images))
        x = lam * np.asarray(images, np.float32) + (1 - lam) * np.asarray(images, np.float32)[perm]
        y = lam * np.asarray(labels, np.float32) + (1 - lam) * np.asarray(labels, np.float32)[perm]
        return x, y


class CutMixBatch:
    def __init__(self, image_batch_format="NHWC", alpha=1.0, prob=1.0):
        self.nchw, self.alpha, self.p = str(image_batch_format).upper().endswith("NCHW"), alpha, prob

    def __call__(self, images, labels):
        x, y = np.array(images), np.asarray(labels, np.float32)
        if np.random.random() >= self.p:
            return x, y
        lam = np.random.beta(self.alpha, self.alpha)
        perm = np.random.permutation(len(x))
        h, w = (x.shape[2], x.shape[3]) if self.nchw else (x.shape[1], x.shape[2])
        ch, cw = int(h * np.sqrt(1 - lam)), int(w * np.sqrt(1 - lam))
        cy, cx = np.random.randint(h), np.random.randint(w)
        y0, y1, x0, x1 = max(cy - ch // 2, 0), min(cy + ch // 2, h), max(cx - cw // 2, 0), min(cx + cw // 2, w)
        if self.nchw:
            x[:, :, y0:y1, x0:x1] = x[perm][:, :, y0:y1, x0:x1]
        else:
            x[:, y0:y1, x0:x1] = x[perm][:, y0:y1, x0:x1]
        lam = 1 - (y1 - y0) * (x1 - x0) / (h * w)
        return x, lam * y + (1 - lam) * y[perm]



def __getattr__(name):
    # the remaining transforms live in vision_ext (which imports this module)
    import importlib
    ext = importlib.import_module(__package__ + ".vision_ext")
    if name in ext.__all__:
        return getattr(ext, name)
    raise AttributeError("module %r has no attribute %r" % (__name__, name))
