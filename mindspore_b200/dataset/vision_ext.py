"""The rest of the image transforms (HWC numpy arrays; PIL does the geometric warps): colour / tone operations,
affine and perspective warps, multi-crop, the bounding-box aware variants, the automatic augmentation policies
(AutoAugment, RandAugment, TrivialAugmentWide, UniformAugment) and the image file helpers.

Parity: python/mindspore/dataset/vision/transforms.py, utils.py.  Bounding boxes are float arrays [n, >= 4] of
(x, y, w, h, ...) in pixels, as in the reference."""
from __future__ import annotations

import enum
import math
import os

import numpy as np

from . import vision as V
from .vision import Border, Inter, _np_img, _pair, _pil, _resample


class ImageTensorOperation:
    """Base of the image transforms: a callable on numpy images."""

    def __call__(self, *args):
        return self._run(*args)


class VideoTensorOperation(ImageTensorOperation):
    pass


class AutoAugmentPolicy(str, enum.Enum):
    IMAGENET, CIFAR10, SVHN = "imagenet", "cifar10", "svhn"


class ConvertMode(enum.IntEnum):
    COLOR_BGR2BGRA, COLOR_RGB2RGBA, COLOR_BGRA2BGR, COLOR_RGBA2RGB, COLOR_BGR2RGBA, COLOR_RGB2BGRA = 0, 0, 1, 1, 2, 2
    COLOR_RGBA2BGR, COLOR_BGRA2RGB, COLOR_BGR2RGB, COLOR_RGB2BGR, COLOR_BGRA2RGBA, COLOR_RGBA2BGRA = 3, 3, 4, 4, 5, 5
    COLOR_BGR2GRAY, COLOR_RGB2GRAY, COLOR_GRAY2BGR, COLOR_GRAY2RGB, COLOR_GRAY2BGRA, COLOR_GRAY2RGBA = 6, 7, 8, 8, 9, 9
    COLOR_BGRA2GRAY, COLOR_RGBA2GRAY = 10, 11


class ImageBatchFormat(enum.IntEnum):
    NHWC, NCHW = 0, 1


class ImageReadMode(enum.IntEnum):
    UNCHANGED, GRAYSCALE, COLOR = 0, 1, 2


class SliceMode(enum.IntEnum):
    PAD, DROP = 0, 1


def not_random(func):
    """Marks a transform as deterministic (its results may be cached)."""
    func.random = False
    return func


def _f(img):
    return np.asarray(img).astype(np.float32)


def _like(out, img):
    a = np.asarray(img)
    return np.clip(out, 0, 255).astype(np.uint8) if a.dtype == np.uint8 else out.astype(a.dtype)


# ---------------------------------------------------------------------------------------------------- colour / tone
class AdjustGamma(ImageTensorOperation):
    def __init__(self, gamma, gain=1):
        if gamma < 0:
            raise ValueError("AdjustGamma: gamma must be non-negative")
        self.gamma, self.gain = gamma, gain

    def _run(self, img):
        a = np.asarray(img)
        scale = 255.0 if a.dtype == np.uint8 else 1.0
        return _like(scale * self.gain * np.power(_f(a) / scale, self.gamma), a)


class AdjustSharpness(ImageTensorOperation):
    def __init__(self, sharpness_factor):
        if sharpness_factor < 0:
            raise ValueError("AdjustSharpness: sharpness_factor must be non-negative")
        self.factor = sharpness_factor

    def _run(self, img):
        return V._enhance("Sharpness", img, self.factor)


class RandomAdjustSharpness(ImageTensorOperation):
    def __init__(self, degree, prob=0.5):
        self.op, self.p = AdjustSharpness(degree), prob

    def _run(self, img):
        return self.op(img) if np.random.random() < self.p else np.asarray(img)


class Posterize(ImageTensorOperation):
    def __init__(self, bits):
        if not 0 <= bits <= 8:
            raise ValueError("Posterize: bits must be in [0, 8]")
        self.bits = bits

    def _run(self, img):
        a = np.asarray(img)
        mask = np.uint8((0xFF << (8 - self.bits)) & 0xFF)
        return a & mask


class RandomPosterize(ImageTensorOperation):
    def __init__(self, bits=(8, 8)):
        self.bits = (bits, bits) if isinstance(bits, int) else tuple(bits)

    def _run(self, img):
        return Posterize(int(np.random.randint(self.bits[0], self.bits[1] + 1)))(img)


class Solarize(ImageTensorOperation):
    """Inverts the pixels whose value lies inside ``threshold`` = (min, max) (a single number means (t, 255))."""

    def __init__(self, threshold):
        self.lo, self.hi = (threshold, 255) if isinstance(threshold, (int, float)) else tuple(threshold)
        if self.lo > self.hi:
            raise ValueError("Solarize: threshold must be (min, max) with min <= max")

    def _run(self, img):
        a = np.asarray(img)
        inside = (a >= self.lo) & (a <= self.hi)
        return np.where(inside, 255 - a, a).astype(a.dtype)


class RandomSolarize(ImageTensorOperation):
    def __init__(self, threshold=(0, 255)):
        self.range = tuple(threshold)

    def _run(self, img):
        a, b = sorted(np.random.randint(self.range[0], self.range[1] + 1, 2).tolist())
        return Solarize((a, b))(img)


class RandomAutoContrast(ImageTensorOperation):
    def __init__(self, cutoff=0.0, ignore=None, prob=0.5):
        self.op, self.p = V.AutoContrast(cutoff, ignore), prob

    def _run(self, img):
        return self.op(img) if np.random.random() < self.p else np.asarray(img)


class RandomEqualize(ImageTensorOperation):
    def __init__(self, prob=0.5):
        self.op, self.p = V.Equalize(), prob

    def _run(self, img):
        return self.op(img) if np.random.random() < self.p else np.asarray(img)


class RandomInvert(ImageTensorOperation):
    def __init__(self, prob=0.5):
        self.op, self.p = V.Invert(), prob

    def _run(self, img):
        return self.op(img) if np.random.random() < self.p else np.asarray(img)


class RandomColor(ImageTensorOperation):
    """Colour balance (saturation) by a factor drawn from ``degrees``."""

    def __init__(self, degrees=(0.1, 1.9)):
        self.range = tuple(degrees)

    def _run(self, img):
        return V._enhance("Color", img, np.random.uniform(*self.range))


class RandomLighting(ImageTensorOperation):
    """AlexNet-style PCA lighting noise: adds ``alpha_i * eigenvalue_i`` along the RGB eigenvectors."""
    _EIGVAL = np.array([55.46, 4.794, 1.148], np.float32)
    _EIGVEC = np.array([[-0.5675, 0.7192, 0.4009], [-0.5808, -0.0045, -0.8140], [-0.5836, -0.6948, 0.4203]],
                       np.float32)

    def __init__(self, alpha=0.05):
        if alpha < 0:
            raise ValueError("RandomLighting: alpha must be non-negative")
        self.alpha = alpha

    def _run(self, img):
        a = np.asarray(img)
        w = np.random.normal(0, self.alpha, 3).astype(np.float32)
        return _like(_f(a) + self._EIGVEC @ (w * self._EIGVAL), a)


def _rgb_to_hsv(a):
    import colorsys
    return np.vectorize(colorsys.rgb_to_hsv)(a[..., 0], a[..., 1], a[..., 2])


class RgbToHsv(ImageTensorOperation):
    """Float RGB in [0, 1] -> HSV in [0, 1]; ``is_hwc=False`` takes CHW."""

    def __init__(self, is_hwc=False):
        self.hwc = is_hwc

    def _run(self, img):
        a = _f(img)
        a = a if self.hwc else np.moveaxis(a, -3, -1)
        out = np.stack(_rgb_to_hsv(a), -1).astype(np.float32)
        return out if self.hwc else np.moveaxis(out, -1, -3)


class HsvToRgb(ImageTensorOperation):
    def __init__(self, is_hwc=False):
        self.hwc = is_hwc

    def _run(self, img):
        import colorsys
        a = _f(img)
        a = a if self.hwc else np.moveaxis(a, -3, -1)
        out = np.stack(np.vectorize(colorsys.hsv_to_rgb)(a[..., 0], a[..., 1], a[..., 2]), -1).astype(np.float32)
        return out if self.hwc else np.moveaxis(out, -1, -3)


class ConvertColor(ImageTensorOperation):
    def __init__(self, convert_mode):
        self.mode = ConvertMode(convert_mode) if not isinstance(convert_mode, ConvertMode) else convert_mode

    def _run(self, img):
        a = np.asarray(img)
        name = self.mode.name
        alpha = np.full(a.shape[:2] + (1,), 255 if a.dtype == np.uint8 else 1, a.dtype)
        gray = lambda rgb: _like((_f(rgb) @ np.array([0.299, 0.587, 0.114], np.float32)), a)
        m = int(self.mode)
        if m == 0:
            return np.concatenate([a[..., :3], alpha], -1)
        if m == 1:
            return a[..., :3]
        if m == 2:
            return np.concatenate([a[..., 2::-1], alpha], -1)
        if m == 3:
            return a[..., 2::-1]
        if m == 4:
            return a[..., ::-1].copy()
        if m == 5:
            return np.concatenate([a[..., 2::-1], a[..., 3:4]], -1)
        if m == 6:
            return gray(a[..., 2::-1])
        if m == 7:
            return gray(a[..., :3])
        if m == 8:
            g = a if a.ndim == 2 else a[..., 0]
            return np.stack([g, g, g], -1)
        if m == 9:
            g = a if a.ndim == 2 else a[..., 0]
            return np.concatenate([np.stack([g, g, g], -1), alpha], -1)
        if m == 10:
            return gray(a[..., 2::-1])
        if m == 11:
            return gray(a[..., :3])
        raise ValueError("ConvertColor: unsupported mode %s" % name)


class NormalizePad(ImageTensorOperation):
    """``Normalize`` plus an extra all-zero channel."""

    def __init__(self, mean, std, dtype="float32", is_hwc=True):
        self.norm, self.dtype, self.hwc = V.Normalize(mean, std, is_hwc), dtype, is_hwc

    def _run(self, img):
        out = self.norm(img)
        zero = np.zeros(out.shape[:2] + (1,) if self.hwc else (1,) + out.shape[1:], out.dtype)
        return np.concatenate([out, zero], -1 if self.hwc else 0).astype(self.dtype)


class LinearTransformation(ImageTensorOperation):
    """(flattened image - mean_vector) @ transformation_matrix, reshaped back (whitening)."""

    def __init__(self, transformation_matrix, mean_vector):
        self.m, self.mean = np.asarray(transformation_matrix, np.float32), np.asarray(mean_vector, np.float32)
        if self.m.ndim != 2 or self.m.shape[0] != self.m.shape[1] or self.mean.shape != (self.m.shape[0],):
            raise ValueError("LinearTransformation: need a square [D, D] matrix and a [D] mean vector")

    def _run(self, img):
        a = _f(img)
        return ((a.reshape(-1) - self.mean) @ self.m).reshape(a.shape)


class ToNumpy(ImageTensorOperation):
    def _run(self, img):
        return np.asarray(img)


# ---------------------------------------------------------------------------------------------------- geometry
def _affine_coeffs(center, angle, translate, scale, shear):
    """Inverse affine matrix (output -> input pixel) in PIL's 6-coefficient form."""
    rot, sx, sy = math.radians(angle), math.radians(shear[0]), math.radians(shear[1])
    cx, cy = center
    tx, ty = translate
    a = math.cos(rot - sy) / math.cos(sy)
    b = -math.cos(rot - sy) * math.tan(sx) / math.cos(sy) - math.sin(rot)
    c = math.sin(rot - sy) / math.cos(sy)
    d = -math.sin(rot - sy) * math.tan(sx) / math.cos(sy) + math.cos(rot)
    m = [d, -b, 0.0, -c, a, 0.0]
    m = [v / scale for v in m]
    m[2] += m[0] * (-cx - tx) + m[1] * (-cy - ty)
    m[5] += m[3] * (-cx - tx) + m[4] * (-cy - ty)
    m[2] += cx
    m[5] += cy
    return m


class Affine(ImageTensorOperation):
    def __init__(self, degrees, translate, scale, shear, resample=Inter.NEAREST, fill_value=0):
        if scale <= 0:
            raise ValueError("Affine: scale must be positive")
        self.deg, self.tr, self.scale = degrees, tuple(translate), scale
        self.shear = (shear, 0.0) if isinstance(shear, (int, float)) else tuple(shear)
        self.rs, self.fill = resample, fill_value

    def _run(self, img):
        from PIL import Image
        p = _pil(img)
        w, h = p.size
        coeffs = _affine_coeffs((w * 0.5, h * 0.5), -self.deg, (self.tr[0] * w if abs(self.tr[0]) <= 1 else self.tr[0],
                                                                 self.tr[1] * h if abs(self.tr[1]) <= 1 else self.tr[1]),
                                self.scale, (-self.shear[0], -self.shear[1]))
        fill = self.fill if isinstance(self.fill, int) or p.mode == "L" else tuple(self.fill)
        return _np_img(p.transform((w, h), Image.AFFINE, coeffs, _resample(self.rs), fillcolor=fill), img)


class RandomAffine(ImageTensorOperation):
    def __init__(self, degrees, translate=None, scale=None, shear=None, resample=Inter.NEAREST, fill_value=0):
        self.deg = (-degrees, degrees) if isinstance(degrees, (int, float)) else tuple(degrees)
        self.tr, self.scale, self.rs, self.fill = translate, scale, resample, fill_value
        if shear is None:
            self.shear = None
        elif isinstance(shear, (int, float)):
            self.shear = (-shear, shear, 0.0, 0.0)
        else:
            self.shear = tuple(shear) if len(shear) == 4 else (shear[0], shear[1], 0.0, 0.0)

    def _run(self, img):
        deg = np.random.uniform(*self.deg)
        tr = (0.0, 0.0)
        if self.tr is not None:
            t = tuple(self.tr)
            tr = (np.random.uniform(-t[0], t[0]), np.random.uniform(-t[1], t[1])) if len(t) == 2 else \
                (np.random.uniform(t[0], t[1]), np.random.uniform(t[2], t[3]))
        sc = np.random.uniform(*self.scale) if self.scale is not None else 1.0
        sh = (np.random.uniform(self.shear[0], self.shear[1]), np.random.uniform(self.shear[2], self.shear[3])) \
            if self.shear is not None else (0.0, 0.0)
        return Affine(deg, tr, sc, sh, self.rs, self.fill)(img)


def _perspective_coeffs(start, end):
    a, b = [], []
    for (sx, sy), (ex, ey) in zip(start, end):
        a.append([ex, ey, 1, 0, 0, 0, -sx * ex, -sx * ey])
        a.append([0, 0, 0, ex, ey, 1, -sy * ex, -sy * ey])
        b += [sx, sy]
    return np.linalg.lstsq(np.asarray(a, np.float64), np.asarray(b, np.float64), rcond=None)[0].tolist()


class Perspective(ImageTensorOperation):
    """Warps so that the four ``start_points`` land on ``end_points`` (each [[x, y]] x 4: tl, tr, br, bl)."""

    def __init__(self, start_points, end_points, interpolation=Inter.BILINEAR):
        if len(start_points) != 4 or len(end_points) != 4:
            raise ValueError("Perspective: start_points and end_points must hold four [x, y] points each")
        self.start, self.end, self.interp = start_points, end_points, interpolation

    def _run(self, img):
        from PIL import Image
        p = _pil(img)
        return _np_img(p.transform(p.size, Image.PERSPECTIVE, _perspective_coeffs(self.start, self.end),
                                   _resample(self.interp)), img)


class RandomPerspective(ImageTensorOperation):
    def __init__(self, distortion_scale=0.5, prob=0.5, interpolation=Inter.BICUBIC):
        if not 0 <= distortion_scale <= 1:
            raise ValueError("RandomPerspective: distortion_scale must be in [0, 1]")
        self.d, self.p, self.interp = distortion_scale, prob, interpolation

    def _run(self, img):
        a = np.asarray(img)
        if np.random.random() >= self.p:
            return a
        h, w = a.shape[:2]
        dx, dy = int(self.d * w / 2), int(self.d * h / 2)
        r = lambda n: int(np.random.randint(0, n + 1))
        start = [[0, 0], [w - 1, 0], [w - 1, h - 1], [0, h - 1]]
        end = [[r(dx), r(dy)], [w - 1 - r(dx), r(dy)], [w - 1 - r(dx), h - 1 - r(dy)], [r(dx), h - 1 - r(dy)]]
        return Perspective(start, end, self.interp)(a)


class ResizedCrop(ImageTensorOperation):
    def __init__(self, top, left, height, width, size, interpolation=Inter.BILINEAR):
        self.box, self.size, self.interp = (top, left, height, width), _pair(size), interpolation

    def _run(self, img):
        t, l, h, w = self.box
        crop = np.asarray(img)[t:t + h, l:l + w]
        return _np_img(_pil(crop).resize((self.size[1], self.size[0]), _resample(self.interp)), img)


class RandomResize(ImageTensorOperation):
    """Resizes with an interpolation mode drawn at random."""

    def __init__(self, size):
        self.size = size

    def _run(self, img):
        mode = [Inter.NEAREST, Inter.BILINEAR, Inter.BICUBIC, Inter.AREA][np.random.randint(4)]
        return V.Resize(self.size, mode)(img)


class PadToSize(ImageTensorOperation):
    def __init__(self, size, offset=None, fill_value=0, padding_mode=Border.CONSTANT):
        self.size, self.offset, self.fill = _pair(size), None if offset is None else _pair(offset), fill_value
        self.mode = Border(padding_mode).value if not isinstance(padding_mode, str) else padding_mode

    def _run(self, img):
        a = np.asarray(img)
        h, w = a.shape[:2]
        th, tw = self.size
        if th < h or tw < w:
            raise RuntimeError("PadToSize: the target size %s is smaller than the image %s" % (self.size, (h, w)))
        top, left = self.offset if self.offset is not None else ((th - h) // 2, (tw - w) // 2)
        pads = ((top, th - h - top), (left, tw - w - left)) + ((0, 0),) * (a.ndim - 2)
        if self.mode == "constant":
            return np.pad(a, pads, constant_values=self.fill if isinstance(self.fill, (int, float)) else 0)
        return np.pad(a, pads, mode=self.mode)


class FiveCrop(ImageTensorOperation):
    def __init__(self, size):
        self.size = _pair(size)

    def _run(self, img):
        a = np.asarray(img)
        h, w = a.shape[:2]
        th, tw = self.size
        if th > h or tw > w:
            raise ValueError("FiveCrop: the crop %s is larger than the image %s" % (self.size, (h, w)))
        ci, cj = (h - th) // 2, (w - tw) // 2
        return (a[:th, :tw], a[:th, w - tw:], a[h - th:, :tw], a[h - th:, w - tw:], a[ci:ci + th, cj:cj + tw])


class TenCrop(ImageTensorOperation):
    def __init__(self, size, use_vertical_flip=False):
        self.five, self.vertical = FiveCrop(size), use_vertical_flip

    def _run(self, img):
        a = np.asarray(img)
        flipped = a[::-1] if self.vertical else a[:, ::-1]
        return self.five(a) + self.five(flipped)


class Erase(ImageTensorOperation):
    def __init__(self, top, left, height, width, value=0, inplace=False):
        self.box, self.value, self.inplace = (top, left, height, width), value, inplace

    def _run(self, img):
        a = np.asarray(img) if self.inplace else np.array(img)
        t, l, h, w = self.box
        a[t:t + h, l:l + w] = self.value
        return a


class CutOut(ImageTensorOperation):
    """``num_patches`` square patches of side ``length`` at random places set to zero."""

    def __init__(self, length, num_patches=1, is_hwc=True):
        if length <= 0 or num_patches <= 0:
            raise ValueError("CutOut: length and num_patches must be positive")
        self.length, self.n, self.hwc = length, num_patches, is_hwc

    def _run(self, img):
        a = np.array(img)
        h, w = (a.shape[0], a.shape[1]) if self.hwc else (a.shape[-2], a.shape[-1])
        for _ in range(self.n):
            cy, cx = np.random.randint(h), np.random.randint(w)
            y0, y1 = max(cy - self.length // 2, 0), min(cy + self.length // 2, h)
            x0, x1 = max(cx - self.length // 2, 0), min(cx + self.length // 2, w)
            if self.hwc:
                a[y0:y1, x0:x1] = 0
            else:
                a[..., y0:y1, x0:x1] = 0
        return a


class SlicePatches(ImageTensorOperation):
    """Cuts the image into ``num_height`` x ``num_width`` equal patches (edges padded or dropped)."""

    def __init__(self, num_height=1, num_width=1, slice_mode=SliceMode.PAD, fill_value=0):
        self.nh, self.nw, self.mode, self.fill = num_height, num_width, SliceMode(slice_mode), fill_value

    def _run(self, img):
        a = np.asarray(img)
        h, w = a.shape[:2]
        if self.mode == SliceMode.PAD:
            ph, pw = -(-h // self.nh), -(-w // self.nw)
            a = np.pad(a, ((0, ph * self.nh - h), (0, pw * self.nw - w)) + ((0, 0),) * (a.ndim - 2),
                       constant_values=self.fill)
        else:
            ph, pw = h // self.nh, w // self.nw
        return tuple(a[i * ph:(i + 1) * ph, j * pw:(j + 1) * pw] for i in range(self.nh) for j in range(self.nw))


class MixUp(ImageTensorOperation):
    """Blends every image of a batch with another one (the next one, or a random one with ``is_single=False``);
    labels must be one-hot."""

    def __init__(self, batch_size, alpha, is_single=True):
        self.n, self.alpha, self.single = batch_size, alpha, is_single

    def _run(self, image, label):
        x, y = _f(image), _f(label)
        lam = np.random.beta(self.alpha, self.alpha) if self.single else \
            np.random.beta(self.alpha, self.alpha, x.shape[0]).astype(np.float32)
        perm = np.roll(np.arange(x.shape[0]), 1) if self.single else np.random.permutation(x.shape[0])
        lx = lam if self.single else lam.reshape((-1,) + (1,) * (x.ndim - 1))
        ly = lam if self.single else lam.reshape(-1, 1)
        return _like(lx * x + (1 - lx) * x[perm], image), ly * y + (1 - ly) * y[perm]


class DecodeVideo(VideoTensorOperation):
    def __init__(self):
        raise NotImplementedError("DecodeVideo needs a video decoder (ffmpeg bindings), which this build does not "
                                  "ship")


# ---------------------------------------------------------------------------------------------------- boxes
def _clip_boxes(boxes, w, h):
    b = np.array(boxes, dtype=np.float32)
    x0, y0 = np.clip(b[:, 0], 0, w), np.clip(b[:, 1], 0, h)
    x1, y1 = np.clip(b[:, 0] + b[:, 2], 0, w), np.clip(b[:, 1] + b[:, 3], 0, h)
    b[:, 0], b[:, 1], b[:, 2], b[:, 3] = x0, y0, x1 - x0, y1 - y0
    return b[(b[:, 2] > 0) & (b[:, 3] > 0)]


class RandomHorizontalFlipWithBBox(ImageTensorOperation):
    def __init__(self, prob=0.5):
        self.p = prob

    def _run(self, img, boxes):
        a, b = np.asarray(img), np.array(boxes, dtype=np.float32)
        if np.random.random() >= self.p:
            return a, b
        b[:, 0] = a.shape[1] - b[:, 0] - b[:, 2]
        return a[:, ::-1].copy(), b


class RandomVerticalFlipWithBBox(ImageTensorOperation):
    def __init__(self, prob=0.5):
        self.p = prob

    def _run(self, img, boxes):
        a, b = np.asarray(img), np.array(boxes, dtype=np.float32)
        if np.random.random() >= self.p:
            return a, b
        b[:, 1] = a.shape[0] - b[:, 1] - b[:, 3]
        return a[::-1].copy(), b


class ResizeWithBBox(ImageTensorOperation):
    def __init__(self, size, interpolation=Inter.LINEAR):
        self.resize = V.Resize(size, interpolation)

    def _run(self, img, boxes):
        a = np.asarray(img)
        out = self.resize(a)
        b = np.array(boxes, dtype=np.float32)
        sy, sx = out.shape[0] / a.shape[0], out.shape[1] / a.shape[1]
        b[:, [0, 2]] *= sx
        b[:, [1, 3]] *= sy
        return out, b


class RandomResizeWithBBox(ImageTensorOperation):
    def __init__(self, size):
        self.size = size

    def _run(self, img, boxes):
        mode = [Inter.NEAREST, Inter.BILINEAR, Inter.BICUBIC, Inter.AREA][np.random.randint(4)]
        return ResizeWithBBox(self.size, mode)(img, boxes)


class RandomCropWithBBox(ImageTensorOperation):
    def __init__(self, size, padding=None, pad_if_needed=False, fill_value=0, padding_mode=Border.CONSTANT):
        self.size, self.padding, self.pad_if_needed, self.fill = _pair(size), padding, pad_if_needed, fill_value

    def _run(self, img, boxes):
        a, b = np.asarray(img), np.array(boxes, dtype=np.float32)
        if self.padding:
            p = self.padding if isinstance(self.padding, int) else self.padding[0]
            a = np.pad(a, ((p, p), (p, p)) + ((0, 0),) * (a.ndim - 2), constant_values=self.fill)
            b[:, 0] += p
            b[:, 1] += p
        th, tw = self.size
        if self.pad_if_needed and (a.shape[0] < th or a.shape[1] < tw):
            ph, pw = max(th - a.shape[0], 0), max(tw - a.shape[1], 0)
            a = np.pad(a, ((0, ph), (0, pw)) + ((0, 0),) * (a.ndim - 2), constant_values=self.fill)
        i, j = np.random.randint(0, a.shape[0] - th + 1), np.random.randint(0, a.shape[1] - tw + 1)
        b[:, 0] -= j
        b[:, 1] -= i
        return a[i:i + th, j:j + tw], _clip_boxes(b, tw, th)


class RandomResizedCropWithBBox(ImageTensorOperation):
    def __init__(self, size, scale=(0.08, 1.0), ratio=(3. / 4., 4. / 3.), interpolation=Inter.BILINEAR,
                 max_attempts=10):
        self.inner = V.RandomResizedCrop(size, scale, ratio, interpolation, max_attempts)

    def _run(self, img, boxes):
        a, b = np.asarray(img), np.array(boxes, dtype=np.float32)
        i, j, ch, cw = self.inner._box(*a.shape[:2])
        b[:, 0] -= j
        b[:, 1] -= i
        b = _clip_boxes(b, cw, ch)
        out = _np_img(_pil(a[i:i + ch, j:j + cw]).resize((self.inner.size[1], self.inner.size[0]),
                                                          _resample(self.inner.interp)), a)
        b[:, [0, 2]] *= self.inner.size[1] / cw
        b[:, [1, 3]] *= self.inner.size[0] / ch
        return out, b


class BoundingBoxAugment(ImageTensorOperation):
    """Applies ``transform`` to the image region of a ``ratio`` share of the boxes."""

    def __init__(self, transform, ratio=0.3):
        if not 0 <= ratio <= 1:
            raise ValueError("BoundingBoxAugment: ratio must be in [0, 1]")
        self.t, self.ratio = transform, ratio

    def _run(self, img, boxes):
        a, b = np.array(img), np.asarray(boxes, dtype=np.float32)
        n = int(round(len(b) * self.ratio))
        for k in np.random.permutation(len(b))[:n]:
            x, y, w, h = (int(v) for v in b[k, :4])
            region = a[y:y + h, x:x + w]
            if region.size:
                a[y:y + h, x:x + w] = np.asarray(self.t(region)).reshape(region.shape)
        return a, b


# ---------------------------------------------------------------------------------------------------- policies
def _shear_x(img, v):
    return Affine(0, (0, 0), 1.0, (math.degrees(math.atan(v)), 0.0), Inter.NEAREST)(img)


def _shear_y(img, v):
    return Affine(0, (0, 0), 1.0, (0.0, math.degrees(math.atan(v))), Inter.NEAREST)(img)


_OPS = {
    "ShearX": (lambda img, m: _shear_x(img, m), 0.3, True), "ShearY": (lambda img, m: _shear_y(img, m), 0.3, True),
    "TranslateX": (lambda img, m: Affine(0, (m, 0.0), 1.0, 0.0)(img), 0.45, True),
    "TranslateY": (lambda img, m: Affine(0, (0.0, m), 1.0, 0.0)(img), 0.45, True),
    "Rotate": (lambda img, m: V.Rotate(m)(img), 30.0, True),
    "Brightness": (lambda img, m: V._enhance("Brightness", img, 1.0 + m), 0.9, True),
    "Color": (lambda img, m: V._enhance("Color", img, 1.0 + m), 0.9, True),
    "Contrast": (lambda img, m: V._enhance("Contrast", img, 1.0 + m), 0.9, True),
    "Sharpness": (lambda img, m: V._enhance("Sharpness", img, 1.0 + m), 0.9, True),
    "Posterize": (lambda img, m: Posterize(int(m))(img), None, False),
    "Solarize": (lambda img, m: Solarize((int(m), 255))(img), None, False),
    "AutoContrast": (lambda img, m: V.AutoContrast()(img), None, False),
    "Equalize": (lambda img, m: V.Equalize()(img), None, False),
    "Invert": (lambda img, m: V.Invert()(img), None, False), "Identity": (lambda img, m: np.asarray(img), None, False),
}


def _magnitude(name, level, bins):
    """The op's parameter at ``level`` of ``bins`` levels (signed ops pick a random sign)."""
    _, top, signed = _OPS[name]
    if name == "Posterize":
        return 8 - int(round(level / max(bins - 1, 1) * 4))
    if name == "Solarize":
        return 255.0 - level / max(bins - 1, 1) * 255.0
    if top is None:
        return 0.0
    m = level / max(bins - 1, 1) * top
    return -m if signed and np.random.random() < 0.5 else m


_POLICIES = {
    "imagenet": [(("Posterize", 0.4, 8), ("Rotate", 0.6, 9)), (("Solarize", 0.6, 5), ("AutoContrast", 0.6, None)),
                 (("Equalize", 0.8, None), ("Equalize", 0.6, None)), (("Posterize", 0.6, 7), ("Posterize", 0.6, 6)),
                 (("Equalize", 0.4, None), ("Solarize", 0.2, 4)), (("Equalize", 0.4, None), ("Rotate", 0.8, 8)),
                 (("Solarize", 0.6, 3), ("Equalize", 0.6, None)), (("Posterize", 0.8, 5), ("Equalize", 1.0, None)),
                 (("Rotate", 0.2, 3), ("Solarize", 0.6, 8)), (("Equalize", 0.6, None), ("Posterize", 0.4, 6)),
                 (("Rotate", 0.8, 8), ("Color", 0.4, 0)), (("Rotate", 0.4, 9), ("Equalize", 0.6, None)),
                 (("Equalize", 0.0, None), ("Equalize", 0.8, None)), (("Invert", 0.6, None), ("Equalize", 1.0, None)),
                 (("Color", 0.6, 4), ("Contrast", 1.0, 8)), (("Rotate", 0.8, 8), ("Color", 1.0, 2)),
                 (("Color", 0.8, 8), ("Solarize", 0.8, 7)), (("Sharpness", 0.4, 7), ("Invert", 0.6, None)),
                 (("ShearX", 0.6, 5), ("Equalize", 1.0, None)), (("Color", 0.4, 0), ("Equalize", 0.6, None)),
                 (("Equalize", 0.4, None), ("Solarize", 0.2, 4)), (("Solarize", 0.6, 5), ("AutoContrast", 0.6, None)),
                 (("Invert", 0.6, None), ("Equalize", 1.0, None)), (("Color", 0.6, 4), ("Contrast", 1.0, 8)),
                 (("Equalize", 0.8, None), ("Equalize", 0.6, None))],
    "cifar10": [(("Invert", 0.1, None), ("Contrast", 0.2, 6)), (("Rotate", 0.7, 2), ("TranslateX", 0.3, 9)),
                (("Sharpness", 0.8, 1), ("Sharpness", 0.9, 3)), (("ShearY", 0.5, 8), ("TranslateY", 0.7, 9)),
                (("AutoContrast", 0.5, None), ("Equalize", 0.9, None)), (("ShearY", 0.2, 7), ("Posterize", 0.3, 7)),
                (("Color", 0.4, 3), ("Brightness", 0.6, 7)), (("Sharpness", 0.3, 9), ("Brightness", 0.7, 9)),
                (("Equalize", 0.6, None), ("Equalize", 0.5, None)), (("Contrast", 0.6, 7), ("Sharpness", 0.6, 5)),
                (("Color", 0.7, 7), ("TranslateX", 0.5, 8)), (("Equalize", 0.3, None), ("AutoContrast", 0.4, None)),
                (("TranslateY", 0.4, 3), ("Sharpness", 0.2, 6)), (("Brightness", 0.9, 6), ("Color", 0.2, 8)),
                (("Solarize", 0.5, 2), ("Invert", 0.0, None)), (("Equalize", 0.2, None), ("AutoContrast", 0.6, None)),
                (("Equalize", 0.2, None), ("Equalize", 0.6, None)), (("Color", 0.9, 9), ("Equalize", 0.6, None)),
                (("AutoContrast", 0.8, None), ("Solarize", 0.2, 8)), (("Brightness", 0.1, 3), ("Color", 0.7, 0)),
                (("Solarize", 0.4, 5), ("AutoContrast", 0.9, None)), (("TranslateY", 0.9, 9), ("TranslateY", 0.7, 9)),
                (("AutoContrast", 0.9, None), ("Solarize", 0.8, 3)), (("Equalize", 0.8, None), ("Invert", 0.1, None)),
                (("TranslateY", 0.7, 9), ("AutoContrast", 0.9, None))],
    "svhn": [(("ShearX", 0.9, 4), ("Invert", 0.2, None)), (("ShearY", 0.9, 8), ("Invert", 0.7, None)),
             (("Equalize", 0.6, None), ("Solarize", 0.6, 6)), (("Invert", 0.9, None), ("Equalize", 0.6, None)),
             (("Equalize", 0.6, None), ("Rotate", 0.9, 3)), (("ShearX", 0.9, 4), ("AutoContrast", 0.8, None)),
             (("ShearY", 0.9, 8), ("Invert", 0.4, None)), (("ShearY", 0.9, 5), ("Solarize", 0.2, 6)),
             (("Invert", 0.9, None), ("AutoContrast", 0.8, None)), (("Equalize", 0.6, None), ("Rotate", 0.9, 3)),
             (("ShearX", 0.9, 4), ("Solarize", 0.3, 3)), (("ShearY", 0.8, 8), ("Invert", 0.7, None)),
             (("Equalize", 0.9, None), ("TranslateY", 0.6, 6)), (("Invert", 0.9, None), ("Equalize", 0.6, None)),
             (("Contrast", 0.3, 3), ("Rotate", 0.8, 4)), (("Invert", 0.8, None), ("TranslateY", 0.0, 2)),
             (("ShearY", 0.7, 6), ("Solarize", 0.4, 8)), (("Invert", 0.6, None), ("Rotate", 0.8, 4)),
             (("ShearY", 0.3, 7), ("TranslateX", 0.9, 3)), (("ShearX", 0.1, 6), ("Invert", 0.6, None)),
             (("Solarize", 0.7, 2), ("TranslateY", 0.6, 7)), (("ShearY", 0.8, 4), ("Invert", 0.8, None)),
             (("ShearX", 0.7, 9), ("TranslateY", 0.8, 3)), (("ShearY", 0.8, 5), ("AutoContrast", 0.7, None)),
             (("ShearX", 0.7, 2), ("Invert", 0.1, None))],
}


class AutoAugment(ImageTensorOperation):
    """One of the learned sub-policies (two ops, each with a probability and a magnitude level out of 10) of the
    chosen policy set, picked at random per image."""

    def __init__(self, policy=AutoAugmentPolicy.IMAGENET, interpolation=Inter.NEAREST, fill_value=0):
        self.policies = _POLICIES[AutoAugmentPolicy(policy).value if not isinstance(policy, str) else policy]

    def _run(self, img):
        a = np.asarray(img)
        for name, prob, level in self.policies[np.random.randint(len(self.policies))]:
            if np.random.random() < prob:
                a = _OPS[name][0](a, _magnitude(name, level if level is not None else 0, 10))
        return a


class RandAugment(ImageTensorOperation):
    def __init__(self, num_ops=2, magnitude=9, num_magnitude_bins=31, interpolation=Inter.NEAREST, fill_value=0):
        if magnitude >= num_magnitude_bins:
            raise ValueError("RandAugment: magnitude must be smaller than num_magnitude_bins")
        self.n, self.mag, self.bins = num_ops, magnitude, num_magnitude_bins
        self.names = [n for n in _OPS if n != "Invert"]

    def _run(self, img):
        a = np.asarray(img)
        for _ in range(self.n):
            name = self.names[np.random.randint(len(self.names))]
            a = _OPS[name][0](a, _magnitude(name, self.mag, self.bins))
        return a


class TrivialAugmentWide(ImageTensorOperation):
    def __init__(self, num_magnitude_bins=31, interpolation=Inter.NEAREST, fill_value=0):
        if num_magnitude_bins < 2:
            raise ValueError("TrivialAugmentWide: num_magnitude_bins must be at least 2")
        self.bins, self.names = num_magnitude_bins, [n for n in _OPS if n != "Invert"]

    def _run(self, img):
        name = self.names[np.random.randint(len(self.names))]
        return _OPS[name][0](np.asarray(img), _magnitude(name, np.random.randint(self.bins), self.bins))


class UniformAugment(ImageTensorOperation):
    """Applies ``num_ops`` transforms drawn uniformly from ``transforms``, each with probability 1/2."""

    def __init__(self, transforms, num_ops=2):
        if num_ops <= 0 or num_ops > len(transforms):
            raise ValueError("UniformAugment: num_ops must be in [1, len(transforms)]")
        self.transforms, self.n = list(transforms), num_ops

    def _run(self, img):
        a = np.asarray(img)
        for k in np.random.permutation(len(self.transforms))[:self.n]:
            if np.random.random() < 0.5:
                a = self.transforms[k](a)
        return a


class RandomSelectSubpolicy(ImageTensorOperation):
    """``policy`` = list of sub-policies, each a list of (transform, probability); one sub-policy runs per image."""

    def __init__(self, policy):
        if not policy or not all(policy):
            raise ValueError("RandomSelectSubpolicy: policy must be a non-empty list of non-empty lists")
        self.policy = policy

    def _run(self, img):
        a = np.asarray(img)
        for t, p in self.policy[np.random.randint(len(self.policy))]:
            if np.random.random() < p:
                a = t(a)
        return a


# ---------------------------------------------------------------------------------------------------- files
def read_file(filename):
    return np.fromfile(filename, dtype=np.uint8)


def write_file(filename, data):
    np.asarray(data, dtype=np.uint8).tofile(filename)


def read_image(filename, mode=ImageReadMode.UNCHANGED):
    from PIL import Image
    with Image.open(filename) as im:
        m = ImageReadMode(mode)
        if m == ImageReadMode.GRAYSCALE:
            return np.asarray(im.convert("L"))[..., None]
        if m == ImageReadMode.COLOR:
            return np.asarray(im.convert("RGB"))
        return np.asarray(im)


def _encode(image, fmt, **kw):
    import io
    buf = io.BytesIO()
    _pil(image).save(buf, fmt, **kw)
    return np.frombuffer(buf.getvalue(), dtype=np.uint8)


def encode_jpeg(image, quality=75):
    if not 1 <= quality <= 100:
        raise ValueError("encode_jpeg: quality must be in [1, 100]")
    return _encode(image, "JPEG", quality=quality)


def encode_png(image, compression_level=6):
    if not 0 <= compression_level <= 9:
        raise ValueError("encode_png: compression_level must be in [0, 9]")
    return _encode(image, "PNG", compress_level=compression_level)


def write_jpeg(filename, image, quality=75):
    write_file(filename, encode_jpeg(image, quality))


def write_png(filename, image, compression_level=6):
    write_file(filename, encode_png(image, compression_level))


def get_image_num_channels(image):
    from PIL import Image
    if isinstance(image, Image.Image):
        return len(image.getbands())
    a = np.asarray(image)
    if a.ndim == 2:
        return 1
    if a.ndim == 3:
        return a.shape[-1]
    raise RuntimeError("get_image_num_channels: invalid image of shape %s" % (a.shape,))


def get_image_size(image):
    from PIL import Image
    if isinstance(image, Image.Image):
        return [image.size[1], image.size[0]]
    a = np.asarray(image)
    if a.ndim < 2:
        raise RuntimeError("get_image_size: invalid image of shape %s" % (a.shape,))
    return [a.shape[0], a.shape[1]]


def parse_padding(padding):
    if isinstance(padding, int):
        return (padding,) * 4
    p = tuple(padding)
    if len(p) == 2:
        return (p[0], p[1], p[0], p[1])
    if len(p) == 4:
        return p
    raise ValueError("padding must be an int or a sequence of 2 or 4 ints, but got %r" % (padding,))


def read_video(filename, start_pts=0, end_pts=None, pts_unit="pts"):
    raise NotImplementedError("read_video needs a video decoder (ffmpeg bindings), which this build does not ship")


def read_video_timestamps(filename, pts_unit="pts"):
    raise NotImplementedError("read_video_timestamps needs a video decoder, which this build does not ship")


__all__ = [n for n, v in list(globals().items()) if not n.startswith("_") and (
    (isinstance(v, type) and v.__module__ == __name__) or (callable(v) and getattr(v, "__module__", "") == __name__))]
