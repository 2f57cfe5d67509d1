"""Dataset helpers: ``LineReader`` (random access to the lines of a large text file through an index of line
offsets built in one pass) and ``imshow_det_bbox`` (draws detection boxes, labels and masks into an image; there is
no window system here, so the picture is returned and written to ``out_file``).

Parity: mindspore/python/mindspore/dataset/utils/{line_reader,browse_dataset}.py.
"""
import os

import numpy as np

__all__ = ["LineReader", "imshow_det_bbox"]


class LineReader:
    """``reader[n]`` / ``reader.readline(n)`` return line ``n`` (1-based) without its line end."""

    def __init__(self, filename):
        if not isinstance(filename, str):
            raise TypeError("Parameter filename should be string.")
        if not os.path.isfile(filename):
            raise RuntimeError("The input file %s does not exist." % filename)
        self.filename = os.path.realpath(filename)
        self.fo = open(self.filename, "rb")
        self.offsets = []                                    # byte offset of the start of every line
        pos = 0
        for line in self.fo:
            self.offsets.append(pos)
            pos += len(line)

    def __getitem__(self, line):
        return self.readline(line)

    def __len__(self):
        return len(self.offsets)

    def len(self):
        return len(self.offsets)

    def readline(self, line):
        if isinstance(line, bool) or not isinstance(line, int):
            raise TypeError("Parameter line should be integer.")
        if line < 1 or line > len(self.offsets):
            raise ValueError("Parameter line exceeds the file length.")
        self.fo.seek(self.offsets[line - 1])
        return self.fo.readline().decode("utf-8").rstrip("\r\n")

    def close(self):
        if self.fo is not None and not self.fo.closed:
            self.fo.close()

    def __del__(self):
        try:
            self.close()
        except Exception:                                                                   # noqa: BLE001
            pass


def _check_color(value, name):
    if not isinstance(value, (tuple, list)) or len(value) != 3 or not all(
            isinstance(v, int) and 0 <= v <= 255 for v in value):
        raise ValueError("%s should be a tuple of three ints in [0, 255], but got %r" % (name, value))
    return tuple(value)


def imshow_det_bbox(image, bboxes, labels, segm=None, class_names=None, score_threshold=0, bbox_color=(0, 255, 0),
                    text_color=(203, 192, 255), mask_color=(128, 0, 128), thickness=2, font_size=0.8, show=True,
                    win_name="win", wait_time=2000, out_file=None):
    """Returns the HWC uint8 picture with boxes ``<x, y, w, h[, score]>``, their labels and, with ``segm`` (one HW
    mask per box), the masks blended in.  ``show`` / ``win_name`` / ``wait_time`` are accepted; nothing is displayed."""
    from PIL import Image, ImageDraw
    image = np.asarray(image)
    if image.ndim != 3:
        raise ValueError("image should have 3 dimensions, but got %d" % image.ndim)
    if image.shape[0] == 3 and image.shape[2] != 3:
        image = image.transpose(1, 2, 0)
    if image.shape[2] != 3:
        raise ValueError("image should be <C, H, W> or <H, W, C> with 3 channels, but got shape %s" % (image.shape,))
    bboxes = np.asarray(bboxes)
    labels = np.asarray(labels).reshape(-1)
    if bboxes.ndim != 2 or bboxes.shape[1] not in (4, 5):
        raise ValueError("bboxes should be shaped <N, 4> or <N, 5>, but got %s" % (bboxes.shape,))
    if bboxes.shape[0] != labels.shape[0]:
        raise ValueError("bboxes and labels should have the same length")
    if class_names is not None and not isinstance(class_names, (list, tuple, dict)):
        raise TypeError("class_names should be a list, a tuple or a dict")
    bbox_color, text_color = _check_color(bbox_color, "bbox_color"), _check_color(text_color, "text_color")
    mask_color = _check_color(mask_color, "mask_color")
    if image.dtype != np.uint8:
        image = np.clip(image * (255.0 if image.max() <= 1.0 else 1.0), 0, 255).astype(np.uint8)
    keep = np.ones(len(labels), bool)
    if bboxes.shape[1] == 5 and score_threshold > 0:
        keep = bboxes[:, 4] > score_threshold
    canvas = image.copy()
    if segm is not None:
        segm = np.asarray(segm).astype(bool)
        if segm.ndim != 3 or segm.shape[1:] != image.shape[:2]:
            raise ValueError("segm should be shaped <M, H, W> matching the image, but got %s" % (segm.shape,))
        for k in np.nonzero(keep[:len(segm)])[0]:
            canvas[segm[k]] = (0.5 * canvas[segm[k]] + 0.5 * np.array(mask_color)).astype(np.uint8)
    pic = Image.fromarray(canvas)
    draw = ImageDraw.Draw(pic)
    for box, label in zip(bboxes[keep], labels[keep]):
        x, y, w, h = (float(v) for v in box[:4])
        draw.rectangle([x, y, x + w, y + h], outline=bbox_color, width=int(thickness))
        if class_names is None:
            text = "class %s" % int(label)
        elif isinstance(class_names, dict):
            text = str(class_names.get(int(label), int(label)))
        else:
            text = str(class_names[int(label)])
        if len(box) == 5:
            text += "|%.2f" % box[4]
        draw.text((x, max(y - 12, 0)), text, fill=text_color)
    out = np.asarray(pic)
    if out_file is not None:
        pic.save(out_file)
    return out
