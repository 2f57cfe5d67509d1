"""More source datasets: the public vision / text / audio corpora in the on-disk layouts their distributors use,
plus ``TFRecordDataset``, ``PaddedDataset``, ``FakeImageDataset``, ``ManifestDataset`` and ``Schema``.

Every class is a random-access source under ``GeneratorDataset`` (so ``shuffle`` / ``sampler`` / ``num_shards`` /
``num_samples`` behave alike).  Images come back as the encoded file bytes unless ``decode=True``; audio comes back
as ``waveform`` float32 [channels, samples] with ``sample_rate``.  Parity: python/mindspore/dataset/engine/
datasets_vision.py, datasets_text.py, datasets_audio.py, datasets_standard_format.py, datasets_user_defined.py."""
from __future__ import annotations

import csv
import json
import os
import re
import struct

import numpy as np

from .engine import GeneratorDataset
from .sources import _find, _Indexed, _read_idx

__all__ = []


def _export(cls):
    __all__.append(cls.__name__)
    return cls


def _check_usage(who, usage, allowed, default="all"):
    usage = usage or default
    if usage not in allowed:
        raise ValueError("For '%s', 'usage' must be one of %s, but got %r" % (who, sorted(allowed), usage))
    return usage


def _image(path, decode):
    if decode:
        from PIL import Image
        with Image.open(path) as im:
            return np.asarray(im.convert("RGB"))
    return np.fromfile(path, dtype=np.uint8)


def _wav(path):
    """(float32 [channels, samples] in [-1, 1], sample rate) of a PCM wav file."""
    import wave
    with wave.open(path, "rb") as w:
        n, ch, width, rate = w.getnframes(), w.getnchannels(), w.getsampwidth(), w.getframerate()
        raw = w.readframes(n)
    if width == 2:
        data = np.frombuffer(raw, dtype="<i2").astype(np.float32) / 32768.0
    elif width == 4:
        data = np.frombuffer(raw, dtype="<i4").astype(np.float32) / 2147483648.0
    elif width == 1:
        data = (np.frombuffer(raw, dtype=np.uint8).astype(np.float32) - 128.0) / 128.0
    else:
        raise ValueError("%s: unsupported sample width %d" % (path, width))
    return data.reshape(-1, ch).T.copy(), rate


class _Rows:
    """Random-access source from a list of records and a loader ``load(record) -> tuple``."""

    def __init__(self, records, load, labels=None):
        self.records, self.load = records, load
        self.labels = labels

    def __len__(self):
        return len(self.records)

    def __getitem__(self, i):
        return self.load(self.records[i])


def _init(self, source, columns, kw):
    GeneratorDataset.__init__(self, source, columns, num_samples=kw.get("num_samples"), shuffle=kw.get("shuffle"),
                              sampler=kw.get("sampler"), num_shards=kw.get("num_shards"), shard_id=kw.get("shard_id"))


def _kw(num_samples=None, num_parallel_workers=None, shuffle=None, sampler=None, num_shards=None, shard_id=None,
        cache=None, **extra):
    return dict(num_samples=num_samples, shuffle=shuffle, sampler=sampler, num_shards=num_shards, shard_id=shard_id)


# ---------------------------------------------------------------------------------------------------- idx / binary vision
def _idx_dataset(name, train_prefix, test_prefix, doc):
    def __init__(self, dataset_dir, usage=None, **kw):
        usage = _check_usage(name, usage, ("train", "test", "all"))
        imgs, labs = [], []
        for part, prefix in (("train", train_prefix), ("test", test_prefix)):
            if usage in (part, "all"):
                imgs.append(_read_idx(_find(dataset_dir, [prefix + "-images-idx3-ubyte", prefix + "-images.idx3-ubyte"])))
                labs.append(_read_idx(_find(dataset_dir, [prefix + "-labels-idx1-ubyte", prefix + "-labels.idx1-ubyte"])))
        images = np.concatenate(imgs)[..., None]
        labels = np.concatenate(labs).astype(np.uint32)
        _init(self, _Indexed([images, labels], labels), ["image", "label"], _kw(**kw))
    return _export(type(name, (GeneratorDataset,), {"__init__": __init__, "__doc__": doc}))


FashionMnistDataset = _idx_dataset("FashionMnistDataset", "train", "t10k",
                                   "Fashion-MNIST idx files: ``image`` uint8 [28, 28, 1], ``label`` uint32.")
KMnistDataset = _idx_dataset("KMnistDataset", "train", "t10k",
                             "Kuzushiji-MNIST idx files: ``image`` uint8 [28, 28, 1], ``label`` uint32.")


@_export
class EMnistDataset(GeneratorDataset):
    """EMNIST split ``name`` ('byclass', 'bymerge', 'balanced', 'letters', 'digits', 'mnist') from
    ``emnist-<name>-{train,test}-{images-idx3,labels-idx1}-ubyte``."""

    def __init__(self, dataset_dir, name, usage=None, **kw):
        if name not in ("byclass", "bymerge", "balanced", "letters", "digits", "mnist"):
            raise ValueError("For 'EMnistDataset', 'name' %r is not an EMNIST split" % (name,))
        usage = _check_usage("EMnistDataset", usage, ("train", "test", "all"))
        imgs, labs = [], []
        for part in ("train", "test"):
            if usage in (part, "all"):
                imgs.append(_read_idx(_find(dataset_dir, ["emnist-%s-%s-images-idx3-ubyte" % (name, part)])))
                labs.append(_read_idx(_find(dataset_dir, ["emnist-%s-%s-labels-idx1-ubyte" % (name, part)])))
        labels = np.concatenate(labs).astype(np.uint32)
        _init(self, _Indexed([np.concatenate(imgs)[..., None], labels], labels), ["image", "label"], _kw(**kw))


@_export
class QMnistDataset(GeneratorDataset):
    """QMNIST: ``qmnist-{train,test,test10k,test50k}-images-idx3-ubyte`` and the idx2-int label files whose first
    column is the class (all eight columns with ``compat=False``)."""

    def __init__(self, dataset_dir, usage=None, compat=True, **kw):
        usage = _check_usage("QMnistDataset", usage, ("train", "test", "test10k", "test50k", "nist", "all"), "train")
        parts = ["train", "test"] if usage == "all" else ["xnist" if usage == "nist" else usage]
        imgs, labs = [], []
        for part in parts:
            base = "qmnist-%s" % part if part != "xnist" else "xnist"
            imgs.append(_read_idx(_find(dataset_dir, [base + "-images-idx3-ubyte"])))
            path = _find(dataset_dir, [base + "-labels-idx2-int"])
            with (open(path, "rb") if not path.endswith(".gz") else __import__("gzip").open(path, "rb")) as f:
                data = f.read()
            rows, cols = struct.unpack_from(">II", data, 4)
            labs.append(np.frombuffer(data, dtype=">i4", offset=12).reshape(rows, cols).astype(np.uint32))
        lab = np.concatenate(labs)
        labels = lab[:, 0] if compat else lab
        _init(self, _Indexed([np.concatenate(imgs)[..., None], labels], lab[:, 0]), ["image", "label"], _kw(**kw))


@_export
class Cifar100Dataset(GeneratorDataset):
    """``train.bin`` / ``test.bin``: columns ``image`` uint8 [32, 32, 3], ``coarse_label`` and ``fine_label`` uint32."""

    def __init__(self, dataset_dir, usage=None, **kw):
        usage = _check_usage("Cifar100Dataset", usage, ("train", "test", "all"))
        files = [f for f in ("train.bin", "test.bin") if usage in (f[:-4], "all")]
        rows = np.concatenate([np.fromfile(os.path.join(dataset_dir, f), dtype=np.uint8).reshape(-1, 3074)
                               for f in files])
        coarse, fine = rows[:, 0].astype(np.uint32), rows[:, 1].astype(np.uint32)
        images = rows[:, 2:].reshape(-1, 3, 32, 32).transpose(0, 2, 3, 1)
        _init(self, _Indexed([images, coarse, fine], fine), ["image", "coarse_label", "fine_label"], _kw(**kw))


@_export
class STL10Dataset(GeneratorDataset):
    """``{train,test,unlabeled}_X.bin`` (uint8 [N, 3, 96, 96] column-major images) and ``_y.bin`` (labels 1..10)."""

    def __init__(self, dataset_dir, usage=None, **kw):
        usage = _check_usage("STL10Dataset", usage, ("train", "test", "unlabeled", "train+unlabeled", "all"))
        parts = {"all": ["train", "test", "unlabeled"], "train+unlabeled": ["train", "unlabeled"]}.get(usage, [usage])
        imgs, labs = [], []
        for part in parts:
            x = np.fromfile(os.path.join(dataset_dir, part + "_X.bin"), dtype=np.uint8).reshape(-1, 3, 96, 96)
            imgs.append(x.transpose(0, 3, 2, 1))
            ypath = os.path.join(dataset_dir, part + "_y.bin")
            labs.append(np.fromfile(ypath, dtype=np.uint8).astype(np.int32) - 1 if os.path.exists(ypath)
                        else np.full(x.shape[0], -1, dtype=np.int32))
        labels = np.concatenate(labs)
        _init(self, _Indexed([np.concatenate(imgs), labels], labels), ["image", "label"], _kw(**kw))


@_export
class SVHNDataset(GeneratorDataset):
    """``{train,test,extra}_32x32.mat`` (X [32, 32, 3, N], y with 10 meaning digit 0)."""

    def __init__(self, dataset_dir, usage=None, **kw):
        import scipy.io
        usage = _check_usage("SVHNDataset", usage, ("train", "test", "extra", "all"))
        parts = ["train", "test", "extra"] if usage == "all" else [usage]
        imgs, labs = [], []
        for part in parts:
            m = scipy.io.loadmat(os.path.join(dataset_dir, part + "_32x32.mat"))
            imgs.append(np.transpose(m["X"], (3, 0, 1, 2)))
            y = m["y"].reshape(-1).astype(np.uint32)
            labs.append(np.where(y == 10, 0, y).astype(np.uint32))
        labels = np.concatenate(labs)
        _init(self, _Indexed([np.concatenate(imgs), labels], labels), ["image", "label"], _kw(**kw))


@_export
class USPSDataset(GeneratorDataset):
    """``usps`` / ``usps.t`` (optionally .bz2) in libsvm text: label then 256 ``index:value`` pairs in [-1, 1]."""

    def __init__(self, dataset_dir, usage=None, **kw):
        import bz2
        usage = _check_usage("USPSDataset", usage, ("train", "test", "all"))
        imgs, labs = [], []
        for part, name in (("train", "usps"), ("test", "usps.t")):
            if usage not in (part, "all"):
                continue
            path = os.path.join(dataset_dir, name)
            opener = open
            if not os.path.exists(path):
                path, opener = path + ".bz2", bz2.open
            with opener(path, "rt") as f:
                for line in f:
                    tok = line.split()
                    if not tok:
                        continue
                    labs.append(int(tok[0]) - 1)
                    px = np.zeros(256, dtype=np.float32)
                    for t in tok[1:]:
                        k, v = t.split(":")
                        px[int(k) - 1] = float(v)
                    imgs.append(((px + 1) / 2 * 255).astype(np.uint8).reshape(16, 16, 1))
        labels = np.array(labs, dtype=np.uint32)
        _init(self, _Indexed([np.stack(imgs), labels], labels), ["image", "label"], _kw(**kw))


@_export
class SemeionDataset(GeneratorDataset):
    """``semeion.data``: 256 pixel values then a ten-way one-hot label per line."""

    def __init__(self, dataset_dir, **kw):
        data = np.loadtxt(os.path.join(dataset_dir, "semeion.data"))
        images = (data[:, :256] * 255).astype(np.uint8).reshape(-1, 16, 16)
        labels = data[:, 256:].argmax(1).astype(np.uint32)
        _init(self, _Indexed([images, labels], labels), ["image", "label"], _kw(**kw))


@_export
class FakeImageDataset(GeneratorDataset):
    """``num_images`` random images of ``image_size`` (H, W, C) with labels below ``num_classes``; image i is drawn
    from seed ``base_seed + i``, so the data do not depend on the visiting order."""

    def __init__(self, num_images=1000, image_size=(224, 224, 3), num_classes=10, base_seed=0, **kw):
        size = tuple(image_size)

        def load(i):
            rng = np.random.default_rng(base_seed + i)
            return (rng.integers(0, 256, size, dtype=np.uint8), np.uint32(rng.integers(0, num_classes)))
        _init(self, _Rows(list(range(num_images)), load), ["image", "label"], _kw(**kw))


# ---------------------------------------------------------------------------------------------------- folder vision
def _class_folder_dataset(name, subdir, doc, skip=()):
    def __init__(self, dataset_dir, usage=None, decode=False, target_type=None, **kw):
        root = os.path.join(dataset_dir, subdir) if subdir and os.path.isdir(os.path.join(dataset_dir, subdir)) \
            else dataset_dir
        if usage in ("train", "val", "valid", "test") and os.path.isdir(os.path.join(root, usage)):
            root = os.path.join(root, usage)
        classes = sorted(d for d in os.listdir(root) if os.path.isdir(os.path.join(root, d)) and d not in skip)
        records = [(os.path.join(root, c, f), i) for i, c in enumerate(classes)
                   for f in sorted(os.listdir(os.path.join(root, c)))
                   if os.path.isfile(os.path.join(root, c, f))]
        self._classes = classes
        labels = np.array([l for _, l in records], dtype=np.int32)
        _init(self, _Rows(records, lambda r: (_image(r[0], decode), np.int32(r[1])), labels), ["image", "label"],
              _kw(**kw))

    def get_class_indexing(self):
        return {c: i for i, c in enumerate(self._classes)}
    return _export(type(name, (GeneratorDataset,), {"__init__": __init__, "get_class_indexing": get_class_indexing,
                                                    "__doc__": doc}))


Caltech101Dataset = _class_folder_dataset("Caltech101Dataset", "101_ObjectCategories",
                                          "``101_ObjectCategories/<class>/*.jpg`` (BACKGROUND_Google skipped).",
                                          ("BACKGROUND_Google",))
Caltech256Dataset = _class_folder_dataset("Caltech256Dataset", "256_ObjectCategories",
                                          "``256_ObjectCategories/<nnn.class>/*.jpg``.")
RenderedSST2Dataset = _class_folder_dataset("RenderedSST2Dataset", "rendered-sst2",
                                            "``<usage>/{negative,positive}/*.png``.")
SUN397Dataset = _class_folder_dataset("SUN397Dataset", "SUN397", "``SUN397/<letter>/...`` one folder per scene class.")
Places365Dataset = _class_folder_dataset("Places365Dataset", "", "``<usage folder>/<class>/*.jpg``.")
LSUNDataset = _class_folder_dataset("LSUNDataset", "", "``<class>_<usage>/`` folders of images.")
EuroSATDataset = _class_folder_dataset("EuroSATDataset", "2750", "``2750/<class>/*.jpg``.")


@_export
class OmniglotDataset(GeneratorDataset):
    """``images_background`` (``background=True``) or ``images_evaluation``: ``<alphabet>/<character>/*.png``; the
    label numbers the (alphabet, character) pairs in sorted order."""

    def __init__(self, dataset_dir, background=True, decode=False, **kw):
        root = os.path.join(dataset_dir, "images_background" if background else "images_evaluation")
        records, label = [], 0
        for alpha in sorted(os.listdir(root)):
            for ch in sorted(os.listdir(os.path.join(root, alpha))):
                d = os.path.join(root, alpha, ch)
                if not os.path.isdir(d):
                    continue
                records += [(os.path.join(d, f), label) for f in sorted(os.listdir(d))]
                label += 1
        labels = np.array([l for _, l in records], dtype=np.int32)
        _init(self, _Rows(records, lambda r: (_image(r[0], decode), np.int32(r[1])), labels), ["image", "label"],
              _kw(**kw))


@_export
class Food101Dataset(GeneratorDataset):
    """``meta/{train,test}.txt`` lists ``<class>/<id>``; images under ``images/``.  ``label`` is the class name."""

    def __init__(self, dataset_dir, usage=None, decode=False, **kw):
        usage = _check_usage("Food101Dataset", usage, ("train", "test", "all"))
        ids = []
        for part in ("train", "test"):
            if usage in (part, "all"):
                with open(os.path.join(dataset_dir, "meta", part + ".txt")) as f:
                    ids += [ln.strip() for ln in f if ln.strip()]
        classes = sorted({i.split("/")[0] for i in ids})
        labels = np.array([classes.index(i.split("/")[0]) for i in ids], dtype=np.int32)
        _init(self, _Rows(ids, lambda i: (_image(os.path.join(dataset_dir, "images", i + ".jpg"), decode),
                                          np.array(i.split("/")[0])), labels), ["image", "label"], _kw(**kw))


@_export
class Flowers102Dataset(GeneratorDataset):
    """``jpg/image_<nnnnn>.jpg``, ``imagelabels.mat`` (labels 1..102) and ``setid.mat`` (trnid / valid / tstid)."""

    def __init__(self, dataset_dir, task="Classification", usage="all", decode=False, **kw):
        import scipy.io
        usage = _check_usage("Flowers102Dataset", usage, ("train", "valid", "test", "all"))
        labels_all = scipy.io.loadmat(os.path.join(dataset_dir, "imagelabels.mat"))["labels"].reshape(-1)
        split = scipy.io.loadmat(os.path.join(dataset_dir, "setid.mat"))
        keys = {"train": ["trnid"], "valid": ["valid"], "test": ["tstid"], "all": ["trnid", "valid", "tstid"]}[usage]
        ids = np.concatenate([split[k].reshape(-1) for k in keys])
        labels = (labels_all[ids - 1] - 1).astype(np.uint32)
        _init(self, _Rows(list(zip(ids.tolist(), labels.tolist())), lambda r: (
            _image(os.path.join(dataset_dir, "jpg", "image_%05d.jpg" % r[0]), decode), np.uint32(r[1])), labels),
            ["image", "label"], _kw(**kw))


@_export
class CelebADataset(GeneratorDataset):
    """``list_attr_celeba.txt`` (count, attribute names, then ``<file> ±1 x 40``) and the images beside it (or under
    ``img_align_celeba``); ``list_eval_partition.txt`` selects ``usage``.  ``attr`` is uint32 [40] of 0 / 1."""

    def __init__(self, dataset_dir, usage="all", decode=False, extensions=None, **kw):
        usage = _check_usage("CelebADataset", usage, ("train", "valid", "test", "all"))
        with open(os.path.join(dataset_dir, "list_attr_celeba.txt")) as f:
            lines = [ln.split() for ln in f if ln.strip()]
        rows = [ln for ln in lines[2:]]
        part = {}
        ppath = os.path.join(dataset_dir, "list_eval_partition.txt")
        if os.path.exists(ppath):
            with open(ppath) as f:
                part = {a: int(b) for a, b in (ln.split() for ln in f if ln.strip())}
        want = {"train": 0, "valid": 1, "test": 2}.get(usage)
        img_dir = os.path.join(dataset_dir, "img_align_celeba")
        img_dir = img_dir if os.path.isdir(img_dir) else dataset_dir
        records = [(os.path.join(img_dir, r[0]), np.array([(int(v) + 1) // 2 for v in r[1:]], dtype=np.uint32))
                   for r in rows if want is None or part.get(r[0], 0) == want]
        _init(self, _Rows(records, lambda r: (_image(r[0], decode), r[1])), ["image", "attr"], _kw(**kw))


@_export
class ManifestDataset(GeneratorDataset):
    """One JSON object per line: ``{"source": path, "usage": "TRAIN", "annotation": [{"name": class}, ...]}``."""

    def __init__(self, dataset_file, usage="train", class_indexing=None, decode=False, **kw):
        records = []
        with open(dataset_file) as f:
            for ln in f:
                if not ln.strip():
                    continue
                rec = json.loads(ln)
                if str(rec.get("usage", "train")).lower() != usage.lower():
                    continue
                names = [a["name"] for a in rec.get("annotation", []) if "name" in a]
                records.append((rec["source"], names[0] if names else ""))
        classes = sorted({c for _, c in records})
        self._index = class_indexing or {c: i for i, c in enumerate(classes)}
        labels = np.array([self._index[c] for _, c in records], dtype=np.int32)
        _init(self, _Rows(records, lambda r: (_image(r[0], decode), np.int32(self._index[r[1]])), labels),
              ["image", "label"], _kw(**kw))

    def get_class_indexing(self):
        return dict(self._index)


@_export
class CocoDataset(GeneratorDataset):
    """COCO annotations.  ``task='Detection'``: ``image``, ``bbox`` float32 [n, 4] (x, y, w, h), ``category_id``
    uint32 [n, 1], ``iscrowd`` uint32 [n, 1]; ``'Keypoint'``: ``image``, ``keypoints`` float32 [n, 51],
    ``num_keypoints``; ``'Stuff'``: ``image``, ``segmentation`` (polygons padded with -1), ``iscrowd``;
    ``'Captioning'``: ``image``, ``captions``.  ``extra_metadata=True`` adds ``_meta-filename``."""

    def __init__(self, dataset_dir, annotation_file, task="Detection", decode=False, extra_metadata=False, **kw):
        if task not in ("Detection", "Stuff", "Panoptic", "Keypoint", "Captioning"):
            raise ValueError("For 'CocoDataset', 'task' %r is not supported" % (task,))
        with open(annotation_file) as f:
            ann = json.load(f)
        by_image = {}
        for a in ann.get("annotations", []):
            by_image.setdefault(a["image_id"], []).append(a)
        cats = ann.get("categories", [])
        self._class_index = {c["name"]: [c["id"]] for c in cats}
        images = [im for im in ann["images"] if by_image.get(im["id"])]

        def load(im):
            anns = by_image[im["id"]]
            img = _image(os.path.join(dataset_dir, im["file_name"]), decode)
            if task == "Detection":
                cols = (img, np.array([a["bbox"] for a in anns], dtype=np.float32).reshape(-1, 4),
                        np.array([[a["category_id"]] for a in anns], dtype=np.uint32),
                        np.array([[a.get("iscrowd", 0)] for a in anns], dtype=np.uint32))
            elif task == "Keypoint":
                cols = (img, np.array([a["keypoints"] for a in anns], dtype=np.float32),
                        np.array([[a.get("num_keypoints", 0)] for a in anns], dtype=np.uint32))
            elif task == "Captioning":
                cols = (img, np.array([a["caption"] for a in anns], dtype=object))
            else:
                polys = [np.asarray(p, dtype=np.float32) for a in anns
                         for p in (a["segmentation"] if isinstance(a.get("segmentation"), list) else [])]
                width = max([len(p) for p in polys] + [1])
                seg = np.full((len(polys), width), -1.0, dtype=np.float32)
                for i, p in enumerate(polys):
                    seg[i, :len(p)] = p
                cols = (img, seg, np.array([[a.get("iscrowd", 0)] for a in anns], dtype=np.uint32))
            return cols + ((np.array(im["file_name"]),) if extra_metadata else ())
        names = {"Detection": ["image", "bbox", "category_id", "iscrowd"],
                 "Keypoint": ["image", "keypoints", "num_keypoints"], "Captioning": ["image", "captions"]}.get(
            task, ["image", "segmentation", "iscrowd"])
        _init(self, _Rows(images, load), names + (["_meta-filename"] if extra_metadata else []), _kw(**kw))

    def get_class_indexing(self):
        return dict(self._class_index)


@_export
class VOCDataset(GeneratorDataset):
    """Pascal VOC: ``ImageSets/{Main,Segmentation}/<usage>.txt`` lists ids.  ``task='Detection'``: ``image``,
    ``bbox`` float32 [n, 4] (xmin, ymin, w, h), ``label`` uint32 [n, 1], ``difficult``, ``truncate`` parsed from
    ``Annotations/<id>.xml``; ``'Segmentation'``: ``image`` and ``target`` (``SegmentationClass/<id>.png``)."""

    def __init__(self, dataset_dir, task="Segmentation", usage="train", class_indexing=None, decode=False,
                 extra_metadata=False, **kw):
        if task not in ("Segmentation", "Detection"):
            raise ValueError("For 'VOCDataset', 'task' must be 'Segmentation' or 'Detection', but got %r" % (task,))
        sets = "Main" if task == "Detection" else "Segmentation"
        with open(os.path.join(dataset_dir, "ImageSets", sets, usage + ".txt")) as f:
            ids = [ln.split()[0] for ln in f if ln.strip()]
        index = dict(class_indexing or {})
        if task == "Detection":
            import xml.etree.ElementTree as ET
            parsed = {}
            for i in ids:
                objs = []
                for o in ET.parse(os.path.join(dataset_dir, "Annotations", i + ".xml")).getroot().iter("object"):
                    b = o.find("bndbox")
                    box = [float(b.find(k).text) for k in ("xmin", "ymin", "xmax", "ymax")]
                    objs.append((o.find("name").text, box, int(getattr(o.find("difficult"), "text", 0) or 0),
                                 int(getattr(o.find("truncated"), "text", 0) or 0)))
                parsed[i] = objs
            if not class_indexing:
                for n in sorted({o[0] for objs in parsed.values() for o in objs}):
                    index[n] = len(index)
            self._index = index

            def load(i):
                objs = [o for o in parsed[i] if o[0] in index]
                box = np.array([[o[1][0], o[1][1], o[1][2] - o[1][0], o[1][3] - o[1][1]] for o in objs],
                               dtype=np.float32).reshape(-1, 4)
                cols = (_image(os.path.join(dataset_dir, "JPEGImages", i + ".jpg"), decode), box,
                        np.array([[index[o[0]]] for o in objs], dtype=np.uint32),
                        np.array([[o[2]] for o in objs], dtype=np.uint32),
                        np.array([[o[3]] for o in objs], dtype=np.uint32))
                return cols + ((np.array(i),) if extra_metadata else ())
            names = ["image", "bbox", "label", "difficult", "truncate"]
        else:
            self._index = index

            def load(i):
                cols = (_image(os.path.join(dataset_dir, "JPEGImages", i + ".jpg"), decode),
                        _image(os.path.join(dataset_dir, "SegmentationClass", i + ".png"), decode))
                return cols + ((np.array(i),) if extra_metadata else ())
            names = ["image", "target"]
        _init(self, _Rows(ids, load), names + (["_meta-filename"] if extra_metadata else []), _kw(**kw))

    def get_class_indexing(self):
        return dict(self._index)


@_export
class CityscapesDataset(GeneratorDataset):
    """``leftImg8bit/<usage>/<city>/*_leftImg8bit.png`` with ``gtFine`` (``quality_mode='fine'``) or ``gtCoarse``
    ``*_<gtFine|gtCoarse>_<instanceIds|labelIds|color>.png`` chosen by ``task`` ('instance', 'semantic', 'color'):
    columns ``image`` and ``task``."""

    def __init__(self, dataset_dir, usage="train", quality_mode="fine", task="instance", decode=False, **kw):
        if task not in ("instance", "semantic", "color", "polygon"):
            raise ValueError("For 'CityscapesDataset', 'task' %r is not supported" % (task,))
        gt = "gtFine" if quality_mode == "fine" else "gtCoarse"
        suffix = "_%s_%s" % (gt, {"instance": "instanceIds.png", "semantic": "labelIds.png", "color": "color.png",
                                  "polygon": "polygons.json"}[task])
        a_dir, b_dir = os.path.join(dataset_dir, "leftImg8bit", usage), os.path.join(dataset_dir, gt, usage)
        records = []
        for root, _, files in sorted(os.walk(a_dir)):
            for f in sorted(files):
                if f.endswith("_leftImg8bit.png"):
                    rel = os.path.relpath(os.path.join(root, f), a_dir)
                    other = os.path.join(b_dir, rel[:-len("_leftImg8bit.png")] + suffix)
                    if os.path.exists(other):
                        records.append((os.path.join(root, f), other))
        _init(self, _Rows(records, lambda r: (_image(r[0], decode), _image(r[1], decode and task != "polygon"))),
              ["image", "task"], _kw(**kw))


@_export
class DIV2KDataset(GeneratorDataset):
    """``DIV2K_<usage>_HR/<id>.png`` with ``DIV2K_<usage>_LR_<downgrade>/X<scale>/<id>x<scale>.png``: ``hr_image``,
    ``lr_image``."""
    _columns = ["hr_image", "lr_image"]

    def __init__(self, dataset_dir, usage="train", downgrade="bicubic", scale=2, decode=False, **kw):
        hr = os.path.join(dataset_dir, "DIV2K_%s_HR" % usage)
        lr = os.path.join(dataset_dir, "DIV2K_%s_LR_%s" % (usage, downgrade), "X%d" % scale)
        records = [(os.path.join(hr, f), os.path.join(lr, f[:-4] + "x%d.png" % scale)) for f in sorted(os.listdir(hr))
                   if f.endswith(".png") and os.path.exists(os.path.join(lr, f[:-4] + "x%d.png" % scale))]
        _init(self, _Rows(records, lambda r: (_image(r[0], decode), _image(r[1], decode))), self._columns, _kw(**kw))


@_export
class FlickrDataset(GeneratorDataset):
    """``annotation_file`` lines ``<image>#<k>\\t<caption>``: ``image`` and ``annotation`` (the captions of it)."""

    def __init__(self, dataset_dir, annotation_file, decode=False, **kw):
        caps = {}
        with open(annotation_file, encoding="utf-8") as f:
            for ln in f:
                if "\t" not in ln:
                    continue
                key, cap = ln.rstrip("\n").split("\t", 1)
                caps.setdefault(key.split("#")[0], []).append(cap)
        records = sorted(caps.items())
        _init(self, _Rows(records, lambda r: (_image(os.path.join(dataset_dir, r[0]), decode),
                                              np.array(r[1], dtype=object))), ["image", "annotation"], _kw(**kw))


@_export
class SBUDataset(GeneratorDataset):
    """``SBU_captioned_photo_dataset_urls.txt`` / ``..._captions.txt`` line-aligned, images in ``sbu_images/``."""

    def __init__(self, dataset_dir, decode=False, **kw):
        with open(os.path.join(dataset_dir, "SBU_captioned_photo_dataset_urls.txt")) as f:
            urls = [ln.strip() for ln in f if ln.strip()]
        with open(os.path.join(dataset_dir, "SBU_captioned_photo_dataset_captions.txt"), encoding="utf-8") as f:
            caps = [ln.rstrip("\n") for ln in f]
        records = [(os.path.join(dataset_dir, "sbu_images", os.path.basename(u)), c) for u, c in zip(urls, caps)
                   if os.path.exists(os.path.join(dataset_dir, "sbu_images", os.path.basename(u)))]
        _init(self, _Rows(records, lambda r: (_image(r[0], decode), np.array(r[1]))), ["image", "caption"], _kw(**kw))


@_export
class LFWDataset(GeneratorDataset):
    """``lfw*/<person>/<person>_<nnnn>.jpg``; ``task='people'``: ``image``, ``label`` (person index)."""

    def __init__(self, dataset_dir, task="people", usage="all", image_set="funneled", decode=False, **kw):
        root = next((os.path.join(dataset_dir, d) for d in ("lfw_funneled", "lfw-deepfunneled", "lfw")
                     if os.path.isdir(os.path.join(dataset_dir, d))), dataset_dir)
        people = sorted(d for d in os.listdir(root) if os.path.isdir(os.path.join(root, d)))
        records = [(os.path.join(root, p, f), i) for i, p in enumerate(people)
                   for f in sorted(os.listdir(os.path.join(root, p)))]
        labels = np.array([l for _, l in records], dtype=np.int32)
        _init(self, _Rows(records, lambda r: (_image(r[0], decode), np.uint32(r[1])), labels), ["image", "label"],
              _kw(**kw))


@_export
class KITTIDataset(GeneratorDataset):
    """``data_object_image_2/<usage>ing/image_2/<id>.png`` and, for 'train', ``data_object_label_2/training/label_2/
    <id>.txt``: ``image``, ``label`` (class names), ``truncated``, ``occluded``, ``alpha``, ``bbox``,
    ``dimensions``, ``location``, ``rotation_y``."""

    def __init__(self, dataset_dir, usage="train", decode=False, **kw):
        usage = _check_usage("KITTIDataset", usage, ("train", "test"), "train")
        img_dir = os.path.join(dataset_dir, "data_object_image_2", usage + "ing", "image_2")
        lab_dir = os.path.join(dataset_dir, "data_object_label_2", "training", "label_2")
        ids = sorted(f[:-4] for f in os.listdir(img_dir) if f.endswith(".png"))

        def load(i):
            img = _image(os.path.join(img_dir, i + ".png"), decode)
            if usage == "test":
                return (img,)
            with open(os.path.join(lab_dir, i + ".txt")) as f:
                rows = [ln.split() for ln in f if ln.strip()]
            num = lambda a, b: np.array([[float(v) for v in r[a:b]] for r in rows], dtype=np.float32)
            return (img, np.array([r[0] for r in rows], dtype=object), num(1, 2), num(2, 3).astype(np.uint32),
                    num(3, 4), num(4, 8), num(8, 11), num(11, 14), num(14, 15))
        cols = ["image"] if usage == "test" else ["image", "label", "truncated", "occluded", "alpha", "bbox",
                                                  "dimensions", "location", "rotation_y"]
        _init(self, _Rows(ids, load), cols, _kw(**kw))


@_export
class WIDERFaceDataset(GeneratorDataset):
    """``wider_face_split/wider_face_<usage>_bbx_gt.txt`` (file, count, then ``x y w h blur expression illumination
    invalid occlusion pose`` rows) with images under ``WIDER_<usage>/images``."""

    def __init__(self, dataset_dir, usage="train", decode=False, **kw):
        usage = _check_usage("WIDERFaceDataset", usage, ("train", "valid", "test", "all"), "train")
        parts = ["train", "val"] if usage == "all" else [{"valid": "val"}.get(usage, usage)]
        records = []
        for part in parts:
            gt = os.path.join(dataset_dir, "wider_face_split", "wider_face_%s_bbx_gt.txt" % part)
            if not os.path.exists(gt):
                continue
            with open(gt) as f:
                lines = [ln.strip() for ln in f]
            k = 0
            while k < len(lines):
                name, n = lines[k], int(lines[k + 1])
                rows = [[int(v) for v in lines[k + 2 + j].split()] for j in range(max(n, 1))]
                records.append((os.path.join(dataset_dir, "WIDER_" + part, "images", name),
                                np.array(rows if n else np.zeros((0, 10)), dtype=np.uint32).reshape(-1, 10)))
                k += 2 + max(n, 1)

        def load(r):
            a = r[1]
            return (_image(r[0], decode), a[:, :4], a[:, 4:5], a[:, 5:6], a[:, 6:7], a[:, 7:8], a[:, 8:9], a[:, 9:10])
        _init(self, _Rows(records, load), ["image", "bbox", "blur", "expression", "illumination", "occlusion", "pose",
                                           "invalid"], _kw(**kw))


@_export
class PhotoTourDataset(GeneratorDataset):
    """``<name>/`` holds 1024 x 1024 bitmaps of 16 x 16 patches of 64 x 64 pixels and ``info.txt`` (point id per
    patch).  'train': column ``image`` uint8 [64, 64, 1]; 'test': ``image1``, ``image2``, ``matches`` from
    ``m50_100000_100000_0.txt``."""

    def __init__(self, dataset_dir, name, usage="train", **kw):
        from PIL import Image
        usage = _check_usage("PhotoTourDataset", usage, ("train", "test"), "train")
        root = os.path.join(dataset_dir, name)
        with open(os.path.join(root, "info.txt")) as f:
            count = sum(1 for ln in f if ln.strip())
        patches = []
        for fname in sorted(x for x in os.listdir(root) if x.endswith(".bmp")):
            with Image.open(os.path.join(root, fname)) as im:
                sheet = np.asarray(im.convert("L"))
            for r in range(16):
                for c in range(16):
                    if len(patches) < count:
                        patches.append(sheet[r * 64:(r + 1) * 64, c * 64:(c + 1) * 64, None])
        if usage == "train":
            _init(self, _Rows(patches, lambda p: (p,)), ["image"], _kw(**kw))
            return
        with open(os.path.join(root, "m50_100000_100000_0.txt")) as f:
            rows = [[int(v) for v in ln.split()] for ln in f if ln.strip()]
        _init(self, _Rows(rows, lambda r: (patches[r[0]], patches[r[3]], np.uint32(r[1] == r[4]))),
              ["image1", "image2", "matches"], _kw(**kw))


@_export
class SBDataset(GeneratorDataset):
    """Semantic Boundaries: ``img/<id>.jpg`` with ``cls/<id>.mat`` (``GTcls.Segmentation`` / ``.Boundaries``); ids
    from ``<usage>.txt``.  ``task='Segmentation'`` gives the label map, ``'Boundaries'`` the 20 boundary maps."""

    def __init__(self, dataset_dir, task="Boundaries", usage="all", decode=False, **kw):
        import scipy.io
        usage = _check_usage("SBDataset", usage, ("train", "val", "train_noval", "all"))
        names = ["train", "val"] if usage == "all" else [usage]
        ids = []
        for n in names:
            with open(os.path.join(dataset_dir, n + ".txt")) as f:
                ids += [ln.strip() for ln in f if ln.strip()]

        def load(i):
            gt = scipy.io.loadmat(os.path.join(dataset_dir, "cls", i + ".mat"))["GTcls"][0, 0]
            if task == "Segmentation":
                target = np.asarray(gt["Segmentation"], dtype=np.uint8)
            else:
                target = np.stack([np.asarray(b[0].todense() if hasattr(b[0], "todense") else b[0], dtype=np.uint8)
                                   for b in gt["Boundaries"]])
            return _image(os.path.join(dataset_dir, "img", i + ".jpg"), decode), target
        _init(self, _Rows(ids, load), ["image", "task"], _kw(**kw))


# ---------------------------------------------------------------------------------------------------- text
def _csv_text_dataset(name, columns, doc):
    def __init__(self, dataset_dir, usage=None, **kw):
        usage = _check_usage(name, usage, ("train", "test", "all"))
        rows = []
        for part in ("train", "test"):
            if usage in (part, "all"):
                with open(os.path.join(dataset_dir, part + ".csv"), newline="", encoding="utf-8") as f:
                    rows += [r for r in csv.reader(f) if r]
        cols = [np.array([r[j] if j < len(r) else "" for r in rows], dtype=object) for j in range(len(columns))]
        _init(self, _Indexed(cols), list(columns), _kw(**kw))
    return _export(type(name, (GeneratorDataset,), {"__init__": __init__, "__doc__": doc}))


AGNewsDataset = _csv_text_dataset("AGNewsDataset", ("index", "title", "description"),
                                  "``{train,test}.csv``: class index, title, description.")
DBpediaDataset = _csv_text_dataset("DBpediaDataset", ("class", "title", "content"), "``{train,test}.csv``.")
AmazonReviewDataset = _csv_text_dataset("AmazonReviewDataset", ("label", "title", "content"), "``{train,test}.csv``.")
YelpReviewDataset = _csv_text_dataset("YelpReviewDataset", ("label", "text"), "``{train,test}.csv``.")
YahooAnswersDataset = _csv_text_dataset("YahooAnswersDataset", ("class", "title", "content", "answer"),
                                        "``{train,test}.csv``.")
SogouNewsDataset = _csv_text_dataset("SogouNewsDataset", ("index", "title", "content"), "``{train,test}.csv``.")


@_export
class IMDBDataset(GeneratorDataset):
    """``<usage>/{pos,neg}/*.txt``: columns ``text`` and ``label`` (1 = pos)."""

    def __init__(self, dataset_dir, usage=None, **kw):
        usage = _check_usage("IMDBDataset", usage, ("train", "test", "all"))
        records = []
        for part in ("train", "test"):
            if usage in (part, "all"):
                for lab, sub in ((1, "pos"), (0, "neg")):
                    d = os.path.join(dataset_dir, part, sub)
                    records += [(os.path.join(d, f), lab) for f in sorted(os.listdir(d)) if f.endswith(".txt")]

        def load(r):
            with open(r[0], encoding="utf-8") as f:
                return np.array(f.read()), np.uint32(r[1])
        _init(self, _Rows(records, load, np.array([l for _, l in records], dtype=np.int32)), ["text", "label"],
              _kw(**kw))


@_export
class SST2Dataset(GeneratorDataset):
    """``{train,dev,test}.tsv`` with a header; train / dev: ``sentence``, ``label``; test: ``sentence``."""

    def __init__(self, dataset_dir, usage=None, **kw):
        usage = _check_usage("SST2Dataset", usage, ("train", "test", "dev"), "train")
        with open(os.path.join(dataset_dir, usage + ".tsv"), encoding="utf-8") as f:
            rows = [ln.rstrip("\n").split("\t") for ln in f][1:]
        if usage == "test":
            _init(self, _Indexed([np.array([r[-1] for r in rows], dtype=object)]), ["sentence"], _kw(**kw))
        else:
            _init(self, _Indexed([np.array([r[0] for r in rows], dtype=object),
                                  np.array([r[1] for r in rows], dtype=object)]), ["sentence", "label"], _kw(**kw))


def _conll_dataset(name, columns, files, doc):
    def __init__(self, dataset_dir, usage=None, **kw):
        usage = _check_usage(name, usage, tuple(files) + ("all",))
        sents = []
        for part in ([k for k in files] if usage == "all" else [usage]):
            with open(os.path.join(dataset_dir, files[part]), encoding="utf-8") as f:
                cur = []
                for ln in f:
                    if not ln.strip():
                        if cur:
                            sents.append(cur)
                        cur = []
                    else:
                        cur.append(ln.split())
                if cur:
                    sents.append(cur)
        cols = [np.empty(len(sents), dtype=object) for _ in columns]
        for i, s in enumerate(sents):
            for j in range(len(columns)):
                cols[j][i] = np.array([t[j] if j < len(t) else "" for t in s], dtype=object)
        _init(self, _Indexed(cols), list(columns), _kw(**kw))
    return _export(type(name, (GeneratorDataset,), {"__init__": __init__, "__doc__": doc}))


CoNLL2000Dataset = _conll_dataset("CoNLL2000Dataset", ("word", "pos_tag", "chunk_tag"),
                                  {"train": "train.txt", "test": "test.txt"},
                                  "``train.txt`` / ``test.txt``: one token per line (word, POS, chunk); blank line "
                                  "between sentences.")
UDPOSDataset = _conll_dataset("UDPOSDataset", ("word", "universal", "stanford"),
                              {"train": "en-ud-tag.v2.train.txt", "test": "en-ud-tag.v2.test.txt",
                               "valid": "en-ud-tag.v2.dev.txt"}, "Universal Dependencies POS files.")


def _lines_dataset(name, files, doc):
    def __init__(self, dataset_dir, usage=None, **kw):
        usage = _check_usage(name, usage, tuple(files) + ("all",))
        lines = []
        for part in ([k for k in files] if usage == "all" else [usage]):
            with open(os.path.join(dataset_dir, files[part]), encoding="utf-8") as f:
                lines += [ln.rstrip("\n") for ln in f if ln.strip()]
        _init(self, _Indexed([np.array(lines, dtype=object)]), ["text"], _kw(**kw))
    return _export(type(name, (GeneratorDataset,), {"__init__": __init__, "__doc__": doc}))


PennTreebankDataset = _lines_dataset("PennTreebankDataset", {"train": "ptb.train.txt", "test": "ptb.test.txt",
                                                             "valid": "ptb.valid.txt"}, "``ptb.<usage>.txt`` lines.")
WikiTextDataset = _lines_dataset("WikiTextDataset", {"train": "wiki.train.tokens", "test": "wiki.test.tokens",
                                                     "valid": "wiki.valid.tokens"}, "``wiki.<usage>.tokens`` lines.")


@_export
class EnWik9Dataset(GeneratorDataset):
    """The lines of ``enwik9``."""

    def __init__(self, dataset_dir, **kw):
        with open(os.path.join(dataset_dir, "enwik9"), encoding="utf-8", errors="replace") as f:
            lines = [ln.rstrip("\n") for ln in f]
        _init(self, _Indexed([np.array(lines, dtype=object)]), ["text"], _kw(**kw))


@_export
class SQuADDataset(GeneratorDataset):
    """``train-v*.json`` / ``dev-v*.json``: ``context``, ``question``, ``text`` (answers), ``answer_start``."""

    def __init__(self, dataset_dir, usage=None, **kw):
        usage = _check_usage("SQuADDataset", usage, ("train", "dev", "all"))
        rows = []
        for part in ("train", "dev"):
            if usage not in (part, "all"):
                continue
            path = next(os.path.join(dataset_dir, f) for f in sorted(os.listdir(dataset_dir))
                        if f.startswith(part + "-v") and f.endswith(".json"))
            with open(path, encoding="utf-8") as f:
                for art in json.load(f)["data"]:
                    for para in art["paragraphs"]:
                        for qa in para["qas"]:
                            ans = qa.get("answers") or [{"text": "", "answer_start": -1}]
                            rows.append((para["context"], qa["question"],
                                         np.array([a["text"] for a in ans], dtype=object),
                                         np.array([a["answer_start"] for a in ans], dtype=np.uint32)))
        _init(self, _Rows(rows, lambda r: (np.array(r[0]), np.array(r[1]), r[2], r[3])),
              ["context", "question", "text", "answer_start"], _kw(**kw))


_CLUE_COLUMNS = {
    ("AFQMC", "train"): ["label", "sentence1", "sentence2"], ("AFQMC", "test"): ["id", "sentence1", "sentence2"],
    ("TNEWS", "train"): ["label", "label_desc", "sentence", "keywords"],
    ("TNEWS", "test"): ["id", "sentence", "keywords"],
    ("IFLYTEK", "train"): ["label", "label_des", "sentence"], ("IFLYTEK", "test"): ["id", "sentence"],
    ("CMNLI", "train"): ["label", "sentence1", "sentence2"], ("CMNLI", "test"): ["id", "sentence1", "sentence2"],
    ("WSC", "train"): ["span1_index", "span2_index", "span1_text", "span2_text", "idx", "label", "text"],
    ("WSC", "test"): ["span1_index", "span2_index", "span1_text", "span2_text", "idx", "text"],
    ("CSL", "train"): ["id", "abst", "keyword", "label"], ("CSL", "test"): ["id", "abst", "keyword"],
}


@_export
class CLUEDataset(GeneratorDataset):
    """JSON-lines files of the CLUE tasks (AFQMC, TNEWS, IFLYTEK, CMNLI, WSC, CSL); ``usage`` 'eval' reads like
    'train'.  Nested ``target`` fields of WSC are flattened to the span columns."""

    def __init__(self, dataset_files, task="AFQMC", usage="train", **kw):
        from .sources import _expand
        if task not in ("AFQMC", "TNEWS", "IFLYTEK", "CMNLI", "WSC", "CSL"):
            raise ValueError("For 'CLUEDataset', 'task' %r is not supported" % (task,))
        cols = _CLUE_COLUMNS[(task, "test" if usage == "test" else "train")]
        rows = []
        for fpath in _expand(dataset_files):
            with open(fpath, encoding="utf-8") as f:
                for ln in f:
                    if not ln.strip():
                        continue
                    rec = json.loads(ln)
                    if isinstance(rec.get("target"), dict):
                        rec.update(rec.pop("target"))
                    if isinstance(rec.get("keyword"), list):
                        rec["keyword"] = np.array(rec["keyword"], dtype=object)
                    rows.append(tuple(rec.get(c, "") for c in cols))
        _init(self, _Rows(rows, lambda r: tuple(v if isinstance(v, np.ndarray) else np.array(v) for v in r)), cols,
              _kw(**kw))


def _parallel_text(name, doc, locate):
    def __init__(self, dataset_dir, usage=None, language_pair=("de", "en"), **kw):
        src, tgt = locate(dataset_dir, usage or "train", tuple(language_pair), kw)
        clean = lambda ln: None if ln.lstrip().startswith("<") else ln.rstrip("\n")
        with open(src, encoding="utf-8") as f:
            a = [c for c in (clean(ln) for ln in f) if c is not None]
        with open(tgt, encoding="utf-8") as f:
            b = [c for c in (clean(ln) for ln in f) if c is not None]
        n = min(len(a), len(b))
        _init(self, _Indexed([np.array(a[:n], dtype=object), np.array(b[:n], dtype=object)]),
              ["text", "translation"], _kw(**{k: v for k, v in kw.items() if k in (
                  "num_samples", "shuffle", "sampler", "num_shards", "shard_id")}))
    return _export(type(name, (GeneratorDataset,), {"__init__": __init__, "__doc__": doc}))


def _multi30k_files(d, usage, pair, kw):
    stem = {"train": "train", "valid": "val", "test": "test_2016_flickr"}.get(usage, usage)
    out = []
    for lang in pair:
        name = "%s.%s" % (stem, lang)
        cands = [os.path.join(d, name), os.path.join(d, usage, name), os.path.join(d, "training", name),
                 os.path.join(d, "validation", name), os.path.join(d, "mmt16_task1_test", name)]
        found = next((c for c in cands if os.path.exists(c)), None)
        if found is None:
            raise FileNotFoundError("Multi30kDataset: %s not found under %s" % (name, d))
        out.append(found)
    return tuple(out)


Multi30kDataset = _parallel_text("Multi30kDataset", "Line-aligned ``<train|val|test_2016_flickr>.<lang>`` files.",
                                 _multi30k_files)
IWSLT2016Dataset = _parallel_text("IWSLT2016Dataset", "``<pair dir>/train.tags.<src>-<tgt>.<lang>`` (tag lines "
                                  "skipped).", lambda d, usage, pair, kw: tuple(
    os.path.join(d, "%s-%s" % pair, "train.tags.%s-%s.%s" % (pair[0], pair[1], lang)) for lang in pair))
IWSLT2017Dataset = _parallel_text("IWSLT2017Dataset", "``train.tags.<src>-<tgt>.<lang>`` (tag lines skipped).",
                                  lambda d, usage, pair, kw: tuple(
                                      os.path.join(d, "train.tags.%s-%s.%s" % (pair[0], pair[1], lang))
                                      for lang in pair))


# ---------------------------------------------------------------------------------------------------- audio
@_export
class YesNoDataset(GeneratorDataset):
    """``<8 digits joined by _>.wav``: ``waveform``, ``sample_rate``, ``labels`` (the eight 0 / 1)."""

    def __init__(self, dataset_dir, **kw):
        files = sorted(f for f in os.listdir(dataset_dir) if f.endswith(".wav"))

        def load(f):
            w, sr = _wav(os.path.join(dataset_dir, f))
            return w, np.int32(sr), np.array([int(c) for c in f[:-4].split("_")], dtype=np.int32)
        _init(self, _Rows(files, load), ["waveform", "sample_rate", "labels"], _kw(**kw))


@_export
class SpeechCommandsDataset(GeneratorDataset):
    """``<word>/<speaker>_nohash_<k>.wav`` with ``validation_list.txt`` / ``testing_list.txt``: ``waveform``,
    ``sample_rate``, ``label``, ``speaker_id``, ``utterance_number``."""

    def __init__(self, dataset_dir, usage=None, **kw):
        usage = _check_usage("SpeechCommandsDataset", usage, ("train", "valid", "test", "all"))

        def listed(name):
            p = os.path.join(dataset_dir, name)
            if not os.path.exists(p):
                return set()
            with open(p) as f:
                return {ln.strip() for ln in f if ln.strip()}
        val, test = listed("validation_list.txt"), listed("testing_list.txt")
        files = []
        for word in sorted(d for d in os.listdir(dataset_dir) if os.path.isdir(os.path.join(dataset_dir, d))
                           and not d.startswith("_")):
            for f in sorted(os.listdir(os.path.join(dataset_dir, word))):
                rel = word + "/" + f
                part = "valid" if rel in val else "test" if rel in test else "train"
                if f.endswith(".wav") and usage in (part, "all"):
                    files.append(rel)

        def load(rel):
            w, sr = _wav(os.path.join(dataset_dir, rel))
            word, name = rel.split("/")
            m = re.match(r"(.+)_nohash_(\d+)\.wav", name)
            return w, np.int32(sr), np.array(word), np.array(m.group(1)), np.int32(m.group(2))
        _init(self, _Rows(files, load), ["waveform", "sample_rate", "label", "speaker_id", "utterance_number"],
              _kw(**kw))


@_export
class LJSpeechDataset(GeneratorDataset):
    """``metadata.csv`` (``id|transcription|normalized``) and ``wavs/<id>.wav``."""

    def __init__(self, dataset_dir, **kw):
        with open(os.path.join(dataset_dir, "metadata.csv"), encoding="utf-8") as f:
            rows = [ln.rstrip("\n").split("|") for ln in f if ln.strip()]

        def load(r):
            w, sr = _wav(os.path.join(dataset_dir, "wavs", r[0] + ".wav"))
            return w, np.int32(sr), np.array(r[1]), np.array(r[2] if len(r) > 2 else r[1])
        _init(self, _Rows(rows, load), ["waveform", "sample_rate", "transcription", "normalized_transcript"],
              _kw(**kw))


@_export
class GTZANDataset(GeneratorDataset):
    """``genres/<genre>/<genre>.<nnnnn>.wav``: ``waveform``, ``sample_rate``, ``label`` (the genre)."""

    def __init__(self, dataset_dir, usage=None, **kw):
        root = os.path.join(dataset_dir, "genres") if os.path.isdir(os.path.join(dataset_dir, "genres")) \
            else dataset_dir
        files = [(os.path.join(root, g, f), g) for g in sorted(os.listdir(root))
                 if os.path.isdir(os.path.join(root, g)) for f in sorted(os.listdir(os.path.join(root, g)))
                 if f.endswith(".wav")]

        def load(r):
            w, sr = _wav(r[0])
            return w, np.int32(sr), np.array(r[1])
        _init(self, _Rows(files, load), ["waveform", "sample_rate", "label"], _kw(**kw))


@_export
class CMUArcticDataset(GeneratorDataset):
    """``cmu_us_<name>_arctic/{etc/txt.done.data, wav/<id>.wav}``: ``waveform``, ``sample_rate``, ``transcript``,
    ``utterance_id``."""

    def __init__(self, dataset_dir, name="aew", **kw):
        root = os.path.join(dataset_dir, "cmu_us_%s_arctic" % name)
        with open(os.path.join(root, "etc", "txt.done.data"), encoding="utf-8") as f:
            rows = [re.match(r'\(\s*(\S+)\s+"(.*)"\s*\)', ln.strip()).groups() for ln in f if ln.strip()]

        def load(r):
            w, sr = _wav(os.path.join(root, "wav", r[0] + ".wav"))
            return w, np.int32(sr), np.array(r[1]), np.array(r[0].split("_")[-1])
        _init(self, _Rows(rows, load), ["waveform", "sample_rate", "transcript", "utterance_id"], _kw(**kw))


@_export
class LibriTTSDataset(GeneratorDataset):
    """``<usage>/<speaker>/<chapter>/<utt>.wav`` with ``.original.txt`` / ``.normalized.txt`` beside it."""

    def __init__(self, dataset_dir, usage=None, **kw):
        parts = [usage] if usage and usage != "all" else sorted(
            d for d in os.listdir(dataset_dir) if os.path.isdir(os.path.join(dataset_dir, d)))
        files = []
        for part in parts:
            for root, _, names in sorted(os.walk(os.path.join(dataset_dir, part))):
                files += [os.path.join(root, n) for n in sorted(names) if n.endswith(".wav")]

        def text(path):
            if not os.path.exists(path):
                return ""
            with open(path, encoding="utf-8") as f:
                return f.read().strip()

        def load(p):
            w, sr = _wav(p)
            utt = os.path.basename(p)[:-4]
            spk, chap = utt.split("_")[0], utt.split("_")[1]
            return (w, np.int32(sr), np.array(text(p[:-4] + ".original.txt")),
                    np.array(text(p[:-4] + ".normalized.txt")), np.int32(spk), np.int32(chap), np.array(utt))
        _init(self, _Rows(files, load), ["waveform", "sample_rate", "original_text", "normalized_text", "speaker_id",
                                         "chapter_id", "utterance_id"], _kw(**kw))


@_export
class TedliumDataset(GeneratorDataset):
    """TED-LIUM: ``<release dir>/<usage>/{stm/<talk>.stm, sph/<talk>.sph}``.  The NIST sphere files must hold
    uncompressed 16-bit PCM (1024-byte text header); each row is one segment of an ``.stm`` line."""

    def __init__(self, dataset_dir, release="release1", usage=None, extensions=".sph", **kw):
        usage = _check_usage("TedliumDataset", usage, ("train", "dev", "test", "all"), "train")
        rows = []
        for part in (["train", "dev", "test"] if usage == "all" else [usage]):
            stm_dir = os.path.join(dataset_dir, part, "stm")
            if not os.path.isdir(stm_dir):
                continue
            for f in sorted(os.listdir(stm_dir)):
                with open(os.path.join(stm_dir, f), encoding="utf-8") as fh:
                    for ln in fh:
                        t = ln.split(" ", 6)
                        if len(t) == 7:
                            rows.append((os.path.join(dataset_dir, part, "sph", t[0] + extensions), t[0], t[2],
                                         float(t[3]), float(t[4]), t[5], t[6].strip()))

        def load(r):
            with open(r[0], "rb") as fh:
                head = fh.read(1024).decode("ascii", "replace")
                rate = int(re.search(r"sample_rate -i (\d+)", head).group(1))
                fh.seek(1024 + int(r[3] * rate) * 2)
                data = np.frombuffer(fh.read(int((r[4] - r[3]) * rate) * 2), dtype=">i2" if "10" in (
                    re.search(r"sample_byte_format -s2 (\d+)", head) or [None, "01"])[1] else "<i2")
            return (data.astype(np.float32)[None] / 32768.0, np.int32(rate), np.array(r[6]), np.array(r[1]),
                    np.array(r[2]), np.array(r[5]))
        _init(self, _Rows(rows, load), ["waveform", "sample_rate", "transcript", "talk_id", "speaker_id",
                                        "identifier"], _kw(**kw))


# ---------------------------------------------------------------------------------------------------- standard formats
@_export
class Schema:
    """Column names, types and shapes of a dataset; ``add_column`` / ``parse_columns`` / ``from_json`` / ``to_json``."""

    def __init__(self, schema_file=None):
        self.columns, self.dataset_type, self.num_rows = [], "", 0
        if schema_file is not None:
            with open(schema_file) as f:
                self.from_json(json.load(f))

    def add_column(self, name, de_type, shape=None):
        if not isinstance(name, str) or not name:
            raise ValueError("Column name must be a non-empty string")
        col = {"name": name, "type": str(de_type).replace("mindspore.", "").replace("torch.", "")}
        if shape is not None:
            col["shape"] = list(shape)
            col["rank"] = len(shape)
        self.columns.append(col)

    def parse_columns(self, columns):
        self.columns = []
        if isinstance(columns, dict):
            columns = [dict(v, name=k) for k, v in columns.items()]
        for c in columns:
            if "name" not in c or "type" not in c:
                raise RuntimeError("Column's name and type are required: %r" % (c,))
            self.add_column(c["name"], c["type"], c.get("shape"))

    def from_json(self, json_obj):
        if not isinstance(json_obj, dict):
            raise TypeError("Expected a json object (dict), but got %s" % type(json_obj).__name__)
        self.parse_columns(json_obj.get("columns", []))
        self.dataset_type = json_obj.get("datasetType", "")
        self.num_rows = json_obj.get("numRows", 0)

    def to_json(self):
        out = {"columns": self.columns}
        if self.dataset_type:
            out["datasetType"] = self.dataset_type
        if self.num_rows:
            out["numRows"] = self.num_rows
        return json.dumps(out, indent=2)

    def __str__(self):
        return self.to_json()


@_export
class TFRecordDataset(GeneratorDataset):
    """``tf.train.Example`` records (decoded here; TensorFlow is not needed).  Columns: ``columns_list``, or the
    schema's, or every feature of the first record; integer lists -> int64, float lists -> float32, bytes -> one
    uint8 array (or an array of strings when there are several)."""

    def __init__(self, dataset_files, schema=None, columns_list=None, num_samples=None, num_parallel_workers=None,
                 shuffle=False, num_shards=None, shard_id=None, shard_equal_rows=False, cache=None,
                 compression_type=None):
        from .mindrecord import TFRecordToMR
        from .sources import _expand
        if compression_type not in (None, ""):
            raise ValueError("TFRecordDataset: compressed files are not supported here (got %r)" % compression_type)
        rows = []
        for f in _expand(dataset_files):
            rows += list(TFRecordToMR(f, "", {})._examples())
        if isinstance(schema, str):
            schema = Schema(schema)
        cols = list(columns_list) if columns_list else [c["name"] for c in schema.columns] if schema \
            else sorted(rows[0]) if rows else []

        def conv(v):
            if v and isinstance(v[0], bytes):
                return np.frombuffer(v[0], dtype=np.uint8) if len(v) == 1 else np.array(
                    [b.decode(errors="replace") for b in v], dtype=object)
            if v and isinstance(v[0], (float, np.floating)):
                return np.asarray(v, dtype=np.float32)
            return np.asarray(v, dtype=np.int64)
        super().__init__(_Rows(rows, lambda r: tuple(conv(r[c]) for c in cols)), cols, num_samples=num_samples,
                         shuffle=bool(shuffle), num_shards=num_shards, shard_id=shard_id)


@_export
class PaddedDataset(GeneratorDataset):
    """Rows given as a list of dicts (one key per column), typically appended to a dataset so that every shard gets
    the same number of rows."""

    def __init__(self, padded_samples):
        if not isinstance(padded_samples, list) or not padded_samples or not all(
                isinstance(s, dict) for s in padded_samples):
            raise TypeError("padded_samples must be a non-empty list of dicts")
        cols = list(padded_samples[0])
        super().__init__(_Rows(padded_samples, lambda s: tuple(np.asarray(s[c]) for c in cols)), cols, shuffle=False)


@_export
class OBSMindDataset(GeneratorDataset):
    """Record files on object storage.  There is no object-storage client here: local paths (or ``file://`` URLs) are
    read like ``MindDataset``; any other scheme raises."""

    def __init__(self, dataset_files, server=None, ak=None, sk=None, sync_obs_path=None, columns_list=None,
                 shuffle=None, num_shards=None, shard_id=None, shard_equal_rows=True):
        from .engine import MindDataset
        files = [dataset_files] if isinstance(dataset_files, str) else list(dataset_files)
        local = []
        for f in files:
            if "://" in f and not f.startswith("file://"):
                raise RuntimeError("OBSMindDataset: no object-storage client in this build; %r is not a local path" % f)
            local.append(f[7:] if f.startswith("file://") else f)
        inner = MindDataset(local, columns_list=columns_list, shuffle=shuffle, num_shards=num_shards,
                            shard_id=shard_id)
        self.__dict__.update(inner.__dict__)


# ---------------------------------------------------------------------------------------------------- callbacks / cache / tools
@_export
class DSCallback:
    """Hooks of a ``map`` stage: ``ds_begin``, ``ds_epoch_begin``, ``ds_epoch_end``, ``ds_step_begin``,
    ``ds_step_end`` (each receives a run context with ``cur_epoch_num`` / ``cur_step_num_in_epoch`` /
    ``cur_step_num``); ``step_size`` = rows per step."""

    def __init__(self, step_size=1):
        if not isinstance(step_size, int) or step_size <= 0:
            raise ValueError("step_size must be a positive int, but got %r" % (step_size,))
        self.step_size = step_size

    def ds_begin(self, ds_run_context):
        pass

    def ds_epoch_begin(self, ds_run_context):
        pass

    def ds_epoch_end(self, ds_run_context):
        pass

    def ds_step_begin(self, ds_run_context):
        pass

    def ds_step_end(self, ds_run_context):
        pass


@_export
class WaitedDSCallback(DSCallback):
    """A ``DSCallback`` that is also a training callback: the data pipeline's step / epoch begin waits until the
    training loop has finished the previous step / epoch, then runs ``sync_step_begin`` / ``sync_epoch_begin``."""

    def __init__(self, step_size=1):
        super().__init__(step_size)
        import threading
        self._step_done, self._epoch_done = threading.Event(), threading.Event()
        self._step_done.set()
        self._epoch_done.set()

    def sync_epoch_begin(self, train_run_context, ds_run_context):
        pass

    def sync_step_begin(self, train_run_context, ds_run_context):
        pass

    # training side
    def step_end(self, run_context):
        self._train_ctx = run_context
        self._step_done.set()

    def epoch_end(self, run_context):
        self._train_ctx = run_context
        self._epoch_done.set()

    on_train_step_end, on_train_epoch_end = step_end, epoch_end

    # data side
    def ds_step_begin(self, ds_run_context):
        if getattr(ds_run_context, "cur_step_num", 1) > 1:
            self._step_done.wait(timeout=60)
            self._step_done.clear()
        self.sync_step_begin(getattr(self, "_train_ctx", None), ds_run_context)

    def ds_epoch_begin(self, ds_run_context):
        if getattr(ds_run_context, "cur_epoch_num", 1) > 1:
            self._epoch_done.wait(timeout=60)
            self._epoch_done.clear()
        self.sync_epoch_begin(getattr(self, "_train_ctx", None), ds_run_context)


@_export
class DatasetCache:
    """An in-process row cache with the reference's constructor (``session_id``, ``size`` in MB, 0 = unlimited):
    ``get`` / ``put`` by row index, least-recently-used rows dropped beyond ``size``."""

    def __init__(self, session_id, size=0, spilling=False, hostname=None, port=None, num_connections=None,
                 prefetch_size=None):
        if not isinstance(session_id, int) or session_id < 0:
            raise ValueError("session_id must be a non-negative int, but got %r" % (session_id,))
        from collections import OrderedDict
        self.session_id, self.size, self.spilling = session_id, size, spilling
        self._rows, self._bytes, self.hits, self.misses = OrderedDict(), 0, 0, 0

    def get(self, key):
        row = self._rows.get(key)
        if row is None:
            self.misses += 1
            return None
        self._rows.move_to_end(key)
        self.hits += 1
        return row

    def put(self, key, row):
        nbytes = sum(np.asarray(v).nbytes for v in row)
        self._rows[key] = row
        self._bytes += nbytes
        limit = self.size * (1 << 20)
        while limit and self._bytes > limit and len(self._rows) > 1:
            _, old = self._rows.popitem(last=False)
            self._bytes -= sum(np.asarray(v).nbytes for v in old)

    def get_stat(self):
        return {"num_rows": len(self._rows), "bytes": self._bytes, "hits": self.hits, "misses": self.misses}


def _describe(ds):
    node = {"op_type": type(ds).__name__.lstrip("_"), "columns": list(ds.get_col_names() or [])}
    for k in ("batch_size", "drop_remainder", "count", "buffer_size", "num_shards", "shard_id"):
        if hasattr(ds, k) and isinstance(getattr(ds, k), (int, bool, type(None))):
            node[k] = getattr(ds, k)
    parents = getattr(ds, "parents", None) or ([ds.parent] if getattr(ds, "parent", None) is not None else [])
    node["children"] = [_describe(p) for p in parents]
    return node


def serialize(dataset, json_filepath=""):
    """The pipeline as a nested dict (op type, columns, scalar settings, children); written to ``json_filepath`` when
    given."""
    tree = _describe(dataset)
    if json_filepath:
        with open(json_filepath, "w") as f:
            json.dump(tree, f, indent=2)
    return tree


def deserialize(input_dict=None, json_filepath=None):
    """Reads back what ``serialize`` wrote.  Sources and user functions are Python objects that a description
    cannot rebuild, so the result is the description itself (for ``show`` / ``compare``), not a runnable pipeline."""
    if json_filepath:
        with open(json_filepath) as f:
            return json.load(f)
    return input_dict


def show(dataset, indentation=2):
    print(json.dumps(serialize(dataset) if not isinstance(dataset, dict) else dataset, indent=indentation))


def compare(pipeline1, pipeline2):
    """True when the two pipelines have the same description."""
    a = pipeline1 if isinstance(pipeline1, dict) else serialize(pipeline1)
    b = pipeline2 if isinstance(pipeline2, dict) else serialize(pipeline2)
    return a == b


def sync_wait_for_dataset(rank_id, rank_size, current_epoch):
    """Blocks until every rank has finished preparing the data of ``current_epoch`` (a barrier when a process group
    is up; nothing to wait for in a single process)."""
    try:
        import torch.distributed as dist
        if dist.is_available() and dist.is_initialized() and rank_size > 1:
            dist.barrier()
    except ImportError:
        pass


__all__ += ["serialize", "deserialize", "show", "compare", "sync_wait_for_dataset"]
