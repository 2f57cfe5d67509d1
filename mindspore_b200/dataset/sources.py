"""Source datasets that read standard on-disk formats: ``MnistDataset`` (idx files), ``Cifar10Dataset`` (binary
batches), ``ImageFolderDataset`` (one directory per class), ``TextFileDataset`` (one row per line), ``CSVDataset``.
Each is a random-access source under ``GeneratorDataset``, so ``shuffle`` / ``sampler`` / ``num_shards`` /
``num_samples`` behave the same for all of them (python/mindspore/dataset/engine/datasets_vision.py,
datasets_text.py, datasets_standard_format.py; the C++ readers are minddata/dataset/engine/datasetops/source/*)."""
from __future__ import annotations

import csv
import gzip
import os
import struct

import numpy as np

from .engine import GeneratorDataset

__all__ = ["MnistDataset", "Cifar10Dataset", "ImageFolderDataset", "TextFileDataset", "CSVDataset"]


def _open(path):
    return gzip.open(path, "rb") if path.endswith(".gz") else open(path, "rb")


def _find(directory, names):
    for n in names:
        for cand in (n, n + ".gz"):
            p = os.path.join(directory, cand)
            if os.path.exists(p):
                return p
    raise FileNotFoundError("none of %s found in %s" % (names, directory))


def _read_idx(path):
    with _open(path) as f:
        data = f.read()
    zero, dtype_code, ndim = struct.unpack_from(">HBB", data, 0)
    if zero != 0 or dtype_code != 0x08:
        raise ValueError("%s is not an idx file of unsigned bytes" % path)
    dims = struct.unpack_from(">" + "I" * ndim, data, 4)
    return np.frombuffer(data, dtype=np.uint8, offset=4 + 4 * ndim).reshape(dims)


class _Indexed:
    def __init__(self, columns, labels=None):
        self._cols, self.labels = columns, labels

    def __len__(self):
        return len(self._cols[0])

    def __getitem__(self, i):
        return tuple(c[i] for c in self._cols)


class MnistDataset(GeneratorDataset):
    """Columns ``image`` (uint8 [28, 28, 1]) and ``label`` (uint32).  ``usage``: 'train', 'test' or 'all'."""

    def __init__(self, dataset_dir, usage=None, num_samples=None, num_parallel_workers=None, shuffle=None, sampler=None,
                 num_shards=None, shard_id=None, cache=None):
        usage = usage or "all"
        if usage not in ("train", "test", "all"):
            raise ValueError("For 'MnistDataset', 'usage' must be train, test or all, got %r" % usage)
        imgs, labs = [], []
        for part, prefix in (("train", "train"), ("test", "t10k")):
            if usage in (part, "all"):
                imgs.append(_read_idx(_find(dataset_dir, [prefix + "-images-idx3-ubyte", prefix + "-images.idx3-ubyte"])))
                labs.append(_read_idx(_find(dataset_dir, [prefix + "-labels-idx1-ubyte", prefix + "-labels.idx1-ubyte"])))
        images = np.concatenate(imgs)[..., None]
        labels = np.concatenate(labs).astype(np.uint32)
        super().__init__(_Indexed([images, labels], labels), ["image", "label"], num_samples=num_samples, shuffle=shuffle,
                         sampler=sampler, num_shards=num_shards, shard_id=shard_id)


class Cifar10Dataset(GeneratorDataset):
    """Columns ``image`` (uint8 [32, 32, 3]) and ``label`` (uint32) from ``data_batch_*.bin`` / ``test_batch.bin``."""

    def __init__(self, dataset_dir, usage=None, num_samples=None, num_parallel_workers=None, shuffle=None, sampler=None,
                 num_shards=None, shard_id=None, cache=None):
        usage = usage or "all"
        if usage not in ("train", "test", "all"):
            raise ValueError("For 'Cifar10Dataset', 'usage' must be train, test or all, got %r" % usage)
        files = sorted(f for f in os.listdir(dataset_dir) if f.endswith(".bin"))
        pick = [f for f in files if (usage in ("train", "all") and f.startswith("data_batch")) or
                (usage in ("test", "all") and f.startswith("test_batch"))]
        if not pick:
            raise FileNotFoundError("no CIFAR-10 .bin files for usage %r in %s" % (usage, dataset_dir))
        rows = np.concatenate([np.fromfile(os.path.join(dataset_dir, f), dtype=np.uint8).reshape(-1, 3073) for f in pick])
        labels = rows[:, 0].astype(np.uint32)
        images = rows[:, 1:].reshape(-1, 3, 32, 32).transpose(0, 2, 3, 1)
        super().__init__(_Indexed([images, labels], labels), ["image", "label"], num_samples=num_samples, shuffle=shuffle,
                         sampler=sampler, num_shards=num_shards, shard_id=shard_id)


class _Folder:
    def __init__(self, root, extensions, class_indexing, decode):
        classes = sorted(d for d in os.listdir(root) if os.path.isdir(os.path.join(root, d)))
        index = class_indexing or {c: i for i, c in enumerate(classes)}
        self.items = []
        for c in classes:
            if c not in index:
                continue
            for f in sorted(os.listdir(os.path.join(root, c))):
                if extensions is None or os.path.splitext(f)[1].lower() in extensions:
                    self.items.append((os.path.join(root, c, f), index[c]))
        self.labels = np.array([l for _, l in self.items], dtype=np.int32)
        self.decode, self.class_indexing = decode, index

    def __len__(self):
        return len(self.items)

    def __getitem__(self, i):
        path, label = self.items[i]
        if self.decode:
            from PIL import Image
            with Image.open(path) as im:
                img = np.asarray(im.convert("RGB"))
        else:
            img = np.fromfile(path, dtype=np.uint8)
        return img, np.int32(label)


class ImageFolderDataset(GeneratorDataset):
    """``dataset_dir/<class>/<file>``: columns ``image`` (encoded bytes, or HWC uint8 with ``decode=True``) and
    ``label`` (int32, classes numbered in sorted order unless ``class_indexing`` maps them)."""

    def __init__(self, dataset_dir, num_samples=None, num_parallel_workers=None, shuffle=None, sampler=None,
                 extensions=None, class_indexing=None, decode=False, num_shards=None, shard_id=None, cache=None,
                 decrypt=None):
        exts = None if not extensions else {e.lower() if e.startswith(".") else "." + e.lower() for e in extensions}
        src = _Folder(dataset_dir, exts, class_indexing, decode)
        self._class_indexing = src.class_indexing
        super().__init__(src, ["image", "label"], num_samples=num_samples, shuffle=shuffle, sampler=sampler,
                         num_shards=num_shards, shard_id=shard_id)

    def get_class_indexing(self):
        return dict(self._class_indexing)


def _expand(files):
    import glob
    files = [files] if isinstance(files, str) else list(files)
    out = []
    for f in files:
        out += sorted(glob.glob(f)) or [f]
    for f in out:
        if not os.path.exists(f):
            raise FileNotFoundError(f)
    return out


class TextFileDataset(GeneratorDataset):
    """One row per line, column ``text`` (numpy str)."""

    def __init__(self, dataset_files, num_samples=None, num_parallel_workers=None, shuffle=False, num_shards=None,
                 shard_id=None, cache=None):
        lines = []
        for f in _expand(dataset_files):
            with open(f, encoding="utf-8") as fh:
                lines += [ln.rstrip("\n").rstrip("\r") for ln in fh if ln.strip("\r\n") != ""]
        super().__init__(_Indexed([np.array(lines, dtype=object)]), ["text"], num_samples=num_samples,
                         shuffle=bool(shuffle), num_shards=num_shards, shard_id=shard_id)


class CSVDataset(GeneratorDataset):
    """Rows of csv files.  Column types come from ``column_defaults`` (a list of example values: int, float or str;
    strings when omitted); names from ``column_names`` or the header line."""

    def __init__(self, dataset_files, field_delim=",", column_defaults=None, column_names=None, num_samples=None,
                 num_parallel_workers=None, shuffle=False, num_shards=None, shard_id=None, cache=None):
        rows, names = [], list(column_names) if column_names else None
        for f in _expand(dataset_files):
            with open(f, newline="", encoding="utf-8") as fh:
                reader = csv.reader(fh, delimiter=field_delim)
                for k, row in enumerate(reader):
                    if not row:
                        continue
                    if k == 0 and column_names is None:
                        if names is None:
                            names = row
                        continue
                    rows.append(row)
        if names is None:
            raise ValueError("CSVDataset: no column names (empty files?)")
        cols = []
        for j, _ in enumerate(names):
            default = column_defaults[j] if column_defaults else ""
            raw = [r[j] if j < len(r) and r[j] != "" else default for r in rows]
            if isinstance(default, bool) or isinstance(default, int):
                cols.append(np.array([int(v) for v in raw], dtype=np.int32))
            elif isinstance(default, float):
                cols.append(np.array([float(v) for v in raw], dtype=np.float32))
            else:
                cols.append(np.array([str(v) for v in raw], dtype=object))
        super().__init__(_Indexed(cols), names, num_samples=num_samples, shuffle=bool(shuffle), num_shards=num_shards,
                         shard_id=shard_id)
