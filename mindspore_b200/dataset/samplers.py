"""Samplers: objects that yield the row indices of an epoch for random-access sources
(python/mindspore/dataset/engine/samplers.py)."""
from __future__ import annotations

import numpy as np

__all__ = ["BuiltinSampler", "IterSampler", "select_sampler", "Sampler", "SequentialSampler", "RandomSampler", "DistributedSampler", "SubsetSampler", "SubsetRandomSampler",
           "WeightedRandomSampler", "PKSampler"]


class Sampler:
    def __init__(self, num_samples=None):
        self.num_samples = num_samples
        self.dataset_size = 0
        self.child = None
        self._epoch = 0

    def bind(self, dataset_size, labels=None):
        self.dataset_size, self._labels = int(dataset_size), labels
        if self.child is not None:
            self.child.bind(dataset_size, labels)
        return self

    def add_child(self, sampler):
        self.child = sampler

    def get_num_samples(self):
        return len(self.indices())

    def _base(self):
        """Indices this sampler draws from: all rows, or what its child produced."""
        return np.arange(self.dataset_size) if self.child is None else np.asarray(self.child.indices())

    def _cut(self, idx):
        return idx if self.num_samples is None else idx[:self.num_samples]

    def indices(self):
        raise NotImplementedError

    def __iter__(self):
        idx = self.indices()
        self._epoch += 1
        return iter(int(i) for i in idx)


class SequentialSampler(Sampler):
    def __init__(self, start_index=None, num_samples=None):
        super().__init__(num_samples)
        self.start_index = start_index or 0

    def indices(self):
        return self._cut(self._base()[self.start_index:])


class RandomSampler(Sampler):
    def __init__(self, replacement=False, num_samples=None, seed=None):
        super().__init__(num_samples)
        self.replacement, self.seed = replacement, seed

    def indices(self):
        from .engine import config
        base = self._base()
        rng = np.random.default_rng((config.get_seed() if self.seed is None else self.seed) + self._epoch)
        n = self.num_samples if self.num_samples is not None else len(base)
        if self.replacement:
            return base[rng.integers(0, len(base), n)]
        return base[rng.permutation(len(base))[:n]]


class DistributedSampler(Sampler):
    def __init__(self, num_shards, shard_id, shuffle=True, num_samples=None, offset=-1):
        super().__init__(num_samples)
        if not 0 <= shard_id < num_shards:
            raise ValueError("shard_id must be in [0, num_shards), got %d of %d" % (shard_id, num_shards))
        self.num_shards, self.shard_id, self.shuffle, self.offset = num_shards, shard_id, shuffle, offset

    def indices(self):
        from .engine import config
        base = self._base()
        if self.shuffle:
            base = base[np.random.default_rng(config.get_seed() + self._epoch).permutation(len(base))]
        per = -(-len(base) // self.num_shards)
        padded = np.resize(base, per * self.num_shards) if len(base) else base        # wrap around to equal shares
        start = max(self.offset, 0)
        padded = np.roll(padded, start)
        return self._cut(padded[self.shard_id::self.num_shards])


class SubsetSampler(Sampler):
    def __init__(self, indices, num_samples=None):
        super().__init__(num_samples)
        self._subset = np.asarray(list(indices), dtype=np.int64)

    def indices(self):
        base = self._base()                       # with a child sampler the subset indexes what the child yields
        if len(self._subset) and (self._subset.min() < 0 or self._subset.max() >= len(base)):
            raise ValueError("SubsetSampler: index out of range for %d rows" % len(base))
        return self._cut(base[self._subset] if self.child is not None else self._subset)


class SubsetRandomSampler(SubsetSampler):
    def indices(self):
        from .engine import config
        idx = super().indices()
        return idx[np.random.default_rng(config.get_seed() + self._epoch).permutation(len(idx))]


class WeightedRandomSampler(Sampler):
    def __init__(self, weights, num_samples=None, replacement=True):
        super().__init__(num_samples)
        w = np.asarray(weights, dtype=np.float64)
        if (w < 0).any() or w.sum() <= 0:
            raise ValueError("weights must be non-negative and not all zero")
        self.weights, self.replacement = w / w.sum(), replacement

    def indices(self):
        from .engine import config
        n = self.num_samples if self.num_samples is not None else len(self.weights)
        rng = np.random.default_rng(config.get_seed() + self._epoch)
        return rng.choice(len(self.weights), size=n, replace=self.replacement, p=self.weights)


class PKSampler(Sampler):
    """``num_val`` rows of each of the classes (needs a source with labels)."""

    def __init__(self, num_val, num_class=None, shuffle=False, class_column="label", num_samples=None):
        super().__init__(num_samples)
        self.num_val, self.num_class, self.shuffle = num_val, num_class, shuffle

    def indices(self):
        from .engine import config
        if self._labels is None:
            raise RuntimeError("PKSampler needs a dataset that exposes its labels")
        labels = np.asarray(self._labels)
        rng = np.random.default_rng(config.get_seed() + self._epoch)
        out = []
        classes = np.unique(labels)[:self.num_class]
        for c in classes:
            rows = np.where(labels == c)[0]
            if self.shuffle:
                rows = rows[rng.permutation(len(rows))]
            out.append(rows[:self.num_val])
        idx = np.stack([r for r in out if len(r) == self.num_val], 1).reshape(-1) if out else np.array([], dtype=np.int64)
        return self._cut(idx)



BuiltinSampler = Sampler


class IterSampler(Sampler):
    """Wraps any iterable of indices as a sampler."""

    def __init__(self, sampler, num_samples=None):
        super().__init__(num_samples)
        self.inner = sampler

    def indices(self):
        return self._cut(np.array([int(i) for i in self.inner], dtype=np.int64))


def select_sampler(num_samples, input_sampler, shuffle, num_shards, shard_id):
    """The sampler a source dataset uses for the given combination of arguments (the reference's rule:
    an explicit sampler excludes shuffle / sharding; sharding gives a DistributedSampler; otherwise random or
    sequential by ``shuffle``, random being the default)."""
    if input_sampler is not None:
        if shuffle is not None or num_shards is not None or shard_id is not None:
            raise RuntimeError("sampler and shuffle / sharding cannot be specified at the same time")
        if not isinstance(input_sampler, Sampler):
            return IterSampler(input_sampler, num_samples)
        return input_sampler
    if num_shards is not None:
        return DistributedSampler(num_shards, shard_id, shuffle=shuffle if shuffle is not None else True,
                                  num_samples=num_samples)
    if shuffle is None or shuffle:
        return RandomSampler(num_samples=num_samples)
    return SequentialSampler(num_samples=num_samples)
