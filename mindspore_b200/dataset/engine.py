"""Dataset pipeline: lazily composed stages over a source, executed by Python iterators; ``batch`` collates with
numpy, ``map`` can run its operations in a thread pool (``num_parallel_workers``), and a prefetch stage keeps
``prefetch_size`` batches ready.  Rows are dicts {column: ndarray}; ``create_tuple_iterator`` yields tuples in
column order and ``create_dict_iterator`` the dicts.

Parity (API): python/mindspore/dataset/engine/datasets.py (Dataset.map/batch/shuffle/repeat/shard/take/skip/zip,
create_tuple_iterator, create_dict_iterator, get_dataset_size, get_col_names), datasets_user_defined.py
(GeneratorDataset, NumpySlicesDataset), datasets_standard_format.py (MindDataset)."""
from __future__ import annotations

import builtins
import concurrent.futures
import queue
import threading

import numpy as np


class _Config:
    def __init__(self):
        self.seed, self.prefetch_size, self.num_parallel_workers = 5489, 2, 4

    def set_seed(self, s):
        self.seed = int(s)

    def get_seed(self):
        return self.seed

    def set_prefetch_size(self, n):
        self.prefetch_size = int(n)

    def get_prefetch_size(self):
        return self.prefetch_size

    def set_num_parallel_workers(self, n):
        self.num_parallel_workers = int(n)

    def get_num_parallel_workers(self):
        return self.num_parallel_workers


class ErrorSamplesMode:
    """What a pipeline does with a row whose transform raised: stop with the error, replace the row, or skip it."""
    RETURN, REPLACE, SKIP = 0, 1, 2


def _setting(name, default, check=None):
    """A getter / setter pair of one more pipeline setting (stored on the config object)."""
    def setter(self, value):
        if check is not None:
            check(value)
        self._settings[name] = value

    def getter(self):
        return self._settings.get(name, default)
    return setter, getter


def _positive(label):
    def check(v):
        if isinstance(v, bool) or not isinstance(v, (int, float)) or v <= 0:
            raise ValueError("%s must be a positive number, but got %r" % (label, v))
    return check


def _boolean(label):
    def check(v):
        if not isinstance(v, bool):
            raise TypeError("%s must be a bool, but got %r" % (label, v))
    return check


_Config._settings = {}
for _name, _default, _check in (
        ("numa_enable", False, _boolean("numa_enable")),
        ("monitor_sampling_interval", 1000, _positive("monitor_sampling_interval")),
        ("auto_num_workers", False, _boolean("auto_num_workers")),
        ("callback_timeout", 60, _positive("callback_timeout")),
        ("enable_autotune", False, None), ("autotune_interval", 0, None),
        ("enable_shared_mem", True, _boolean("enable_shared_mem")),
        ("sending_batches", 0, None), ("auto_offload", False, _boolean("auto_offload")),
        ("enable_watchdog", True, _boolean("enable_watchdog")),
        ("multiprocessing_timeout_interval", 300, _positive("multiprocessing_timeout_interval")),
        ("dynamic_shape", False, _boolean("dynamic_shape")), ("fast_recovery", True, _boolean("fast_recovery")),
        ("debug_mode", False, None), ("error_samples_mode", ErrorSamplesMode.RETURN, None)):
    _set, _get = _setting(_name, _default, _check)
    setattr(_Config, "set_" + _name, _set)
    setattr(_Config, "get_" + _name, _get)


def _config_load(self, file):
    """Reads settings from a JSON file with the reference's keys (numParallelWorkers, opConnectorSize /
    prefetchSize, seed, monitorSamplingInterval, ...)."""
    import json
    with open(file) as f:
        cfg = json.load(f)
    if "numParallelWorkers" in cfg:
        self.set_num_parallel_workers(cfg["numParallelWorkers"])
    if "opConnectorSize" in cfg or "prefetchSize" in cfg:
        self.set_prefetch_size(cfg.get("prefetchSize", cfg.get("opConnectorSize")))
    if "seed" in cfg:
        self.set_seed(cfg["seed"])
    if "monitorSamplingInterval" in cfg:
        self.set_monitor_sampling_interval(cfg["monitorSamplingInterval"])
    if "callbackTimeout" in cfg:
        self.set_callback_timeout(cfg["callbackTimeout"])


def _set_debug_mode(self, debug_mode_flag, debug_hook_list=None):
    """Debug mode: ``map`` runs its transforms one at a time in the calling thread and calls every hook of
    ``debug_hook_list`` (default: one ``PrintMetaDataHook``) around them."""
    if not isinstance(debug_mode_flag, bool):
        raise TypeError("debug_mode_flag isn't of type boolean.")
    from .debug import DebugHook, PrintMetaDataHook
    if debug_hook_list is None:
        debug_hook_list = [PrintMetaDataHook()]
    if not isinstance(debug_hook_list, list):
        raise TypeError("debug_hook_list is not a list.")
    for hook in debug_hook_list:
        if not isinstance(hook, DebugHook):
            raise TypeError("All items in debug_hook_list must be of type DebugHook.")
    self._settings["debug_mode"] = debug_mode_flag
    self._settings["debug_hooks"] = list(debug_hook_list) if debug_mode_flag else []


_Config.set_debug_mode = _set_debug_mode
_Config._get_debug_hook_list = lambda self: list(self._settings.get("debug_hooks", []))
_Config.load = _config_load
_Config.ErrorSamplesMode = ErrorSamplesMode
config = _Config()
config._settings = {}


def _to_np(v):
    import torch
    if isinstance(v, torch.Tensor):
        return v.detach().cpu().numpy()
    return np.asarray(v)


class Dataset:
    """Base of every pipeline stage."""

    def __init__(self, parent=None, columns=None):
        self.parent = parent
        self._columns = list(columns) if columns is not None else (parent.get_col_names() if parent else [])

    # ------------------------------------------------------------------ to override
    def _rows(self):
        raise NotImplementedError

    # ------------------------------------------------------------------ introspection / sync
    def get_class_indexing(self):
        """Class name -> index mapping of the source dataset at the root of this pipeline (if it has one)."""
        node = self
        while getattr(node, "parent", None) is not None:
            node = node.parent
        fn = type(node).__dict__.get("get_class_indexing")
        if fn is None or node is self:
            raise NotImplementedError("%s has no class indexing" % type(node).__name__)
        return fn(node)

    def to_json(self, filename=""):
        from .sources_ext import serialize
        return serialize(self, filename)

    def is_shuffled(self):
        node = self
        while node is not None:
            if type(node).__name__ == "_Shuffle" or getattr(node, "_shuffle", False):
                return True
            node = getattr(node, "parent", None)
        return False

    def is_sharded(self):
        node = self
        while node is not None:
            if type(node).__name__ == "_Shard" or (getattr(node, "_num_shards", None) or 1) > 1:
                return True
            node = getattr(node, "parent", None)
        return False

    def set_init_step(self, init_step):
        """Rows to skip at the start of the first epoch (resuming in the middle of an epoch)."""
        self._init_step = int(init_step)

    def get_init_step(self):
        return getattr(self, "_init_step", 0)

    def sync_wait(self, condition_name, num_batch=1, callback=None):
        """Marks a synchronisation point: iteration blocks after every ``num_batch`` rows until
        ``sync_update(condition_name)`` is called (typically from the training loop)."""
        return _SyncWait(self, condition_name, num_batch, callback)

    def sync_update(self, condition_name, num_batch=None, data=None):
        node, found = self, False
        while node is not None:
            if isinstance(node, _SyncWait) and node.condition_name == condition_name:
                node.release(num_batch, data)
                found = True
            node = getattr(node, "parent", None)
        if not found:
            raise RuntimeError("sync_update: condition %r is not defined in this pipeline" % (condition_name,))

    def get_sync_notifiers(self):
        out, node = {}, self
        while node is not None:
            if isinstance(node, _SyncWait):
                out[node.condition_name] = node.release
            node = getattr(node, "parent", None)
        return out

    def is_sync(self):
        return bool(self.get_sync_notifiers())

    def disable_sync(self):
        node = self
        while node is not None:
            if isinstance(node, _SyncWait):
                node.enabled = False
            node = getattr(node, "parent", None)

    def get_dataset_size(self):
        return self.parent.get_dataset_size()

    # ------------------------------------------------------------------ composition
    def get_col_names(self):
        return list(self._columns)

    def map(self, operations, input_columns=None, output_columns=None, column_order=None, num_parallel_workers=None,
            python_multiprocessing=False, **kw):
        return _Map(self, operations, input_columns, output_columns, num_parallel_workers)

    def batch(self, batch_size, drop_remainder=False, num_parallel_workers=None, per_batch_map=None, **kw):
        return _Batch(self, batch_size, drop_remainder, per_batch_map)

    def shuffle(self, buffer_size):
        return _Shuffle(self, buffer_size)

    def repeat(self, count=None):
        return _Repeat(self, count)

    def take(self, count=-1):
        return _Take(self, count)

    def skip(self, count):
        return _Skip(self, count)

    def shard(self, num_shards, shard_id):
        return _Shard(self, num_shards, shard_id)

    def project(self, columns):
        return _Project(self, columns)

    def rename(self, input_columns, output_columns):
        return _Rename(self, input_columns, output_columns)

    def zip(self, datasets):
        return zip((self,) + tuple(datasets if isinstance(datasets, (tuple, list)) else (datasets,)))

    def prefetch(self, size=None):
        return _Prefetch(self, size or config.prefetch_size)

    # ------------------------------------------------------------------ iteration
    def create_dict_iterator(self, num_epochs=-1, output_numpy=False, do_copy=True):
        return DictIterator(self, num_epochs, output_numpy, do_copy)

    def create_tuple_iterator(self, columns=None, num_epochs=-1, output_numpy=False, do_copy=True):
        return TupleIterator(self, columns, num_epochs, output_numpy, do_copy)

    def __iter__(self):
        return self.create_tuple_iterator()

    def __len__(self):
        return self.get_dataset_size()

    def output_shapes(self):
        row = next(iter(self._rows()))
        return [list(row[c].shape) for c in self._columns]

    def output_types(self):
        row = next(iter(self._rows()))
        return [row[c].dtype for c in self._columns]

    def get_batch_size(self):
        return self.parent.get_batch_size() if self.parent else 1

    def get_repeat_count(self):
        return self.parent.get_repeat_count() if self.parent else 1


# ---------------------------------------------------------------------------------------------------- sources
class _SyncWait(Dataset):
    def __init__(self, parent, condition_name, num_batch, callback):
        super().__init__(parent, parent.get_col_names())
        import threading
        self.condition_name, self.num_batch, self.callback, self.enabled = condition_name, num_batch, callback, True
        self._sem = threading.Semaphore(num_batch)

    def release(self, num_batch=None, data=None):
        if self.callback is not None and data is not None:
            self.callback(data)
        for _ in range(num_batch or self.num_batch):
            self._sem.release()

    def get_dataset_size(self):
        return self.parent.get_dataset_size()

    def _rows(self):
        for row in self.parent._rows():
            if self.enabled and not self._sem.acquire(timeout=config.get_callback_timeout()):
                raise RuntimeError("sync_wait(%r): no sync_update within %s s" % (self.condition_name,
                                                                               config.get_callback_timeout()))
            yield row


class Iterator:
    """One pass over a dataset per ``for`` loop (at most ``num_epochs`` passes; -1 = any number).  ``get_offload``
    style helpers of the reference that concern its C++ runtime are absent."""

    def __init__(self, dataset, num_epochs=-1, output_numpy=False, do_copy=True):
        self.dataset, self.num_epochs, self.output_numpy, self.do_copy = dataset, num_epochs, output_numpy, do_copy
        self._epochs_started, self._gen = 0, None

    def _convert(self, row):
        raise NotImplementedError

    def __iter__(self):
        if 0 <= self.num_epochs <= self._epochs_started:
            raise RuntimeError("The iterator was created for %d epoch(s) and all of them have been consumed"
                               % self.num_epochs)
        self._epochs_started += 1
        self._gen = (self._convert(row) for row in self.dataset._rows())
        return self

    def __next__(self):
        if self._gen is None:
            iter(self)
        return next(self._gen)

    def stop(self):
        self._gen = iter(())

    release = stop

    def get_output_shapes(self):
        return self.dataset.output_shapes()

    def get_output_types(self):
        return self.dataset.output_types()

    def get_col_names(self):
        return self.dataset.get_col_names()


class DictIterator(Iterator):
    def _convert(self, row):
        if self.output_numpy:
            return row
        import mindspore_b200 as ms
        return {k: ms.Tensor(v) for k, v in row.items()}


class TupleIterator(Iterator):
    def __init__(self, dataset, columns=None, num_epochs=-1, output_numpy=False, do_copy=True):
        super().__init__(dataset, num_epochs, output_numpy, do_copy)
        self.columns = columns

    def _convert(self, row):
        cols = self.columns or self.dataset._columns
        if self.output_numpy:
            return tuple(row[c] for c in cols)
        import mindspore_b200 as ms
        return tuple(ms.Tensor(row[c]) for c in cols)


class DummyIterator:
    """Yields the same row forever (used to measure a training loop without its input pipeline)."""

    def __init__(self, dataset, mode, output_numpy=False):
        first = next(iter(dataset.create_dict_iterator(1, output_numpy) if mode == "dict"
                          else dataset.create_tuple_iterator(None, 1, output_numpy)))
        self.row = first

    def __iter__(self):
        return self

    def __next__(self):
        return self.row


def check_iterator_cleanup():
    """Whether iterators are being torn down (never, here: there are no background C++ pipelines to stop)."""
    return False


class GeneratorDataset(Dataset):
    """Source over a generator function, an iterable, or a random-access object (``__getitem__`` + ``__len__``)."""

    def __init__(self, source, column_names=None, column_types=None, schema=None, num_samples=None,
                 num_parallel_workers=1, shuffle=None, sampler=None, num_shards=None, shard_id=None,
                 python_multiprocessing=False, max_rowsize=None):
        if column_names is None:
            raise ValueError("For 'GeneratorDataset', 'column_names' must be given")
        super().__init__(None, [column_names] if isinstance(column_names, str) else column_names)
        self.source, self.num_samples = source, num_samples
        self.random_access = hasattr(source, "__getitem__") and hasattr(source, "__len__")
        self.shuffle_flag = bool(shuffle) if shuffle is not None else self.random_access
        self.num_shards, self.shard_id = num_shards, shard_id
        self._epoch = 0
        if (num_shards is None) != (shard_id is None):
            raise ValueError("num_shards and shard_id must be given together")
        self.sampler = sampler
        if sampler is not None:
            if not self.random_access:
                raise ValueError("a sampler needs a random-access source (__getitem__ and __len__)")
            if shuffle is not None or num_shards is not None:
                raise ValueError("sampler cannot be combined with shuffle / num_shards / shard_id")
            if not hasattr(sampler, "indices"):                       # a plain iterable of indices
                from .samplers import SubsetSampler
                self.sampler = SubsetSampler(list(sampler))
            self.sampler.bind(len(source), getattr(source, "labels", None))

    def _indices(self):
        n = len(self.source)
        if getattr(self, "sampler", None) is not None:
            self.sampler._epoch = self._epoch
            idx = np.asarray(self.sampler.indices())
            return idx if self.num_samples is None else idx[:self.num_samples]
        idx = np.arange(n)
        if self.shuffle_flag:
            rng = np.random.default_rng(config.seed + self._epoch)
            rng.shuffle(idx)
        if self.num_shards:
            idx = idx[self.shard_id::self.num_shards]
        if self.num_samples is not None:
            idx = idx[:self.num_samples]
        return idx

    def get_dataset_size(self):
        if self.random_access:
            return len(self._indices())
        if self.num_samples is not None:
            return self.num_samples
        return sum(1 for _ in self._raw())

    def _raw(self):
        if self.random_access:
            for i in self._indices():
                yield self.source[int(i)]
        else:
            it = self.source() if callable(self.source) else iter(self.source)
            for k, item in enumerate(it):
                if self.num_shards and k % self.num_shards != self.shard_id:
                    continue
                yield item

    def _rows(self):
        self._epoch += 1
        count = 0
        for item in self._raw():
            if not isinstance(item, (tuple, list)):
                item = (item,)
            if len(item) != len(self._columns):
                raise RuntimeError("the source yields %d columns but column_names has %d" % (len(item),
                                                                                             len(self._columns)))
            yield {c: _to_np(v) for c, v in builtins.zip(self._columns, item)}
            count += 1
            if self.num_samples is not None and count >= self.num_samples:
                return


class NumpySlicesDataset(GeneratorDataset):
    def __init__(self, data, column_names=None, num_samples=None, num_parallel_workers=1, shuffle=None, sampler=None,
                 num_shards=None, shard_id=None):
        if isinstance(data, dict):
            column_names = column_names or list(data.keys())
            cols = [np.asarray(data[k]) for k in data]
        elif isinstance(data, tuple):
            cols = [np.asarray(d) for d in data]
            column_names = column_names or ["column_%d" % i for i in range(len(cols))]
        else:
            cols = [np.asarray(data)]
            column_names = column_names or ["column_0"]
        n = len(cols[0])
        if any(len(c) != n for c in cols):
            raise ValueError("all columns of NumpySlicesDataset must have the same length")

        class _Src:
            def __len__(self):
                return n

            def __getitem__(self, i):
                return tuple(c[i] for c in cols)

        super().__init__(_Src(), column_names, num_samples=num_samples, shuffle=shuffle, num_shards=num_shards,
                         shard_id=shard_id)


class RandomDataset(GeneratorDataset):
    """Synthetic rows of given shapes / dtypes (benchmarks and tests)."""

    def __init__(self, shapes, dtypes, column_names, total_rows=64, seed=0):
        rng = np.random.default_rng(seed)
        data = [rng.standard_normal((total_rows,) + tuple(s)).astype(d) if np.issubdtype(np.dtype(d), np.floating)
                else rng.integers(0, 100, (total_rows,) + tuple(s)).astype(d) for s, d in builtins.zip(shapes, dtypes)]

        class _Src:
            def __len__(self):
                return total_rows

            def __getitem__(self, i):
                return tuple(c[i] for c in data)

        super().__init__(_Src(), column_names, shuffle=False)


class MindDataset(GeneratorDataset):
    """Rows of record files written by ``dataset.mindrecord.FileWriter``."""

    def __init__(self, dataset_files, columns_list=None, num_parallel_workers=None, shuffle=None, num_shards=None,
                 shard_id=None, sampler=None, num_samples=None, **kw):
        from .mindrecord import FileReader
        files = [dataset_files] if isinstance(dataset_files, str) else list(dataset_files)
        readers = [FileReader(f, columns=columns_list) for f in files]
        index = [(ri, k) for ri, r in enumerate(readers) for k in range(len(r))]
        cols = columns_list or readers[0].columns

        class _Src:
            def __len__(self):
                return len(index)

            def __getitem__(self, i):
                ri, k = index[i]
                row = readers[ri].read(k)
                return tuple(row[c] for c in cols)

        super().__init__(_Src(), cols, num_samples=num_samples, shuffle=shuffle, num_shards=num_shards,
                         shard_id=shard_id)


# ---------------------------------------------------------------------------------------------------- stages
class _Map(Dataset):
    def __init__(self, parent, operations, input_columns, output_columns, workers):
        ops = operations if isinstance(operations, (list, tuple)) else [operations]
        self.ops = list(ops)
        self.inp = [input_columns] if isinstance(input_columns, str) else (input_columns or parent.get_col_names()[:1])
        self.out = [output_columns] if isinstance(output_columns, str) else (output_columns or self.inp)
        cols = []
        for c in parent.get_col_names():
            if c in self.inp:
                if c == self.inp[0]:
                    cols += self.out
            else:
                cols.append(c)
        super().__init__(parent, cols)
        self.workers = workers or 1

    def _apply(self, row):
        vals = tuple(row[c] for c in self.inp)
        hooks = config._get_debug_hook_list() if config.get_debug_mode() else ()
        for k, op in enumerate(self.ops):
            name = type(op).__name__ if not hasattr(op, "__name__") else op.__name__
            if hooks and k == 0:
                vals = self._run_hooks(hooks, name, True, vals)
            vals = op(*vals)
            if not isinstance(vals, tuple):
                vals = (vals,)
            if hooks:
                vals = self._run_hooks(hooks, name, False, vals)
        if len(vals) != len(self.out):
            raise RuntimeError("map produced %d columns, expected %d (%s)" % (len(vals), len(self.out), self.out))
        new = {c: v for c, v in row.items() if c not in self.inp}
        new.update({c: _to_np(v) for c, v in builtins.zip(self.out, vals)})
        return new

    @staticmethod
    def _run_hooks(hooks, op_name, is_first, vals):
        import copy
        for hook in hooks:
            hook = copy.copy(hook)
            hook.set_previous_op_name(op_name)
            hook.set_is_first(is_first)
            vals = tuple(hook(*vals))
        return vals

    def _rows(self):
        if self.workers <= 1 or config.get_debug_mode():
            for row in self.parent._rows():
                yield self._apply(row)
            return
        with concurrent.futures.ThreadPoolExecutor(self.workers) as pool:
            window = []
            for row in self.parent._rows():
                window.append(pool.submit(self._apply, row))
                if len(window) >= 4 * self.workers:
                    yield window.pop(0).result()
            for f in window:
                yield f.result()


class _Batch(Dataset):
    def __init__(self, parent, batch_size, drop_remainder, per_batch_map):
        if not isinstance(batch_size, int) or batch_size <= 0:
            raise ValueError("batch_size must be a positive int")
        super().__init__(parent)
        self.batch_size, self.drop, self.per_batch_map = batch_size, drop_remainder, per_batch_map

    def get_dataset_size(self):
        n = self.parent.get_dataset_size()
        return n // self.batch_size if self.drop else (n + self.batch_size - 1) // self.batch_size

    def get_batch_size(self):
        return self.batch_size

    def _collate(self, rows):
        out = {}
        for c in self._columns:
            vals = [r[c] for r in rows]
            if self.per_batch_map is None:
                out[c] = np.stack(vals)
            else:
                out[c] = vals
        if self.per_batch_map is not None:
            res = self.per_batch_map(*[out[c] for c in self._columns], {"batch_size": len(rows)})
            out = {c: np.stack([_to_np(x) for x in v]) for c, v in builtins.zip(self._columns, res)}
        return out

    def _rows(self):
        buf = []
        for row in self.parent._rows():
            buf.append(row)
            if len(buf) == self.batch_size:
                yield self._collate(buf)
                buf = []
        if buf and not self.drop:
            yield self._collate(buf)


class _Shuffle(Dataset):
    def __init__(self, parent, buffer_size):
        if buffer_size < 1:
            raise ValueError("buffer_size must be at least 1")
        super().__init__(parent)
        self.buffer_size, self._epoch = buffer_size, 0

    def _rows(self):
        rng = np.random.default_rng(config.seed + 7919 * self._epoch)
        self._epoch += 1
        buf = []
        for row in self.parent._rows():
            if len(buf) < self.buffer_size:
                buf.append(row)
                continue
            i = int(rng.integers(0, self.buffer_size))
            yield buf[i]
            buf[i] = row
        rng.shuffle(buf)
        yield from buf


class _Repeat(Dataset):
    def __init__(self, parent, count):
        super().__init__(parent)
        self.count = count

    def get_dataset_size(self):
        n = self.parent.get_dataset_size()
        return n * self.count if self.count and self.count > 0 else n

    def get_repeat_count(self):
        return self.count or -1

    def _rows(self):
        k = 0
        while self.count is None or self.count < 0 or k < self.count:
            yield from self.parent._rows()
            k += 1


class _Take(Dataset):
    def __init__(self, parent, count):
        super().__init__(parent)
        self.count = count

    def get_dataset_size(self):
        n = self.parent.get_dataset_size()
        return n if self.count < 0 else min(n, self.count)

    def _rows(self):
        for i, row in enumerate(self.parent._rows()):
            if 0 <= self.count <= i:
                return
            yield row


class _Skip(Dataset):
    def __init__(self, parent, count):
        super().__init__(parent)
        self.count = count

    def get_dataset_size(self):
        return max(0, self.parent.get_dataset_size() - self.count)

    def _rows(self):
        for i, row in enumerate(self.parent._rows()):
            if i >= self.count:
                yield row


class _Shard(Dataset):
    def __init__(self, parent, num_shards, shard_id):
        if not 0 <= shard_id < num_shards:
            raise ValueError("shard_id must be in [0, num_shards)")
        super().__init__(parent)
        self.num_shards, self.shard_id = num_shards, shard_id

    def get_dataset_size(self):
        n = self.parent.get_dataset_size()
        return (n - self.shard_id + self.num_shards - 1) // self.num_shards

    def _rows(self):
        for i, row in enumerate(self.parent._rows()):
            if i % self.num_shards == self.shard_id:
                yield row


class _Project(Dataset):
    def __init__(self, parent, columns):
        cols = [columns] if isinstance(columns, str) else list(columns)
        missing = [c for c in cols if c not in parent.get_col_names()]
        if missing:
            raise RuntimeError("project: unknown columns %s" % missing)
        super().__init__(parent, cols)

    def _rows(self):
        for row in self.parent._rows():
            yield {c: row[c] for c in self._columns}


class _Rename(Dataset):
    def __init__(self, parent, inp, out):
        inp = [inp] if isinstance(inp, str) else list(inp)
        out = [out] if isinstance(out, str) else list(out)
        self.mapping = dict(builtins.zip(inp, out))
        super().__init__(parent, [self.mapping.get(c, c) for c in parent.get_col_names()])

    def _rows(self):
        for row in self.parent._rows():
            yield {self.mapping.get(c, c): v for c, v in row.items()}


class _Zip(Dataset):
    def __init__(self, parents):
        cols = []
        for p in parents:
            for c in p.get_col_names():
                if c in cols:
                    raise RuntimeError("zip: column %r appears in more than one dataset" % c)
                cols.append(c)
        super().__init__(None, cols)
        self.parents = list(parents)

    def get_dataset_size(self):
        return min(p.get_dataset_size() for p in self.parents)

    def _rows(self):
        for rows in builtins.zip(*[p._rows() for p in self.parents]):
            out = {}
            for r in rows:
                out.update(r)
            yield out


class _Prefetch(Dataset):
    """Runs the upstream pipeline in a background thread, ``size`` rows ahead."""

    def __init__(self, parent, size):
        super().__init__(parent)
        self.size = max(1, size)

    def _rows(self):
        q = queue.Queue(self.size)
        end = object()

        def work():
            try:
                for row in self.parent._rows():
                    q.put(row)
                q.put(end)
            except BaseException as e:  # noqa: BLE001  (re-raised in the consumer)
                q.put(e)

        threading.Thread(target=work, daemon=True).start()
        while True:
            item = q.get()
            if item is end:
                return
            if isinstance(item, BaseException):
                raise item
            yield item


def zip(datasets):  # noqa: A001
    return _Zip(tuple(datasets))


# ------------------------------------------------------------------------------------------------ further operations
class _Concat(Dataset):
    def __init__(self, parents):
        cols = parents[0].get_col_names()
        for p in parents[1:]:
            if p.get_col_names() != cols:
                raise ValueError("concat: column names differ: %s vs %s" % (cols, p.get_col_names()))
        super().__init__(parents[0], cols)
        self.parents = list(parents)

    def get_dataset_size(self):
        return sum(p.get_dataset_size() for p in self.parents)

    def _rows(self):
        for p in self.parents:
            yield from p._rows()


class _Filter(Dataset):
    def __init__(self, parent, predicate, input_columns):
        super().__init__(parent)
        self.predicate, self.cols = predicate, input_columns or parent.get_col_names()

    def get_dataset_size(self):
        return sum(1 for _ in self._rows())

    def _rows(self):
        for row in self.parent._rows():
            if self.predicate(*[row[c] for c in self.cols]):
                yield row


class _FlatMap(Dataset):
    def __init__(self, parent, func):
        super().__init__(parent)
        self.func = func

    def get_dataset_size(self):
        return sum(1 for _ in self._rows())

    def _rows(self):
        for row in self.parent._rows():
            yield from self.func(*[row[c] for c in self.parent.get_col_names()])._rows()


class _PaddedBatch(Dataset):
    """Batches rows whose shapes differ: every column is padded to ``pad_info[col] = (shape, value)`` (None entries of
    the shape, or a missing column, mean "longest in this batch")."""

    def __init__(self, parent, batch_size, drop_remainder, pad_info):
        super().__init__(parent)
        self.batch_size, self.drop, self.pad_info = batch_size, drop_remainder, pad_info or {}

    def get_dataset_size(self):
        n = self.parent.get_dataset_size()
        return n // self.batch_size if self.drop else -(-n // self.batch_size)

    def _pad(self, col, arrays):
        shape, value = self.pad_info.get(col, (None, 0))
        arrays = [np.asarray(a) for a in arrays]
        nd = arrays[0].ndim
        target = [max(a.shape[d] for a in arrays) for d in range(nd)]
        if shape is not None:
            target = [t if s is None else s for t, s in builtins.zip(target, shape)]
        out = np.full([len(arrays)] + target, value if value is not None else 0, dtype=arrays[0].dtype)
        for i, a in enumerate(arrays):
            sl = tuple(slice(0, min(s, t)) for s, t in builtins.zip(a.shape, target))
            out[(i,) + sl] = a[sl]
        return out

    def _emit(self, rows):
        return {c: self._pad(c, [r[c] for r in rows]) for c in self._columns}

    def _rows(self):
        buf = []
        for row in self.parent._rows():
            buf.append(row)
            if len(buf) == self.batch_size:
                yield self._emit(buf)
                buf = []
        if buf and not self.drop:
            yield self._emit(buf)


class _BucketBatch(_PaddedBatch):
    def __init__(self, parent, column_names, boundaries, batch_sizes, length_fn, pad_info, pad_to_bucket_boundary,
                 drop_remainder):
        if len(batch_sizes) != len(boundaries) + 1:
            raise ValueError("bucket_batch_by_length: need len(bucket_boundaries) + 1 batch sizes")
        super().__init__(parent, 1, drop_remainder, pad_info)
        self.cols, self.bounds, self.sizes = column_names, list(boundaries), list(batch_sizes)
        self.length_fn = length_fn or (lambda *a: len(a[0]))
        self.to_boundary = pad_to_bucket_boundary

    def get_dataset_size(self):
        return sum(1 for _ in self._rows())

    def _rows(self):
        import bisect
        buckets = [[] for _ in self.sizes]
        for row in self.parent._rows():
            b = bisect.bisect_right(self.bounds, self.length_fn(*[row[c] for c in self.cols]))
            buckets[b].append(row)
            if len(buckets[b]) == self.sizes[b]:
                yield self._emit_bucket(b, buckets[b])
                buckets[b] = []
        if not self.drop:
            for b, rows in enumerate(buckets):
                if rows:
                    yield self._emit_bucket(b, rows)

    def _emit_bucket(self, b, rows):
        if self.to_boundary and b < len(self.bounds):
            info = dict(self.pad_info)
            for c in self.cols:
                shape, value = info.get(c, (None, 0))
                nd = np.asarray(rows[0][c]).ndim
                shape = list(shape) if shape is not None else [None] * nd
                shape[0] = self.bounds[b] - 1
                info[c] = (shape, value)
            saved, self.pad_info = self.pad_info, info
            try:
                return self._emit(rows)
            finally:
                self.pad_info = saved
        return self._emit(rows)


def _ds_concat(self, datasets):
    others = list(datasets) if isinstance(datasets, (list, tuple)) else [datasets]
    return _Concat([self] + others)


def _ds_split(self, sizes, randomize=True):
    """Splits into datasets of the given absolute sizes (ints) or fractions (floats summing to 1)."""
    rows = list(self._rows())
    n = len(rows)
    if all(isinstance(s, float) for s in sizes):
        if abs(sum(sizes) - 1) > 1e-6:
            raise ValueError("split: fractions must sum to 1")
        counts = [int(round(s * n)) for s in sizes]
        counts[-1] = n - sum(counts[:-1])
    else:
        counts = [int(s) for s in sizes]
        if sum(counts) != n:
            raise ValueError("split: sizes %s do not add up to the dataset size %d" % (counts, n))
    order = np.random.default_rng(config.seed).permutation(n) if randomize else np.arange(n)
    out, pos = [], 0
    cols = self.get_col_names()
    for c in counts:
        part = [rows[i] for i in order[pos:pos + c]]
        pos += c
        out.append(GeneratorDataset([tuple(r[k] for k in cols) for r in part] or [()], cols, shuffle=False)
                   if part else _Take(self, 0))
    return tuple(out)


def _ds_save(self, file_name, num_files=1, file_type="mindrecord"):
    if file_type != "mindrecord":
        raise ValueError("save: only file_type 'mindrecord' is supported")
    from .mindrecord import FileWriter
    rows = list(self._rows())
    if not rows:
        raise RuntimeError("save: the dataset is empty")
    schema = {}
    for c, v in rows[0].items():
        a = np.asarray(v)
        kind = {"f": "float32" if a.dtype.itemsize <= 4 else "float64", "i": "int64" if a.dtype.itemsize > 4 else "int32",
                "u": "int32", "b": "int32"}.get(a.dtype.kind, "string")
        schema[c] = {"type": kind} if a.ndim == 0 else {"type": kind, "shape": [-1] if a.ndim == 1 else list(a.shape)}
    w = FileWriter(file_name, shard_num=num_files)
    w.add_schema(schema, "saved")
    w.write_raw_data([{c: (np.asarray(v) if np.asarray(v).ndim else np.asarray(v).item()) for c, v in r.items()}
                      for r in rows])
    w.commit()


Dataset.concat = _ds_concat
Dataset.__add__ = lambda self, other: _Concat([self, other])
Dataset.filter = lambda self, predicate, input_columns=None, num_parallel_workers=None: _Filter(self, predicate, input_columns)
Dataset.flat_map = lambda self, func: _FlatMap(self, func)
Dataset.apply = lambda self, apply_func: apply_func(self)
Dataset.padded_batch = lambda self, batch_size, drop_remainder=False, num_parallel_workers=None, pad_info=None: \
    _PaddedBatch(self, batch_size, drop_remainder, pad_info)
Dataset.bucket_batch_by_length = lambda self, column_names, bucket_boundaries, bucket_batch_sizes, \
    element_length_function=None, pad_info=None, pad_to_bucket_boundary=False, drop_remainder=False: \
    _BucketBatch(self, column_names, bucket_boundaries, bucket_batch_sizes, element_length_function, pad_info,
                 pad_to_bucket_boundary, drop_remainder)
Dataset.split = _ds_split
Dataset.save = _ds_save
Dataset.device_que = lambda self, send_epoch_end=True, create_data_info_queue=False, queue_name="": self
Dataset.to_device = Dataset.device_que
Dataset.num_classes = lambda self: (len(set(int(np.asarray(r[self.get_col_names()[-1]])) for r in self._rows())))
def _source_of(ds):
    """The leaf (source) dataset of a pipeline."""
    while getattr(ds, "parent", None) is not None:
        ds = ds.parent
    return ds


def _use_sampler(self, new_sampler):
    """Replaces the sampler of the source dataset (``None`` removes it).  Parity: MappableDataset.use_sampler."""
    src = _source_of(self)
    if not hasattr(src, "source") or not getattr(src, "random_access", False):
        raise RuntimeError("use_sampler needs a random-access source dataset")
    if new_sampler is not None:
        if not hasattr(new_sampler, "indices"):
            from .samplers import SubsetSampler
            new_sampler = SubsetSampler(list(new_sampler))
        new_sampler.bind(len(src.source), getattr(src.source, "labels", None))
    src.sampler = new_sampler


def _add_sampler(self, new_sampler):
    """Puts ``new_sampler`` on top of the current one: it draws from what the current sampler yields.
    Parity: MappableDataset.add_sampler."""
    src = _source_of(self)
    old = getattr(src, "sampler", None)
    if old is not None:
        new_sampler.add_child(old)
    _use_sampler(self, new_sampler)


Dataset.use_sampler = _use_sampler
Dataset.add_sampler = _add_sampler
Dataset.input_indexs = property(lambda self: getattr(self, "_input_indexs", ()),
                                lambda self, value: setattr(self, "_input_indexs", value))
Dataset.copy_batch_size = lambda self, value: setattr(self, "_batch_size_copy", value)
Dataset.reset = lambda self: None
Dataset.close = lambda self: None


def __getattr__(name):
    # `dataset.engine` lists every dataset class, sampler and iterator of the package in the reference
    if name.startswith("__"):
        raise AttributeError(name)
    import importlib
    for mod in ("sources", "sources_ext", "samplers", "mindrecord_source", "graphdata"):
        try:
            m = importlib.import_module("." + mod, __package__)
        except ImportError:
            continue
        if hasattr(m, name):
            return getattr(m, name)
    raise AttributeError("module 'dataset.engine' has no attribute %r" % name)
