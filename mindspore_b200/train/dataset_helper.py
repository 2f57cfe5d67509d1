"""Dataset iteration helpers.

``DatasetHelper(dataset, dataset_sink_mode)`` iterates any iterable of batches (lists / tuples of arrays or
tensors, objects with ``create_tuple_iterator`` / ``get_dataset_size``).  In sink mode a background thread
stages the next batches in pinned host memory and issues the host->device copies on a side CUDA stream, the
role of the reference's device data queue (runtime/data_queue, GetNext op).
Parity: mindspore/python/mindspore/train/dataset_helper.py:213 (connect_network_with_dataset), :311.
"""
import queue
import threading

import numpy as np
import torch

_queues = {}


def _pop_queue(name):
    return _queues[name].get()


def _as_tensor(x, pin):
    if isinstance(x, np.ndarray):
        x = torch.from_numpy(np.ascontiguousarray(x))
    if isinstance(x, torch.Tensor) and pin and not x.is_cuda:
        try:
            x = x.pin_memory()
        except RuntimeError:
            pass
    return x


class DatasetHelper:
    def __init__(self, dataset, dataset_sink_mode=True, sink_size=-1, epoch_num=1):
        self.dataset = dataset
        self.sink = bool(dataset_sink_mode) and torch.cuda.is_available()
        self.sink_size = sink_size

    def dataset_size(self):
        ds = self.dataset
        if hasattr(ds, "get_dataset_size"):
            return ds.get_dataset_size()
        try:
            return len(ds)
        except TypeError:
            return 1

    get_dataset_size = dataset_size

    def _source(self):
        ds = self.dataset
        if hasattr(ds, "create_tuple_iterator"):
            return ds.create_tuple_iterator()
        return iter(ds)

    def __iter__(self):
        if not self.sink:
            for b in self._source():
                yield tuple(_as_tensor(x, False) for x in (b if isinstance(b, (tuple, list)) else (b,)))
            return
        q = queue.Queue(maxsize=2)
        stream = torch.cuda.Stream()
        dev = torch.device("cuda", torch.cuda.current_device())

        def worker():
            try:
                for b in self._source():
                    host = tuple(_as_tensor(x, True) for x in (b if isinstance(b, (tuple, list)) else (b,)))
                    with torch.cuda.stream(stream):
                        devb = tuple(x.to(dev, non_blocking=True) if isinstance(x, torch.Tensor) else x for x in host)
                        ev = torch.cuda.Event()
                        ev.record(stream)
                    q.put((devb, ev, host))
            finally:
                q.put(None)

        threading.Thread(target=worker, daemon=True).start()
        while True:
            item = q.get()
            if item is None:
                return
            devb, ev, _host = item
            torch.cuda.current_stream().wait_event(ev)
            yield devb

    def types_shapes(self):
        return None, None

    def sink_size_(self):
        return self.sink_size

    def stop_send(self):
        pass

    def release(self):
        pass


def connect_network_with_dataset(network, dataset_helper):
    return network
