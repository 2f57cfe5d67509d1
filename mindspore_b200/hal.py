"""``mindspore_b200.hal``: streams, events, device and memory queries
(python/mindspore/hal/{stream,event,device,memory}.py)."""
from __future__ import annotations

import torch


def is_initialized(device_target="GPU"):
    return torch.cuda.is_initialized() if device_target == "GPU" else True


def is_available(device_target="GPU"):
    return torch.cuda.is_available() if device_target == "GPU" else device_target == "CPU"


def device_count(device_target="GPU"):
    return torch.cuda.device_count() if device_target == "GPU" else 1


def get_device_name(device_id=0, device_target="GPU"):
    return torch.cuda.get_device_name(device_id) if device_target == "GPU" else "CPU"


def get_device_capability(device_id=0, device_target="GPU"):
    return torch.cuda.get_device_capability(device_id) if device_target == "GPU" else None


def get_device_properties(device_id=0, device_target="GPU"):
    return torch.cuda.get_device_properties(device_id) if device_target == "GPU" else None


def get_arch_list(device_target="GPU"):
    return ["sm_100a"] if device_target == "GPU" else []


class Stream:
    def __init__(self, priority=0, **kwargs):
        self._s = kwargs.get("stream") or (torch.cuda.Stream(priority=priority) if torch.cuda.is_available() else None)

    @property
    def id(self):
        return self._s.cuda_stream if self._s is not None else 0

    def record_event(self, event=None):
        event = event or Event()
        event.record(self)
        return event

    def wait_event(self, event):
        if self._s is not None:
            self._s.wait_event(event._e)

    def wait_stream(self, stream):
        if self._s is not None:
            self._s.wait_stream(stream._s)

    def synchronize(self, timeout=None):
        if self._s is None:
            return
        if timeout is None:
            self._s.synchronize()
            return
        ev = torch.cuda.Event()
        ev.record(self._s)
        wait_event(ev.query, timeout, "the stream")

    def query(self):
        return self._s.query() if self._s is not None else True

    def __enter__(self):
        self._ctx = torch.cuda.stream(self._s) if self._s is not None else None
        if self._ctx:
            self._ctx.__enter__()
        return self

    def __exit__(self, *exc):
        if self._ctx:
            self._ctx.__exit__(*exc)


class StreamCtx:
    def __init__(self, ctx_stream):
        self.stream = ctx_stream

    def __enter__(self):
        return self.stream.__enter__()

    def __exit__(self, *exc):
        return self.stream.__exit__(*exc)


class Event:
    def __init__(self, enable_timing=False, blocking=False):
        self._e = torch.cuda.Event(enable_timing=enable_timing, blocking=blocking) if torch.cuda.is_available() \
            else None

    def record(self, stream=None):
        if self._e is not None:
            self._e.record(stream._s if stream is not None else None)

    def wait(self, stream=None):
        if self._e is not None:
            (stream._s if stream is not None else torch.cuda.current_stream()).wait_event(self._e)

    def synchronize(self):
        if self._e is not None:
            self._e.synchronize()

    def query(self):
        return self._e.query() if self._e is not None else True

    def elapsed_time(self, end_event):
        return self._e.elapsed_time(end_event._e)


def current_stream():
    return Stream(stream=torch.cuda.current_stream()) if torch.cuda.is_available() else Stream()


def default_stream():
    return Stream(stream=torch.cuda.default_stream()) if torch.cuda.is_available() else Stream()


def set_cur_stream(stream):
    if stream._s is not None:
        torch.cuda.set_stream(stream._s)


class StreamSyncTimeout(RuntimeError):
    """The device did not finish the work queued before ``synchronize(timeout=...)`` within the limit (a hung
    collective after a peer was lost, typically): the caller can tear the communicator down and recover instead of
    blocking for ever in the driver."""


def wait_event(query, timeout, what="the device", poll_s=0.001, clock=None, sleep=None):
    """Polls ``query()`` (true when done) until it holds or ``timeout`` seconds pass; raises StreamSyncTimeout."""
    import time
    clock = clock or time.monotonic
    sleep = sleep or time.sleep
    deadline = clock() + float(timeout)
    while not query():
        if clock() >= deadline:
            raise StreamSyncTimeout("%s did not finish within %.1f s" % (what, float(timeout)))
        sleep(poll_s)
        poll_s = min(poll_s * 2, 0.05)


def synchronize(timeout=None):
    """Waits for all queued device work.  With ``timeout`` (seconds; default from ``MS_STREAM_SYNC_TIMEOUT`` when
    set) the wait polls an event instead of blocking in the driver and raises ``StreamSyncTimeout`` when it runs out;
    afterwards the per-device status word of the kernels' own bounded waits is checked as well
    (runtime/device/stream_synchronizer.cc:33-63 waits with a time limit when recovery is enabled)."""
    import os
    if not torch.cuda.is_available():
        return
    if timeout is None and os.environ.get("MS_STREAM_SYNC_TIMEOUT"):
        timeout = float(os.environ["MS_STREAM_SYNC_TIMEOUT"])
    if timeout is None:
        torch.cuda.synchronize()
        return
    ev = torch.cuda.Event()
    ev.record()
    wait_event(ev.query, timeout, "device %d" % torch.cuda.current_device())
    from . import _native
    status = _native.device_status(clear=False) if _native._cuda is not None else 0
    if status:
        raise StreamSyncTimeout("a kernel gave up a bounded wait (device status word %d)" % status)


def memory_stats(device_target="GPU"):
    if not torch.cuda.is_available():
        return {}
    s = torch.cuda.memory_stats()
    return {"total_reserved_memory": s.get("reserved_bytes.all.current", 0),
            "total_allocated_memory": s.get("allocated_bytes.all.current", 0),
            "max_reserved_memory": s.get("reserved_bytes.all.peak", 0),
            "max_allocated_memory": s.get("allocated_bytes.all.peak", 0)}


def memory_reserved(device_target="GPU"):
    return torch.cuda.memory_reserved() if torch.cuda.is_available() else 0


def max_memory_reserved(device_target="GPU"):
    return torch.cuda.max_memory_reserved() if torch.cuda.is_available() else 0


def memory_allocated(device_target="GPU"):
    return torch.cuda.memory_allocated() if torch.cuda.is_available() else 0


def max_memory_allocated(device_target="GPU"):
    return torch.cuda.max_memory_allocated() if torch.cuda.is_available() else 0


def reset_peak_memory_stats(device_target="GPU"):
    if torch.cuda.is_available():
        torch.cuda.reset_peak_memory_stats()


def reset_max_memory_reserved(device_target="GPU"):
    reset_peak_memory_stats(device_target)


def reset_max_memory_allocated(device_target="GPU"):
    reset_peak_memory_stats(device_target)


def empty_cache():
    if torch.cuda.is_available():
        torch.cuda.empty_cache()


def memory_summary(device_target="GPU"):
    """Readable table of the allocator's counters."""
    if not torch.cuda.is_available():
        return "no CUDA device: the allocator keeps no statistics on CPU"
    return torch.cuda.memory_summary()


class contiguous_tensors_handle:      # noqa: N801  (name of the reference's module-level helper namespace)
    """Views a list of same-dtype tensors as slices of one flat buffer (python/mindspore/hal/contiguous_tensors_handle.py):
    ``handle[i]`` is tensor i backed by the flat storage, ``handle.buffer`` the whole buffer, ``slice_by_tensor_index``
    / ``slice_by_padding_index`` give sub-ranges of it."""

    def __init__(self, tensor_list, enable_mem_align=True):
        if not tensor_list:
            raise ValueError("contiguous_tensors_handle needs at least one tensor")
        dt, dev = tensor_list[0].dtype, tensor_list[0].device
        if any(t.dtype != dt for t in tensor_list):
            raise TypeError("all tensors must have the same dtype")
        align = (512 // tensor_list[0].element_size()) if enable_mem_align else 1
        self.offsets, pos = [], 0
        for t in tensor_list:
            self.offsets.append((pos, pos + t.numel()))
            pos = (pos + t.numel() + align - 1) // align * align
        self.buffer = torch.zeros(pos, dtype=dt, device=dev)
        self.tensors = []
        for t, (a, b) in zip(tensor_list, self.offsets):
            view = self.buffer[a:b].view(t.shape)
            view.copy_(t.detach())
            self.tensors.append(view)

    def __getitem__(self, i):
        return self.tensors[i]

    def __len__(self):
        return len(self.tensors)

    def slice_by_tensor_index(self, start=None, end=None):
        start, end = start or 0, len(self.tensors) if end is None else end
        if not 0 <= start < end <= len(self.tensors):
            raise ValueError("invalid tensor index range [%s, %s)" % (start, end))
        return self.buffer[self.offsets[start][0]:self.offsets[end - 1][1]]

    def slice_by_padding_index(self, start=None, end=None):
        return self.buffer[start or 0:self.buffer.numel() if end is None else end]
