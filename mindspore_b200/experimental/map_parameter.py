"""``MapParameter``: a parameter that is a key -> row table whose key set grows while training (embedding tables of
recommendation models; python/mindspore/experimental/map_parameter.py over the GPU hash table
plugin/device/gpu/hal/device/gpu_hash_table.cu).  Keys are integers, every value is a row of ``value_shape``; ``get``
on an unknown key inserts it with the default value.  The table lives in host memory here: rows are gathered into a
dense tensor for the step and written back with ``put`` / ``scatter_update``."""
from __future__ import annotations

import numpy as np
import torch

from ..common import dtype as mstype
from ..common.tensor import Tensor


class MapParameter:
    def __init__(self, key_dtype=mstype.int32, value_dtype=mstype.float32, value_shape=1, key_tensor=None,
                 value_tensor=None, default_value="normal", permit_filter_value=1, evict_filter_value=2 ** 63 - 1,
                 name=None, requires_grad=True, **kwargs):
        self.key_dtype, self.value_dtype = key_dtype, value_dtype
        self.value_shape = (int(value_shape),) if isinstance(value_shape, int) else tuple(int(v) for v in value_shape)
        self.default_value = default_value
        self.permit_filter_value, self.evict_filter_value = permit_filter_value, evict_filter_value
        self.name = name or "map_parameter"
        self.requires_grad = requires_grad
        self._rows = {}
        self._counts = {}
        self._gen = torch.Generator().manual_seed(0)
        if key_tensor is not None and value_tensor is not None:
            self.put(key_tensor, value_tensor)

    # ------------------------------------------------------------------ helpers
    def _default_row(self):
        dv = self.default_value
        if isinstance(dv, str):
            if dv == "zeros":
                return torch.zeros(self.value_shape, dtype=self.value_dtype)
            if dv == "ones":
                return torch.ones(self.value_shape, dtype=self.value_dtype)
            if dv == "normal":
                return (torch.randn(self.value_shape, generator=self._gen) * 0.01).to(self.value_dtype)
            raise ValueError("default_value must be 'normal', 'zeros', 'ones' or a number, got %r" % (dv,))
        return torch.full(self.value_shape, float(dv), dtype=self.value_dtype)

    @staticmethod
    def _keys(key_tensor):
        k = key_tensor.detach().cpu().reshape(-1) if isinstance(key_tensor, torch.Tensor) else \
            torch.as_tensor(np.asarray(key_tensor)).reshape(-1)
        return [int(x) for x in k.tolist()]

    # ------------------------------------------------------------------ table operations
    def get(self, key_tensor, insert_default_value=True):
        """Rows of the given keys, [len(keys), *value_shape]; unknown keys are inserted with the default value (or
        returned as zeros without insertion when ``insert_default_value`` is False).  A key is only admitted after
        ``permit_filter_value`` lookups."""
        rows = []
        for k in self._keys(key_tensor):
            row = self._rows.get(k)
            if row is None:
                self._counts[k] = self._counts.get(k, 0) + 1
                if insert_default_value and self._counts[k] >= self.permit_filter_value:
                    row = self._default_row()
                    self._rows[k] = row
                else:
                    row = torch.zeros(self.value_shape, dtype=self.value_dtype)
            rows.append(row)
        out = torch.stack(rows) if rows else torch.zeros((0,) + self.value_shape, dtype=self.value_dtype)
        return Tensor(out)

    def __getitem__(self, key_tensor):
        return self.get(key_tensor, True)

    def put(self, key_tensor, value_tensor):
        vals = value_tensor.detach().cpu().to(self.value_dtype).reshape((-1,) + self.value_shape)
        keys = self._keys(key_tensor)
        if len(keys) != vals.shape[0]:
            raise ValueError("put: %d keys but %d rows" % (len(keys), vals.shape[0]))
        for k, v in zip(keys, vals):
            self._rows[k] = v.clone()
        return self

    def __setitem__(self, key_tensor, value_tensor):
        self.put(key_tensor, value_tensor)

    def erase(self, key_tensor):
        for k in self._keys(key_tensor):
            self._rows.pop(k, None)
            self._counts.pop(k, None)
        return self

    def scatter_update(self, key_tensor, delta, lr=1.0):
        """rows[key] -= lr * delta[i] for every i (duplicate keys accumulate): the sparse optimizer step."""
        d = delta.detach().cpu().to(self.value_dtype).reshape((-1,) + self.value_shape)
        for k, g in zip(self._keys(key_tensor), d):
            if k in self._rows:
                self._rows[k] = self._rows[k] - lr * g
        return self

    # ------------------------------------------------------------------ whole-table access
    def get_keys(self):
        return Tensor(torch.tensor(sorted(self._rows), dtype=self.key_dtype))

    def get_values(self):
        keys = sorted(self._rows)
        if not keys:
            return Tensor(torch.zeros((0,) + self.value_shape, dtype=self.value_dtype))
        return Tensor(torch.stack([self._rows[k] for k in keys]))

    def get_data(self):
        return self.get_keys(), self.get_values()

    def export_data(self, incremental=False):
        """(keys, values, statuses) as numpy arrays, the triple a checkpoint stores for a map parameter."""
        keys, values = self.get_data()
        status = np.zeros(len(self._rows), dtype=np.int32)
        return keys.numpy(), values.numpy(), status

    def import_data(self, data):
        keys, values = data[0], data[1]
        self._rows.clear()
        self.put(torch.as_tensor(np.asarray(keys)), torch.as_tensor(np.asarray(values)))
        return self

    def __len__(self):
        return len(self._rows)

    def __repr__(self):
        return "MapParameter(name=%s, size=%d, value_shape=%s)" % (self.name, len(self._rows), self.value_shape)
