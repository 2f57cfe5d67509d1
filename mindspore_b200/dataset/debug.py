"""Hooks of the pipeline's debug mode: with ``config.set_debug_mode(True, [hooks])`` every ``map`` runs its
transforms one by one in the calling thread and calls each hook on the input of the first transform and on the output
of every transform.  A hook's ``compute`` is the place for a breakpoint.

Parity: mindspore/python/mindspore/dataset/debug/{debug_hook,pre_defined_hook}.py, the hook insertion in
dataset/engine/datasets.py (MapDataset.__insert_debug_wrapper).
"""
import collections.abc
from abc import ABC, abstractmethod

import numpy as np

__all__ = ["DebugHook", "PrintMetaDataHook", "PrintDataHook"]


class DebugHook(ABC):
    def __init__(self, prev_op_name=None):
        self.prev_op_name = prev_op_name
        self.is_first_op = None

    def __call__(self, *args):
        if self.prev_op_name:
            print("[Dataset debugger] Print the [%s] of the operation [%s]."
                  % ("INPUT" if self.is_first_op else "OUTPUT", self.prev_op_name), flush=True)
        self.compute(args)
        return args

    @abstractmethod
    def compute(self, *args):
        raise RuntimeError("compute() is not overridden in subclass of class DebugHook.")

    def set_previous_op_name(self, prev_op_name):
        self.prev_op_name = prev_op_name

    def set_is_first(self, is_first_op):
        self.is_first_op = is_first_op


def _is_image(col):
    return type(col).__module__.startswith("PIL.") and hasattr(col, "size")


class PrintMetaDataHook(DebugHook):
    """Prints dtype and shape (or type and size) of every column."""

    def compute(self, *args):
        for idx, col in enumerate(*args):
            msg = "Column %d. " % idx
            if isinstance(col, np.ndarray):
                msg += "The dtype is [%s]. The shape is [%s]." % (col.dtype, col.shape)
            elif _is_image(col):
                msg += "The type is [%s]. The shape is [%s]." % (type(col), col.size)
            elif isinstance(col, collections.abc.Sized):
                msg += "The type is [%s]. The size is [%s]." % (type(col), len(col))
            print(msg, flush=True)
        return args


class PrintDataHook(DebugHook):
    """Prints the data of every column."""

    def compute(self, *args):
        for idx, col in enumerate(*args):
            data = np.asarray(col) if _is_image(col) else col
            print("Column %d. The data is [%s]." % (idx, data), flush=True)
        return args
