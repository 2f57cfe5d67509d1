"""``mindspore_b200.dataset``: input pipelines (sources, ``map`` / ``batch`` / ``shuffle`` / ``repeat`` / ``shard``
/ ``take`` / ``skip`` / ``zip``, iterators) and record files."""
from .engine import (Dataset, DictIterator, DummyIterator, GeneratorDataset, Iterator, MindDataset,  # noqa: A004
                     NumpySlicesDataset, RandomDataset, TupleIterator, check_iterator_cleanup, config, zip)
from .mindrecord import FileReader, FileWriter
from .native_loader import NativeBatchLoader
from . import audio, text, transforms, vision
from . import samplers  # noqa: E402
from .samplers import *  # noqa: E402,F401,F403
from .sources import *  # noqa: E402,F401,F403
from .sources_ext import *  # noqa: E402,F401,F403
