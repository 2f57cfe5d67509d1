"""``mindspore_b200.dataset``: input pipelines (sources, ``map`` / ``batch`` / ``shuffle`` / ``repeat`` / ``shard``
/ ``take`` / ``skip`` / ``zip``, iterators) and record files."""
from .engine import (Dataset, GeneratorDataset, MindDataset, NumpySlicesDataset, RandomDataset, config, zip)  # noqa: A004
from .mindrecord import FileReader, FileWriter
from .native_loader import NativeBatchLoader
from . import audio, text, transforms, vision
from . import samplers  # noqa: E402
from .samplers import *  # noqa: E402,F401,F403
from .sources import *  # noqa: E402,F401,F403
from .sources_ext import *  # noqa: E402,F401,F403
