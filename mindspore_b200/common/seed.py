"""Global / per-op random seeds.  Parity: mindspore/python/mindspore/common/seed.py (set_seed, get_seed)."""
import random

import numpy as np
import torch

_GLOBAL_SEED = None


def set_seed(seed):
    global _GLOBAL_SEED
    if not isinstance(seed, int) or seed < 0:
        raise ValueError("The argument 'seed' must be a non-negative int, but got %r" % (seed,))
    _GLOBAL_SEED = seed
    random.seed(seed)
    np.random.seed(seed % (2 ** 32))
    torch.manual_seed(seed)


def get_seed():
    return _GLOBAL_SEED


def get_rng_state():
    """State saved under the ``random_op`` tag of a checkpoint (serialization.py:312-321)."""
    return torch.get_rng_state()


def set_rng_state(state):
    torch.set_rng_state(state)
