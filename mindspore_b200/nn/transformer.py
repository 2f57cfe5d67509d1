"""``mindspore.nn.transformer`` (the earlier home of the transformer building blocks)."""
from ..parallel._transformer import *          # noqa: F401,F403
from ..parallel._transformer import __all__    # noqa: F401
