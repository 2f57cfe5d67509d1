from . import dtype
from .dtype import *  # noqa: F401,F403
from .initializer import initializer
from .parameter import Parameter, ParameterTuple
from .seed import get_seed, set_seed
from .tensor import Tensor, as_tensor
from . import tensor_ext  # noqa: E402,F401  (attaches the MindSpore-only Tensor methods)
