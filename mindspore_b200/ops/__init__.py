"""``mindspore_b200.ops``: primitive classes, the functional API and composite operators."""
from . import composite, functional, operations
from .composite import (GradOperation, HyperMap, Map, MultitypeFuncGraph, Partial, clip_by_global_norm,
                        clip_by_value, grad, jacfwd, jacrev, jvp, stop_gradient, value_and_grad, vjp)
from .functional import *  # noqa: F401,F403
from .operations import *  # noqa: F401,F403
from .primitive import (Primitive, PrimitiveWithCheck, PrimitiveWithInfer, constexpr, prim_attr_register)
from . import functional as F  # noqa: N812
from . import operations as P  # noqa: N812
from . import composite as C  # noqa: N812
from .composite import (Shard, UnpackCall, ZipOperation, choice_with_mask, count_nonzero, dot, gamma, laplace,  # noqa: E402,F401
                        poisson, repeat_elements, sequence_mask, tensor_dot, vmap)
