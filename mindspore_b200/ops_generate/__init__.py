"""Operator definitions in yaml and the generator that turns them into ``Primitive`` classes and functional wrappers
(python/mindspore/ops_generate/gen_ops.py with ops/ops_def/*.yaml in the reference, which also emits C++ op
definitions and pyboost glue; here the only target is Python, since primitives dispatch to torch / CUDA kernels
directly)."""
from .gen_ops import generate, load_definitions, main  # noqa: F401
