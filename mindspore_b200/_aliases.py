"""The reference's import paths that live elsewhere in this package.

``import mindspore_b200.amp`` (or ``from mindspore_b200.nn.learning_rate_schedule import CosineDecayLR``, ...)
resolves to the module named in the table below; nothing is copied, the alias IS that module.  The finder sits at
the end of ``sys.meta_path``, so real files always win."""
from __future__ import annotations

import importlib
import importlib.abc
import importlib.machinery
import sys

_PKG = "mindspore_b200"

ALIASES = {
    "amp": "train.amp",
    "log": "utils.log",
    "mindrecord": "dataset.mindrecord",
    "run_check": "common.api",
    "common.lazy_inline": "common.api",
    "common.recompute": "common.api",
    "common.mutable": "common.api",
    "common.generator": "common.api",
    "common.symbol": "common.api",
    "common.hook_handle": "nn.cell",
    "common.dump": "utils.dump",
    "common.jit_context": "graph.jit",
    "nn.learning_rate_schedule": "nn.lr_schedule",
    "nn.dynamic_lr": "nn.lr_schedule",
    "nn.wrap.cell_wrapper": "nn.wrap",
    "nn.wrap.grad_reducer": "nn.wrap",
    "nn.wrap.loss_scale": "nn.wrap",
    "ops.function": "ops.functional",
    "ops.operations.comm_ops": "ops.comm_ops",
    "ops._grad_experimental": "graph.autodiff",
    "parallel.algo_parameter_config": "common.api",
    "parallel._cost_model_context": "parallel.cost_model",
    "parallel.parameter_broadcast": "parallel",
    "parallel.cluster": "msrun",
    "parallel.cluster.run": "msrun",
    "parallel._recovery_context": "parallel.recovery",
    "parallel._ps_context": "context",
    "parallel._offload_context": "context",
    "parallel._auto_parallel_context": "context",
    "parallel._dp_allreduce_fusion": "parallel.comm_fusion",
    "parallel._cell_wrapper": "parallel.checkpoint",
    "parallel._utils": "parallel.layout",
    "parallel._tensor": "parallel.layout",
    "parallel._parallel_serialization": "parallel.strategy_ckpt",
    "parallel.nn": "parallel.transformer",
    "train.train_thor": "train.thor_convert",
    "train.summary.summary_record": "train.summary",
    "train.anf_ir_pb2": "graph.mindir_proto",
    "train.mind_ir_pb2": "graph.mindir_proto",
    "communication.comm_func": "communication",
    "communication._comm_helper": "communication.management",
    "profiler.profiling": "profiler",
    "dataset.engine.datasets": "dataset.engine",
    "_extends.parse": "graph.ast_transform",
    "offline_debug": "utils.offline_debug",
    "offline_debug.dbg_services": "utils.offline_debug",
    "nn.metrics": "train.metrics",
    "nn.optim.optimizer": "nn.optim",
    "nn.optim.adasum": "nn.optim_ext",
    "nn.extend.basic": "nn.extend",
    "nn.extend.pooling": "nn.extend",
    "nn.extend.embedding": "nn.extend",
    "nn.extend.layer": "nn.extend",
    "nn.extend.layer.normalization": "nn.extend",
    "nn.sparse": "nn",
    "nn.grad": "nn",
    "nn.reinforcement": "nn.layer_ext",
    "nn.probability.bnn_layers.layer_distribution": "nn.probability.bnn_layers",
    "nn.probability.bnn_layers.bnn_cell_wrapper": "nn.probability.bnn_layers",
    "nn.probability.bnn_layers.dense_variational": "nn.probability.bnn_layers",
    "nn.probability.bnn_layers.conv_variational": "nn.probability.bnn_layers",
    "ops.extend": "ops",
    "ops.extend.array_func": "ops",
    "ops.extend.nn_func": "ops",
    "ops.extend.math_func": "ops",
    "common.sparse_tensor": "common.api",
    "experimental.optim.optimizer": "experimental.optim",
    "train.train_thor.convert_utils": "train.thor_convert",
    "train.train_thor.model_thor": "train.thor_convert",
    "dataset.callback": "dataset.sources_ext",
    "dataset.core": "dataset.core_config",
    "dataset.core.config": "dataset.core_config",
}
for _sub in ("math", "image", "container", "rnns", "basic", "pooling", "timedistributed", "dense", "conv", "combined",
             "activation", "normalization", "thor_layer", "rnn_cells", "transformer", "embedding", "padding",
             "channel_shuffle", "flatten"):
    ALIASES["nn.layer." + _sub] = "nn"
for _sub in ("shardreader", "shardheader", "filereader", "shardsegment", "config", "filewriter", "shardindexgenerator",
             "mindpage", "shardwriter", "shardutils", "tools", "tools.mnist_to_mr", "tools.tfrecord_to_mr",
             "tools.cifar10_to_mr", "tools.cifar100_to_mr", "tools.cifar10", "tools.cifar100", "tools.csv_to_mr",
             "tools.imagenet_to_mr"):
    ALIASES["mindrecord." + _sub] = "dataset.mindrecord"
for _sub in ("boost", "boost_cell_wrapper", "base", "grad_freeze", "group_loss_scale_manager", "grad_accumulation",
             "adasum", "dim_reduce", "less_batch_normalization"):
    ALIASES["boost." + _sub] = "boost"


class _AliasFinder(importlib.abc.MetaPathFinder, importlib.abc.Loader):
    def find_spec(self, fullname, path=None, target=None):
        if not fullname.startswith(_PKG + "."):
            return None
        rel = fullname[len(_PKG) + 1:]
        real = ALIASES.get(rel)
        if real is None or real == rel:
            return None
        return importlib.machinery.ModuleSpec(fullname, self, is_package=False)

    def create_module(self, spec):
        real = importlib.import_module(_PKG + "." + ALIASES[spec.name[len(_PKG) + 1:]])
        self._saved = getattr(real, "__spec__", None)
        return real

    def exec_module(self, module):
        alias = module.__spec__.name[len(_PKG) + 1:] if module.__spec__ is not None else ""
        if getattr(self, "_saved", None) is not None:
            module.__spec__ = self._saved          # the import machinery pointed it at the alias: put it back
        if not hasattr(module, "__path__") and any(k.startswith(alias + ".") for k in ALIASES):
            module.__path__ = []                   # so that aliases below this one can be imported through it


def install():
    if not any(isinstance(f, _AliasFinder) for f in sys.meta_path):
        sys.meta_path.append(_AliasFinder())
    # real single-file modules that the reference has as packages: give them an (empty) search path so that the
    # aliases below them are looked up at all
    for key in ALIASES:
        parent = key.rsplit(".", 1)[0] if "." in key else None
        if parent and parent not in ALIASES:
            try:
                mod = importlib.import_module(_PKG + "." + parent)
            except ImportError:
                continue
            if not hasattr(mod, "__path__"):
                mod.__path__ = []


def lazy_attribute(name):
    """Package-level ``__getattr__``: ``mindspore_b200.amp`` without an import statement."""
    if name in ALIASES and "." not in name:
        return importlib.import_module(_PKG + "." + name)
    raise AttributeError("module %r has no attribute %r" % (_PKG, name))
