"""mindspore_b200: a Blackwell-native deep-learning framework with MindSpore's training API.

PyTorch is the tensor / eager substrate; hot ops are hand-written sm_100a kernels
(``mindspore_b200/csrc/cuda``), the planner / runtime pieces are C++ (``mindspore_b200/csrc/host``).
"""
from . import common, communication, context, dataset, nn, ops, parallel, train
from .common import Parameter, ParameterTuple, Tensor, dtype, get_seed, set_seed
from .common.initializer import initializer  # noqa: F401
from .common.dtype import *  # noqa: F401,F403
from .common.dtype import Type, dtype_to_nptype, pytype_to_dtype
from .context import (GRAPH_MODE, PYNATIVE_MODE, ParallelMode, get_auto_parallel_context, get_context,
                      reset_auto_parallel_context, set_auto_parallel_context, set_context, set_offload_context,
                      set_ps_context)
from .graph.jit import jit, ms_function
from .ops.composite import grad, jacfwd, jacrev, jvp, value_and_grad, vjp
from .parallel.layout import Layout
from .parallel.shard import shard
from .train import Model
from .train.callback import (Callback, CheckpointConfig, LossMonitor, ModelCheckpoint, TimeMonitor)
from .train.serialization import (export, load, load_checkpoint, load_param_into_net, save_checkpoint)
from . import train as _train
from .train import amp
from .parallel import (build_searched_strategy, load_distributed_checkpoint, merge_pipeline_strategys,
                       merge_sliced_parameter, rank_list_for_transform, restore_group_info_list,
                       sync_pipeline_shared_parameters, transform_checkpoint_by_rank, transform_checkpoints)
from .train.serialization import async_ckpt_thread_status, load_segmented_checkpoints

from .profiler import EnvProfiler, Profiler

from .utils.dump import set_dump
from .train.summary import SummaryRecord
from . import hal, mint

from .common.api import *  # noqa: E402,F401,F403
from .ops.primitive import constexpr  # noqa: E402
from . import boost, experimental, rewrite, scipy  # noqa: E402
from . import numpy  # noqa: E402
from .dataset import mindrecord  # noqa: E402
import multiprocessing  # noqa: E402  (the reference re-exports a fork-safe wrapper of the same module)
from .graph.mindir import load_mindir  # noqa: E402

from .common.dtype import QuantDtype  # noqa: E402
from .common.jit_config import JitConfig  # noqa: E402
from .common.api import jit_class as ms_class  # noqa: E402
from .graph.flops import flops_collection  # noqa: E402
from .dataset.mindrecord import *  # noqa: E402,F401,F403
from .train.dataset_helper import DatasetHelper, connect_network_with_dataset  # noqa: E402
from .train.amp import build_train_network  # noqa: E402
from .train.loss_scale_manager import (DynamicLossScaleManager, FixedLossScaleManager,  # noqa: E402
                                       LossScaleManager)
from .train.serialization import (check_checkpoint, ckpt_to_safetensors, convert_model,  # noqa: E402
                                  export_split_mindir, get_ckpt_path_with_strategy, load_checkpoint_async,
                                  parse_print, safetensors_to_ckpt, save_mindir)
from .train.callback import *  # noqa: E402,F401,F403
from .utils.log import get_level, get_log_config  # noqa: E402
from .ops import reshard  # noqa: E402
from .rewrite import Node, NodeType, ScopedValue, SymbolTree  # noqa: E402
from .safeguard import load_obf_params_into_net, obfuscate_ckpt, obfuscate_model  # noqa: E402
from .context import get_ps_context, reset_ps_context, set_ps_context, set_offload_context  # noqa: E402
from .nn.cell import GraphCell  # noqa: E402
from . import _aliases  # noqa: E402

_aliases.install()


def __getattr__(name):
    return _aliases.lazy_attribute(name)


mstype = dtype
__version__ = "0.1.0"
