from . import amp, callback, metrics
from .callback import (BackupAndRestore, Callback, CheckpointConfig, ClusterMonitor, EarlyStopping,
                       FlopsUtilizationCollector, History, LambdaCallback, LearningRateScheduler, LossMonitor,
                       ModelCheckpoint, OnRequestExit, ReduceLROnPlateau, RunContext, SummaryCollector, TimeMonitor)
from .dataset_helper import DatasetHelper, connect_network_with_dataset
from .loss_scale_manager import DynamicLossScaleManager, FixedLossScaleManager, LossScaleManager
from .model import Model
from .serialization import (async_ckpt_thread_status, export, export_split_mindir, load, load_checkpoint,
                            load_checkpoint_async, load_param_into_net, load_segmented_checkpoints, parse_print,
                            save_checkpoint)
from .amp import build_train_network
from .safetensors_io import (check_checkpoint, ckpt_to_safetensors, get_ckpt_path_with_strategy,  # noqa: E402,F401
                             load_safetensors, safetensors_to_ckpt, save_safetensors)
from .metrics import Metric  # noqa: E402,F401


def __getattr__(name):
    # functions that live in `parallel` are also reachable as `train.<name>`, as in the reference
    if name in ("build_searched_strategy", "merge_sliced_parameter", "load_distributed_checkpoint",
                "restore_group_info_list", "merge_pipeline_strategys", "rank_list_for_transform",
                "transform_checkpoint_by_rank", "transform_checkpoints", "sync_pipeline_shared_parameters"):
        from .. import parallel
        return getattr(parallel, name)
    if name in ("ConvertNetUtils", "ConvertModelUtils", "ModelThor"):
        from . import thor_convert
        return getattr(thor_convert, name)
    if name == "data_sink":
        from ..common.api import data_sink
        return data_sink
    if name in ("convert_model", "obfuscate_model"):
        def unavailable(*a, **k):
            raise NotImplementedError("%s targets other runtimes (ONNX conversion / model obfuscation) and is not "
                                      "provided" % name)
        return unavailable
    if name in ("ConvertModelUtils", "ConvertNetUtils"):
        from ..nn.optim_ext import ConvertModelUtils, ConvertNetUtils
        return {"ConvertModelUtils": ConvertModelUtils, "ConvertNetUtils": ConvertNetUtils}[name]
    raise AttributeError("module 'train' has no attribute %r" % name)
