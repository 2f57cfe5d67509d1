from . import amp, callback, metrics
from .callback import (BackupAndRestore, Callback, CheckpointConfig, ClusterMonitor, EarlyStopping,
                       FlopsUtilizationCollector, History, LambdaCallback, LearningRateScheduler, LossMonitor,
                       ModelCheckpoint, OnRequestExit, ReduceLROnPlateau, RunContext, SummaryCollector, TimeMonitor)
from .dataset_helper import DatasetHelper, connect_network_with_dataset
from .loss_scale_manager import DynamicLossScaleManager, FixedLossScaleManager, LossScaleManager
from .model import Model
from .serialization import (async_ckpt_thread_status, export, load, load_checkpoint, load_param_into_net,
                            load_segmented_checkpoints, save_checkpoint)
