"""``mindspore_b200.nn``: Cell, layers, losses, optimizers, LR schedules and training wrappers."""
from . import lr_schedule, optim, wrap
from .cell import Cell, GraphCell
from .layer import *  # noqa: F401,F403
from .layer import get_activation
from .layer_ext import *  # noqa: F401,F403
from .optim_ext import *  # noqa: F401,F403
from .loss import *  # noqa: F401,F403
from .lr_schedule import (CosineDecayLR, ExponentialDecayLR, InverseDecayLR, LearningRateSchedule, NaturalExpDecayLR,
                          PolynomialDecayLR, WarmUpLR, cosine_decay_lr, exponential_decay_lr, inverse_decay_lr,
                          natural_exp_decay_lr, piecewise_constant_lr, polynomial_decay_lr, warmup_lr)
from .optim import (ASGD, FTRL, LARS, SGD, AdaFactor, Adadelta, Adagrad, Adam, AdaMax, AdamW, AdamWeightDecay, Lamb,
                    Momentum, Optimizer, ParamArena, ProximalAdagrad, RMSProp, Rprop, thor)
from .wrap import (DistributedGradReducer, DynamicLossScaleUpdateCell, FixedLossScaleUpdateCell, ForwardValueAndGrad,
                   GetNextSingleOp, GradAccumulationCell, MicroBatchInterleaved, PipelineCell, PipelineGradReducer,
                   TimeDistributed, ParameterUpdate, TrainOneStepCell, TrainOneStepWithLossScaleCell,
                   VirtualDatasetCellTriple, WithEvalCell, WithGradCell, WithLossCell)
from . import probability  # noqa: E402,F401
