"""``mindspore_b200.parallel``: layouts, shard strategies, SPMD execution, pipeline runtime, fused NVLink
collectives, checkpoint transformation."""
from .checkpoint_transform import (load_distributed_checkpoint, merge_pipeline_strategys, merge_sliced_parameter,
                                   rank_list_for_transform, sync_pipeline_shared_parameters,
                                   transform_checkpoint_by_rank, transform_checkpoints)
from .layout import Layout
from .shard import shard
from .strategy_ckpt import build_searched_strategy, restore_group_info_list
