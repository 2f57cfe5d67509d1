"""Collective communication: bootstrap, groups and functional collectives."""
from . import comm_func
from .management import (HCCL_WORLD_COMM_GROUP, MCCL_WORLD_COMM_GROUP, NCCL_WORLD_COMM_GROUP, GlobalComm,
                         create_group, destroy_group, get_group_rank_from_world_rank, get_group_size,
                         get_local_rank, get_local_rank_size, get_process_group_ranks, get_rank,
                         get_world_rank_from_group_rank, init, release)
