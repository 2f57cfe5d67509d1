"""Collective communication: bootstrap, groups and functional collectives."""
from . import comm_func
from .management import (HCCL_WORLD_COMM_GROUP, MCCL_WORLD_COMM_GROUP, NCCL_WORLD_COMM_GROUP, GlobalComm,
                         create_group, destroy_group, get_group_rank_from_world_rank, get_group_size,
                         get_local_rank, get_local_rank_size, get_process_group_ranks, get_rank,
                         get_world_rank_from_group_rank, init, release)
from .comm_func import (P2POp, all_gather_into_tensor, all_reduce, all_to_all_single_with_output_shape,  # noqa: E402
                        all_to_all_with_output_shape, barrier, batch_isend_irecv, broadcast, gather_into_tensor,
                        irecv, isend, reduce, reduce_scatter_tensor, scatter_tensor)
