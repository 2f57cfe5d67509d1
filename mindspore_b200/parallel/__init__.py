"""``mindspore_b200.parallel``: layouts, shard strategies, SPMD execution, pipeline runtime, fused NVLink
collectives, checkpoint transformation."""
from .checkpoint_transform import (load_distributed_checkpoint, merge_pipeline_strategys, merge_sliced_parameter,
                                   rank_list_for_transform, sync_pipeline_shared_parameters,
                                   transform_checkpoint_by_rank, transform_checkpoints)
from .layout import Layout
from .shard import shard
from .strategy_ckpt import build_searched_strategy, restore_group_info_list
from ..common.api import get_algo_parameters, reset_algo_parameters, set_algo_parameters  # noqa: E402,F401


def load_segmented_checkpoints(*args, **kwargs):
    from ..train.serialization import load_segmented_checkpoints as _f
    return _f(*args, **kwargs)


def parameter_broadcast(net, layout=None, cur_rank=0, initial_rank=0):
    """Broadcasts every parameter of ``net`` from the first rank of its replica group, so that ranks holding the same
    slice start from identical values (parallel/parameter_broadcast.py).  Without ``layout`` all ranks form one group
    rooted at ``initial_rank``."""
    from ..communication import comm_func as _cf
    from ..communication import management as _m
    if not _m.GlobalComm.INITED or _m.get_group_size() == 1:
        return
    import torch
    for p in net.get_parameters():
        t = p.detach().as_subclass(torch.Tensor)
        _cf.broadcast(t, initial_rank)
        with torch.no_grad():
            p.copy_(t)
