"""Parallel checkpoint helpers: gathering sliced parameters for an integrated save.
Parity: mindspore/python/mindspore/train/serialization.py:656-706,1703-1763 (_get_merged_param_data,
AllGatherCell path)."""
import torch

from ..communication import comm_func as CF
from ..communication import management as M


def gather_full_parameters(net):
    """[(name, full tensor)] - parameters that carry a layout are all-gathered back to their full shape."""
    out = []
    for p in net.get_parameters():
        lay = p.param_layout
        if lay is None or not p.sliced or not M.GlobalComm.INITED or M.is_simulation():
            out.append((p.name, p))
            continue
        world = M._group(None)
        gathered = CF._all_gather(p.detach().as_subclass(torch.Tensor).unsqueeze(0).contiguous(), world)
        import numpy as np
        from .layout import assemble_full
        slices = {r: gathered[r].float().cpu().numpy() for r in range(world.size)}
        if lay.opt_shard_size and lay.opt_shard_size > 1:
            from .checkpoint_transform import merge_opt_shard_slices
            full = merge_opt_shard_slices(slices, lay)
        else:
            full = assemble_full(slices, lay)
        out.append((p.name, torch.from_numpy(np.ascontiguousarray(full)).to(p.dtype)))
    return out
