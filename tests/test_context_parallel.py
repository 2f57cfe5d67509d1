"""Ring attention and Ulysses (all-to-all) attention over gloo ranks against single-device attention."""
import pytest
import torch

from _mp import run_ranks


def _worker(rank, world, scheme, causal):
    import mindspore_b200 as ms
    from mindspore_b200.communication import GlobalComm, init
    from mindspore_b200.ops.attention import reference_attention
    from mindspore_b200.parallel import context_parallel as CP
    ms.set_context(device_target="CPU")
    init("mccl")
    B, S, H, D = 2, 16 * world, 4, 8
    g = torch.Generator().manual_seed(0)
    q, k, v, do = (torch.randn(B, S, H, D, generator=g) for _ in range(4))
    qf, kf, vf = (t.clone().requires_grad_(True) for t in (q, k, v))
    ref = reference_attention(qf, kf, vf, causal)
    ref.backward(do)
    sl = slice(rank * S // world, (rank + 1) * S // world)
    ql, kl, vl = (t[:, sl].clone().requires_grad_(True) for t in (q, k, v))
    fn = CP.ring_attention if scheme == "ring" else CP.ulysses_attention
    out = fn(ql, kl, vl, GlobalComm.WORLD_COMM_GROUP, causal=causal)
    out.backward(do[:, sl])
    errs = [float((out - ref[:, sl]).abs().max()), float((ql.grad - qf.grad[:, sl]).abs().max()),
            float((kl.grad - kf.grad[:, sl]).abs().max()), float((vl.grad - vf.grad[:, sl]).abs().max())]
    torch.distributed.barrier()
    return errs


@pytest.mark.parametrize("scheme,causal,world", [("ring", True, 2), ("ring", False, 3), ("ring", True, 4),
                                                  ("ulysses", True, 2), ("ulysses", False, 4)])
def test_context_parallel_attention(scheme, causal, world):
    for errs in run_ranks(_worker, world, scheme, causal):
        assert max(errs) < 1e-4, errs
