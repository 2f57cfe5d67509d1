"""Ring attention and Ulysses (all-to-all) attention against single-device attention: over gloo ranks on CPU, and on
2 / 4 GPUs (NCCL point-to-point / all-to-all, per-block work on the tcgen05 FlashAttention kernels)."""
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


def _zigzag_worker(rank, world):
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
    ref = reference_attention(qf, kf, vf, True)
    ref.backward(do)
    ql, kl, vl = (CP.zigzag_split(t, world, rank).clone().requires_grad_(True) for t in (q, k, v))
    out = CP.ring_attention(ql, kl, vl, GlobalComm.WORLD_COMM_GROUP, causal=True, load_balance=True)
    out.backward(CP.zigzag_split(do, world, rank))
    pick = lambda t: CP.zigzag_split(t, world, rank)
    errs = [float((out - pick(ref)).abs().max()), float((ql.grad - pick(qf.grad)).abs().max()),
            float((kl.grad - pick(kf.grad)).abs().max()), float((vl.grad - pick(vf.grad)).abs().max())]
    torch.distributed.barrier()
    return errs, out.detach().numpy()


@pytest.mark.parametrize("world", [2, 3, 4])
def test_load_balanced_ring_attention(world):
    """Zigzag layout: every rank does the same work per ring step and the result equals single-device causal
    attention; zigzag_merge puts the pieces back in sequence order."""
    from mindspore_b200.ops.attention import reference_attention
    from mindspore_b200.parallel import context_parallel as CP
    res = run_ranks(_zigzag_worker, world)
    for errs, _ in res:
        assert max(errs) < 1e-4, errs
    B, S, H, D = 2, 16 * world, 4, 8
    g = torch.Generator().manual_seed(0)
    q, k, v = (torch.randn(B, S, H, D, generator=g) for _ in range(3))
    full = CP.zigzag_merge([torch.from_numpy(o) for _, o in res])
    assert float((full - reference_attention(q, k, v, True)).abs().max()) < 1e-4


@pytest.mark.parametrize("scheme,causal,world", [("ring", True, 2), ("ring", False, 3), ("ring", True, 4),
                                                  ("ulysses", True, 2), ("ulysses", False, 4)])
def test_context_parallel_attention(scheme, causal, world):
    for errs in run_ranks(_worker, world, scheme, causal):
        assert max(errs) < 1e-4, errs


def _gpu_worker(rank, world, scheme, causal):
    import mindspore_b200 as ms
    from mindspore_b200 import _native
    from mindspore_b200.communication import GlobalComm, init
    from mindspore_b200.ops.attention import reference_attention
    from mindspore_b200.parallel import context_parallel as CP
    torch.cuda.set_device(rank)
    ms.set_context(device_target="GPU", device_id=rank)
    init("nccl")
    B, S, H, D = 1, 256 * world, 4, 128
    g = torch.Generator().manual_seed(0)
    q, k, v, do = (torch.randn(B, S, H, D, generator=g).cuda().bfloat16() for _ in range(4))
    qf, kf, vf = (t.float().clone().requires_grad_(True) for t in (q, k, v))
    ref = reference_attention(qf, kf, vf, causal)
    ref.backward(do.float())
    sl = slice(rank * S // world, (rank + 1) * S // world)
    ql, kl, vl = (t[:, sl].clone().requires_grad_(True) for t in (q, k, v))
    if scheme == "zigzag":
        pick = lambda t: CP.zigzag_split(t, world, rank).contiguous()
        ql, kl, vl = (pick(t).clone().requires_grad_(True) for t in (q, k, v))
        out = CP.ring_attention(ql, kl, vl, GlobalComm.WORLD_COMM_GROUP, causal=True, load_balance=True)
        out.backward(pick(do))
        torch.cuda.synchronize()
        rel = lambda a, b: float((a.float() - b.float()).abs().max() / (b.float().abs().max() + 1e-6))
        errs = [rel(out, pick(ref)), rel(ql.grad, pick(qf.grad)), rel(kl.grad, pick(kf.grad)),
                rel(vl.grad, pick(vf.grad))]
        status = _native.device_status()
        torch.distributed.barrier()
        return errs, status
    fn = CP.ring_attention if scheme == "ring" else CP.ulysses_attention
    out = fn(ql, kl, vl, GlobalComm.WORLD_COMM_GROUP, causal=causal)
    out.backward(do[:, sl].contiguous())
    torch.cuda.synchronize()

    def rel(a, b):
        return float((a.float() - b.float()).abs().max() / (b.float().abs().max() + 1e-6))
    errs = [rel(out, ref[:, sl]), rel(ql.grad, qf.grad[:, sl]), rel(kl.grad, kf.grad[:, sl]),
            rel(vl.grad, vf.grad[:, sl])]
    status = _native.device_status()
    torch.distributed.barrier()
    return errs, status


@pytest.mark.gpu
@pytest.mark.parametrize("scheme,causal,world", [("ring", True, 2), ("ulysses", True, 2), ("zigzag", True, 2),
                                                  ("ring", True, 4), ("ulysses", False, 4), ("zigzag", True, 4)])
def test_context_parallel_attention_gpu(scheme, causal, world):
    if torch.cuda.device_count() < world:
        pytest.skip("needs %d GPUs" % world)
    for errs, status in run_ranks(_gpu_worker, world, scheme, causal):
        assert status == 0
        assert max(errs) < 4e-2, errs
