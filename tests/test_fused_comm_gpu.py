"""Fused compute + collective kernels over NVLink at 2, 4 and 8 ranks against GEMM + NCCL on the same data:
MatMul -> ReduceScatter (push epilogue), AllGather -> MatMul (copy-engine gather and in-kernel gather), the bucket
all-reduce and six back-to-back calls (the two-buffer rotation of the symmetric staging).  Row counts per rank
include odd multiples of the 128-row tile.  Every case ends with the device status word at zero (no bounded wait
ran out)."""
import pytest
import torch

from _mp import run_ranks

pytestmark = pytest.mark.gpu


def _worker(rank, world, ag_dma):
    import mindspore_b200 as ms
    from mindspore_b200 import _native
    from mindspore_b200.communication import comm_func as CF
    from mindspore_b200.communication import init
    from mindspore_b200.communication import management as M
    from mindspore_b200.parallel import fused_comm as FC
    from mindspore_b200.parallel import tp as TP
    torch.cuda.set_device(rank)
    ms.set_context(device_target="GPU", device_id=rank)
    init("nccl")
    FC._AG_DMA = int(ag_dma)
    g = M._group(None)
    tp = TP.TPGroup()
    assert FC.get_context(g) is not None, "symmetric memory is not available"
    torch.manual_seed(100 + rank)
    worst = {}

    def rel(a, b):
        return float((a.float() - b.float()).abs().max() / (b.float().abs().max() + 1e-6))

    # rows per rank: 128 (one tile), 384 (odd multiple), 512
    for rows, Kd, N in ((128, 512, 768), (384, 1024, 1536), (512, 4096, 512)):
        T = rows * world
        # row-parallel: x [T, K/mp] @ w[N, K/mp]^T -> reduce-scatter rows
        xs = torch.randn(T, Kd, device="cuda").bfloat16().requires_grad_(True)
        w = (torch.randn(N, Kd, device="cuda") * 0.05).bfloat16().requires_grad_(True)
        y = FC.matmul_reduce_scatter(xs, w, tp)
        dyv = torch.randn_like(y)
        y.backward(dyv)
        xr = xs.detach().clone().requires_grad_(True)
        wr = w.detach().clone().requires_grad_(True)
        yr = TP.scatter_tokens_reduce(torch.nn.functional.linear(xr, wr), tp)
        yr.backward(dyv)
        torch.cuda.synchronize()
        key = "rs_%d" % rows
        worst[key] = max(rel(y, yr), rel(xs.grad, xr.grad), rel(w.grad, wr.grad))
        # column-parallel: gather(x_shard [T/mp, K]) @ w[N, K]^T
        xs = torch.randn(rows, Kd, device="cuda").bfloat16().requires_grad_(True)
        w = (torch.randn(N, Kd, device="cuda") * 0.05).bfloat16().requires_grad_(True)
        y = FC.allgather_matmul(xs, w, tp)
        dyv = torch.randn_like(y)
        y.backward(dyv)
        xr = xs.detach().clone().requires_grad_(True)
        wr = w.detach().clone().requires_grad_(True)
        yr = torch.nn.functional.linear(TP.gather_tokens(xr, tp), wr)
        yr.backward(dyv)
        torch.cuda.synchronize()
        worst["ag_%d" % rows] = max(rel(y, yr), rel(xs.grad, xr.grad), rel(w.grad, wr.grad))
    # six calls in a row without host synchronisation: staging buffers rotate, results must not mix
    rows, Kd, N = 256, 512, 1024
    xs = [torch.randn(rows, Kd, device="cuda").bfloat16() for _ in range(6)]
    w = (torch.randn(N, Kd, device="cuda") * 0.05).bfloat16()
    with torch.no_grad():
        outs = [FC.allgather_matmul(x, w, tp) for x in xs]
        outs_rs = [FC.matmul_reduce_scatter(o[:, :Kd].contiguous(), w, tp) for o in outs]
        refs = [torch.nn.functional.linear(CF._all_gather(x, g), w) for x in xs]
        refs_rs = [CF._reduce_scatter(torch.nn.functional.linear(r[:, :Kd].contiguous(), w), "sum", g) for r in refs]
    torch.cuda.synchronize()
    worst["rotation"] = max(max(rel(a, b) for a, b in zip(outs, refs)), max(rel(a, b) for a, b in zip(outs_rs, refs_rs)))
    # bucket all-reduce (odd length)
    x = torch.randn(3_000_001, device="cuda")
    ref = x.clone()
    torch.distributed.all_reduce(ref)
    FC.all_reduce_(x, g, 0.5)
    torch.cuda.synchronize()
    worst["allreduce"] = rel(x, ref * 0.5)
    status = _native.device_status()
    torch.distributed.barrier()
    M.release()
    return worst, status


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("ag_dma", [1, 0])
def test_fused_collective_gemms_match_gemm_plus_nccl(world, ag_dma):
    if torch.cuda.device_count() < world:
        pytest.skip("needs %d GPUs" % world)
    for worst, status in run_ranks(_worker, world, ag_dma, timeout=420):
        assert status == 0, (status, worst)
        for k, v in worst.items():
            assert v < (1e-5 if k == "allreduce" else 3e-2), (k, v, worst)
