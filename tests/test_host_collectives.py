"""Native TCP ring collectives (csrc/host/host_collectives.cpp) on 3 and 4 CPU ranks against locally computed
expectations; a rank that never joins is reported as a timeout, not a hang."""
import numpy as np
import pytest
import torch

from _mp import run_ranks


def _worker(rank, world):
    from mindspore_b200.communication.host_collectives import HostCommunicator
    comm = HostCommunicator.from_env(timeout=30.0)
    out = {}
    g = torch.Generator().manual_seed(7)
    base = [torch.randn(1003, generator=g) for _ in range(world)]          # odd length: uneven chunks
    t = base[rank].clone()
    comm.all_reduce(t)
    out["ar"] = float((t - sum(base)).abs().max())
    m = base[rank].clone()
    comm.all_reduce(m, "max")
    out["armax"] = float((m - torch.stack(base).max(0).values).abs().max())
    h = base[rank][:16].bfloat16()
    comm.all_reduce(h)
    out["ar_bf16"] = float((h.float() - sum(b[:16].bfloat16().float() for b in base)).abs().max())
    big = torch.full((3 * 1024 * 1024 + 5,), float(rank + 1))                # larger than the socket buffers
    comm.all_reduce(big)
    out["big"] = float((big - world * (world + 1) / 2).abs().max())
    ints = torch.arange(8, dtype=torch.int64) + rank
    out["ag"] = comm.all_gather(ints).tolist()
    full = torch.arange(world * 6, dtype=torch.float32).reshape(world * 2, 3) * (rank + 1)
    out["rs"] = comm.reduce_scatter(full).tolist()
    b = np.full(2_500_000, rank, dtype=np.int32)
    comm.broadcast(b, root=1)
    out["bc"] = int(b.min()), int(b.max())
    if world > 1:
        comm.send_next(torch.tensor([rank], dtype=torch.int32))
        got = torch.zeros(1, dtype=torch.int32)
        comm.recv_prev(got)
        out["p2p"] = int(got)
    comm.barrier()
    comm.close()
    return out


@pytest.mark.parametrize("world", [3, 4])
def test_ring_collectives(world):
    res = run_ranks(_worker, world)
    s = world * (world + 1) / 2
    for rank, r in enumerate(res):
        assert r["ar"] < 1e-5 and r["armax"] == 0.0 and r["big"] == 0.0
        assert r["ar_bf16"] < 0.1
        assert r["ag"] == [i + k for k in range(world) for i in range(8)]
        expect = (torch.arange(world * 6, dtype=torch.float32).reshape(world * 2, 3) * s)[2 * rank:2 * rank + 2]
        assert r["rs"] == expect.tolist()
        assert r["bc"] == (1, 1)
        assert r["p2p"] == (rank - 1) % world


def _lonely(rank, world):
    from mindspore_b200.communication.host_collectives import HostCollectiveError, HostCommunicator
    if rank == 1:
        return "absent"                       # never joins the ring
    try:
        HostCommunicator.from_env(timeout=2.0)
    except HostCollectiveError as e:
        return str(e)
    return "joined"


def test_missing_rank_times_out():
    res = run_ranks(_lonely, 2)
    assert res[1] == "absent" and "timed out" in res[0]


def test_single_rank_is_identity():
    from mindspore_b200.communication.host_collectives import HostCommunicator
    c = HostCommunicator(0, 1, ["127.0.0.1:1"])
    t = torch.arange(5.0)
    assert c.all_reduce(t.clone()).tolist() == t.tolist()
    assert c.all_gather(t).tolist() == t.tolist()
    assert c.reduce_scatter(t).tolist() == t.tolist()
    c.barrier()
    c.close()
