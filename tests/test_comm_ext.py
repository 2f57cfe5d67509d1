"""NeighborExchangeV2 (halo exchange) and _AllSwap on CPU ranks."""
import torch

from _mp import run_ranks


def _halo(rank, world):
    import mindspore_b200 as ms
    from mindspore_b200.communication import init
    from mindspore_b200.ops import comm_ops as CO
    ms.set_context(device_target="CPU")
    init("gloo")
    # two ranks stacked vertically: rank 0 on top, rank 1 below; 1-row halos
    x = torch.full((1, 1, 3, 4), float(rank + 1))
    x[0, 0, :, 0] += 0.5
    if rank == 0:
        op = CO.NeighborExchangeV2([-1, -1, -1, -1, 1, -1, -1, -1], [0, 1, 0, 0], [-1, -1, -1, -1, 1, -1, -1, -1],
                                   [0, 1, 0, 0])
    else:
        op = CO.NeighborExchangeV2([0, -1, -1, -1, -1, -1, -1, -1], [1, 0, 0, 0], [0, -1, -1, -1, -1, -1, -1, -1],
                                   [1, 0, 0, 0])
    y = op(ms.Tensor(x))
    swap = CO._AllSwap()
    send = torch.arange(3.0) + 10 * rank                 # rank 0 sends [1, 2] elements to (0, 1); rank 1 sends [2, 1]
    sizes = [1, 2] if rank == 0 else [2, 1]
    recv = [1, 2] if rank == 0 else [2, 1]
    got = swap(ms.Tensor(send), sizes, recv)
    return y.numpy().tolist(), got.numpy().tolist()


def test_halo_exchange_and_allswap():
    (y0, s0), (y1, s1) = run_ranks(_halo, 2)
    assert len(y0[0][0]) == 4 and len(y1[0][0]) == 4
    assert y0[0][0][3] == [2.5, 2.0, 2.0, 2.0]            # rank 0's bottom halo = rank 1's top row
    assert y1[0][0][0] == [1.5, 1.0, 1.0, 1.0]            # rank 1's top halo = rank 0's bottom row
    assert y0[0][0][0] == [1.5, 1.0, 1.0, 1.0] and y1[0][0][3] == [2.5, 2.0, 2.0, 2.0]
    assert s0 == [0.0, 10.0, 11.0]                         # own first element, then rank 1's first two
    assert s1 == [1.0, 2.0, 12.0]
