"""MPMD by placement labels on CPU ranks: each labelled cell runs on its rank only, the result matches one process."""
import pytest
import torch

from _mp import run_ranks


def _build(ms, nn):
    ms.set_seed(5)

    class Net(nn.Cell):
        def __init__(self):
            super().__init__()
            self.enc = nn.Dense(6, 8)
            self.mid = nn.Dense(8, 8)
            self.dec = nn.Dense(8, 3)
            self.ran = []

        def construct(self, x):
            h = torch.tanh(self.enc(x))
            h = self.mid(h) + 1.0                      # unlabelled arithmetic between placed cells
            return self.dec(h) * 2.0, h

    return Net()


def _worker(rank, world):
    import mindspore_b200 as ms
    from mindspore_b200 import nn
    from mindspore_b200.communication import init
    from mindspore_b200.parallel.mpmd import run_placed
    ms.set_context(device_target="CPU")
    init("gloo")
    net = _build(ms, nn)
    x = ms.Tensor(torch.arange(24.0).reshape(4, 6) / 10)
    ref = [t.detach().clone() for t in net(x)]
    counts = {}
    for name in ("enc", "mid", "dec"):
        cell = getattr(net, name)
        cell.register_forward_hook(lambda c, i, o, n=name: counts.__setitem__(n, counts.get(n, 0) + 1))
    net.enc.place("MS_WORKER", 0)
    net.mid.place("MS_WORKER", 1)
    net.dec.place("MS_WORKER", 0)
    out = run_placed(net, x)
    err = max(float((a - b).abs().max()) for a, b in zip(out, ref))
    torch.distributed.barrier()
    return err, counts


def test_placed_cells_run_on_their_rank_only():
    res = run_ranks(_worker, 2, timeout=120)
    for err, _ in res:
        assert err < 1e-6
    assert res[0][1] == {"enc": 1, "dec": 1} and res[1][1] == {"mid": 1}


def test_place_validates_arguments():
    from mindspore_b200 import nn
    with pytest.raises(ValueError):
        nn.Dense(2, 2).place("WORKER", 0)
    with pytest.raises(ValueError):
        nn.Dense(2, 2).place("MS_WORKER", -1)
