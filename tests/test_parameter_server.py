"""Parameter server: two worker processes + a server thread reproduce single-process training on the joint batch."""
import numpy as np
import torch

from _mp import run_ranks

PORT = 29731


def _build(ms, nn):
    ms.set_seed(2)

    class Net(nn.Cell):
        def __init__(self):
            super().__init__()
            self.emb = nn.Embedding(12, 4)
            self.fc = nn.Dense(4, 1)

        def construct(self, ids):
            return self.fc(self.emb(ids).mean(1))

    net = Net()
    for p in net.get_parameters():
        p.set_param_ps()
    return net


def _data():
    g = torch.Generator().manual_seed(4)
    return torch.randint(0, 6, (8, 3), generator=g), torch.randn(8, 1, generator=g)      # rows 6..11 are never used


def _rank(rank, world):
    import mindspore_b200 as ms
    from mindspore_b200 import nn
    from mindspore_b200.parallel.ps import ParameterServer, PSWorker
    ms.set_context(device_target="CPU")
    if rank == 0:
        ParameterServer(("127.0.0.1", PORT), num_workers=2, optimizer="sgd", learning_rate=0.2, momentum=0.9).start()
    net = _build(ms, nn)
    worker = PSWorker(("127.0.0.1", PORT), rank)
    worker.init_params(net)
    ids, y = _data()
    n = ids.shape[0] // 2
    ids, y = ids[rank * n:(rank + 1) * n], y[rank * n:(rank + 1) * n]
    for _ in range(3):
        worker.pull(net)
        loss = ((net(ms.Tensor(ids)) - ms.Tensor(y)) ** 2).mean()
        loss.backward()
        worker.push(net, sparse=True)
    worker.pull(net)
    out = {p.name: p.detach().numpy().copy() for p in net.get_parameters()}
    worker.close()
    return out


def test_two_workers_match_single_process():
    import mindspore_b200 as ms
    from mindspore_b200 import nn
    ref_net = _build(ms, nn)
    ids, y = _data()
    opt = torch.optim.SGD([p for p in ref_net.get_parameters()], lr=0.2, momentum=0.9)
    for _ in range(3):
        opt.zero_grad()
        ((ref_net(ms.Tensor(ids)) - ms.Tensor(y)) ** 2).mean().backward()
        opt.step()
    ref = {p.name: p.detach().numpy() for p in ref_net.get_parameters()}
    res = run_ranks(_rank, 2, timeout=120)
    for got in res:
        for k in ref:
            np.testing.assert_allclose(got[k], ref[k], rtol=1e-5, atol=1e-6)
