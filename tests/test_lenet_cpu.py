"""Config 1: LeNet-5 on CPU, graph mode == pynative, matches a PyTorch reference, .ckpt round trip."""
import numpy as np
import torch
import torch.nn.functional as F

import mindspore_b200 as ms
from mindspore_b200 import nn
from mindspore_b200.models.lenet import LeNet5


def _data(n, bs=32):
    rng = np.random.RandomState(0)
    return [(rng.randn(bs, 1, 32, 32).astype(np.float32), rng.randint(0, 10, (bs,)).astype(np.int32)) for _ in range(n)]


def _train(mode, steps=6):
    ms.set_context(mode=mode, device_target="CPU")
    ms.set_seed(1)
    net = LeNet5()
    init = {p.name: p.detach().clone() for p in net.get_parameters()}
    model = ms.Model(net, nn.SoftmaxCrossEntropyWithLogits(sparse=True, reduction="mean"),
                     nn.Momentum(net.trainable_params(), 0.01, 0.9))
    mon = ms.LossMonitor(1000)
    model.train(1, _data(steps), callbacks=[mon])
    return net, init, mon.losses


def test_graph_mode_equals_pynative_and_torch():
    _, init, eager = _train(ms.PYNATIVE_MODE)
    _, _, graph = _train(ms.GRAPH_MODE)
    assert eager == graph
    w = {k: v.clone().requires_grad_(True) for k, v in init.items()}
    mom = {k: torch.zeros_like(v) for k, v in w.items()}
    ref = []
    for x, y in _data(6):
        h = F.max_pool2d(F.relu(F.conv2d(torch.from_numpy(x), w["conv1.weight"])), 2)
        h = F.max_pool2d(F.relu(F.conv2d(h, w["conv2.weight"])), 2).flatten(1)
        h = F.relu(F.linear(h, w["fc1.weight"], w["fc1.bias"]))
        h = F.relu(F.linear(h, w["fc2.weight"], w["fc2.bias"]))
        loss = F.cross_entropy(F.linear(h, w["fc3.weight"], w["fc3.bias"]), torch.from_numpy(y).long())
        gs = torch.autograd.grad(loss, list(w.values()))
        with torch.no_grad():
            for (k, p), g in zip(w.items(), gs):
                mom[k].mul_(0.9).add_(g)
                p.sub_(0.01 * mom[k])
        ref.append(loss.item())
    np.testing.assert_allclose(eager, ref, rtol=1e-5)


def test_loss_decreases_100_steps_graph_mode():
    ms.set_context(mode=ms.GRAPH_MODE, device_target="CPU")
    ms.set_seed(3)
    net = LeNet5()
    model = ms.Model(net, nn.SoftmaxCrossEntropyWithLogits(sparse=True, reduction="mean"),
                     nn.Momentum(net.trainable_params(), 0.01, 0.9))
    mon = ms.LossMonitor(1000)
    batch = _data(1)
    model.train(100, batch, callbacks=[mon])   # 100 steps on one fixed batch must overfit it
    assert len(mon.losses) == 100
    assert mon.losses[-1] < 0.5 * mon.losses[0]


def test_checkpoint_round_trip(tmp_path):
    net, _, _ = _train(ms.PYNATIVE_MODE, 2)
    path = ms.save_checkpoint(net, str(tmp_path / "lenet.ckpt"), append_dict={"epoch_num": 3, "note": "hello"})
    d = ms.load_checkpoint(path)
    assert int(d["epoch_num"]) == 3 and d["note"] == "hello"
    net2 = LeNet5()
    not_loaded, _ = ms.load_param_into_net(net2, d)
    assert not_loaded == []
    for a, b in zip(net.get_parameters(), net2.get_parameters()):
        assert a.name == b.name and torch.equal(a, b)
    # byte-exact: saving the loaded net gives the same file apart from nothing at all
    p2 = ms.save_checkpoint(net2, str(tmp_path / "again.ckpt"), append_dict={"epoch_num": 3, "note": "hello"})
    assert open(path, "rb").read() == open(p2, "rb").read()
