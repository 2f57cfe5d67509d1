"""Optimizer state in checkpoints: a run that is saved after N steps and resumed in a fresh net + optimizer must
continue exactly like an uninterrupted run of 2N steps - moments, fp32 master weights and the step that drives the
learning-rate schedule and Adam's bias correction all come back (arena form included).
Parity: the reference saves adam_m.* / adam_v.* / moments.* / global_step as Parameters of the train network
(mindspore/python/mindspore/nn/optim/adam.py:866, momentum.py:50, optimizer.py:72)."""
import pytest
import torch

import mindspore_b200 as ms
from mindspore_b200 import nn


def _build(dtype, arena):
    ms.set_seed(11)
    net = nn.SequentialCell([nn.Dense(6, 8), nn.ReLU(), nn.Dense(8, 3)])
    if dtype != torch.float32:
        net.to_float(dtype)
        for p in net.get_parameters():
            p.set_data(p.detach().to(dtype), slice_shape=True)
    loss = nn.SoftmaxCrossEntropyWithLogits(sparse=True, reduction="mean")
    opt = nn.AdamWeightDecay(net.trainable_params(), learning_rate=nn.ExponentialDecayLR(0.05, 0.8, 2),
                             weight_decay=0.01, use_arena=arena, bias_correction=True)
    step = nn.TrainOneStepCell(nn.WithLossCell(net, loss), opt)
    step.set_train()
    return net, step, opt


def _data(i, dtype):
    g = torch.Generator().manual_seed(100 + i)
    return (ms.Tensor(torch.randn(16, 6, generator=g).to(dtype)),
            ms.Tensor(torch.randint(0, 3, (16,), generator=g).to(torch.int32)))


@pytest.mark.parametrize("dtype,arena", [(torch.float32, False), (torch.float32, True), (torch.bfloat16, True)])
def test_resume_equals_uninterrupted(tmp_path, dtype, arena):
    n = 4
    net, step, opt = _build(dtype, arena)
    for i in range(2 * n):
        step(*_data(i, dtype))
    want = {p.name: p.detach().float().clone() for p in net.get_parameters()}

    net, step, opt = _build(dtype, arena)
    for i in range(n):
        step(*_data(i, dtype))
    path = ms.save_checkpoint(step, str(tmp_path / "half.ckpt"))
    saved = ms.load_checkpoint(path)
    assert any(k.startswith("adam_m.") for k in saved) and any(k.startswith("adam_v.") for k in saved)
    assert int(saved["global_step"].reshape(-1)[0]) == n
    if arena and dtype != torch.float32:
        assert any(k.startswith("fp32_master.") for k in saved)

    net2, step2, opt2 = _build(dtype, arena)
    ms.load_param_into_net(step2, saved)
    assert opt2._step_host == n
    for i in range(n, 2 * n):
        step2(*_data(i, dtype))
    for p in net2.get_parameters():
        torch.testing.assert_close(p.detach().float(), want[p.name], rtol=0, atol=0)


def test_load_state_dict_and_set_data_reach_the_master_copy():
    net, step, opt = _build(torch.bfloat16, True)
    step(*_data(0, torch.bfloat16))
    new = {p.name: torch.full(tuple(p.shape), 0.25) for p in net.get_parameters()}
    net.load_state_dict(new, strict=True)
    opt.arena.grads.zero_()
    opt._m.zero_()
    opt._v.zero_()
    opt.weight_decay = 0.0
    opt._arena_groups = [(f, l, 0.0) for f, l, _ in opt._arena_groups]
    opt.fused_step()                      # zero gradient, zero moments, no decay: the weights must not move
    for p in net.get_parameters():
        assert torch.all(p.detach().float() == 0.25), p.name
    p0 = next(iter(net.get_parameters()))
    p0.set_data(torch.full(tuple(p0.shape), -0.5, dtype=torch.bfloat16))
    opt.fused_step()
    assert torch.all(p0.detach().float() == -0.5)
