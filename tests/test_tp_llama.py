"""Tensor + sequence parallel Llama (mp=2) must reproduce the single-device loss and gradients.
CPU ranks over gloo exercise the parallel logic; the GPU variant runs the same check through NCCL and the
sm_100a kernels on 2 GPUs."""
import os
import sys

import pytest
import torch
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, device, q):
    sys.path.insert(0, ROOT)
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port),
                      LOCAL_RANK=str(rank))
    import mindspore_b200 as ms
    from mindspore_b200.communication import init
    from mindspore_b200.models.llama_tp import LlamaConfig, LlamaForCausalLM, shard_full_weights
    from mindspore_b200.parallel import tp as TP
    ms.set_context(device_target="GPU" if device == "cuda" else "CPU", device_id=rank if device == "cuda" else 0)
    init("nccl" if device == "cuda" else "mccl")
    ms.set_auto_parallel_context(parallel_mode="semi_auto_parallel", device_num=world, global_rank=rank)
    dt = torch.bfloat16 if device == "cuda" else torch.float32
    base = dict(vocab_size=512, hidden_size=256, num_layers=2, num_heads=2, num_kv_heads=2, ffn_hidden_size=512,
                seq_length=128, dtype=dt)
    torch.manual_seed(7)
    ms.set_seed(7)
    full = LlamaForCausalLM(LlamaConfig(model_parallel=1, **base))
    tokens = torch.randint(0, 512, (2, 129), generator=torch.Generator().manual_seed(3)).to(torch.int32)
    if device == "cuda":
        tokens = tokens.cuda()
    loss_ref = full(ms.Tensor(tokens))
    loss_ref.backward()
    full_w = {p.name: p.detach().clone() for p in full.get_parameters()}
    full_g = {p.name: p.grad.detach().clone() for p in full.get_parameters()}
    cfg = LlamaConfig(model_parallel=world, **base)
    net = LlamaForCausalLM(cfg, TP.TPGroup())
    shard = shard_full_weights(full_w, cfg, world, rank)
    for p in net.get_parameters():
        p.set_data(shard[p.name].to(p.device))
    loss = net(ms.Tensor(tokens))
    loss.backward()
    g_ref = shard_full_weights(full_g, cfg, world, rank)
    worst = 0.0
    for p in net.get_parameters():
        g = p.grad.detach().float()
        if getattr(p, "tp_grad_reduce", False):
            torch.distributed.all_reduce(g)
        r = g_ref[p.name].float().to(g.device)
        worst = max(worst, float((g - r).abs().max() / (r.abs().max() + 1e-8)))
    q.put((rank, float(loss), float(loss_ref), worst))
    torch.distributed.barrier()


def _run(world, device):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + (os.getpid() % 2000)
    procs = [ctx.Process(target=_worker, args=(r, world, port, device, q)) for r in range(world)]
    for p in procs:
        p.start()
    import queue as _q
    import time
    res, deadline = [], time.time() + 300
    while len(res) < world:
        try:
            res.append(q.get(timeout=2))
        except _q.Empty:
            dead = [p.exitcode for p in procs if p.exitcode not in (None, 0)]
            if dead or time.time() > deadline:
                for p in procs:
                    p.kill()
                raise AssertionError("worker failed or timed out: exit codes %s" % [p.exitcode for p in procs])
    for p in procs:
        p.join(60)
        assert p.exitcode == 0
    return res


def test_tp2_matches_single_cpu():
    for rank, loss, ref, worst in _run(2, "cpu"):
        assert abs(loss - ref) < 1e-4, (rank, loss, ref)
        assert worst < 1e-3, (rank, worst)


@pytest.mark.gpu
def test_tp2_matches_single_gpu():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    for rank, loss, ref, worst in _run(2, "cuda"):
        assert abs(loss - ref) < 3e-2, (rank, loss, ref)
        assert worst < 8e-2, (rank, worst)
