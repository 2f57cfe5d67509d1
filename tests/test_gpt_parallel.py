"""GPT built from the parallel transformer blocks: dp x mp (+ sharded optimizer) over gloo ranks reproduces the
single-process training trajectory."""
import pytest
import torch

from _mp import run_ranks

BASE = dict(seq_length=32, vocab_size=128, hidden_size=32, num_layers=2, num_heads=4, dtype=torch.float32)


def _tokens():
    return torch.randint(0, 128, (4, 33), generator=torch.Generator().manual_seed(3)).to(torch.int32)


def _single(steps):
    import mindspore_b200 as ms
    from mindspore_b200 import nn
    from mindspore_b200.models.gpt import GPTConfig, GPTForCausalLM
    ms.set_seed(5)
    torch.manual_seed(5)
    net = GPTForCausalLM(GPTConfig(**BASE))
    init_w = {p.name: p.detach().clone() for p in net.get_parameters()}
    opt = nn.AdamWeightDecay(net.trainable_params(), learning_rate=1e-2, weight_decay=0.0, use_arena=True,
                             max_grad_norm=1.0)
    step = nn.TrainOneStepCell(net, opt)
    losses = [float(step(ms.Tensor(_tokens()))) for _ in range(steps)]
    return init_w, losses, {p.name: p.detach().clone() for p in net.get_parameters()}


def _worker(rank, world, dp, mp, shard, init_w, steps):
    import mindspore_b200 as ms
    from mindspore_b200 import nn
    from mindspore_b200.communication import init
    from mindspore_b200.models.gpt import GPTConfig, GPTForCausalLM, shard_full_weights
    from mindspore_b200.parallel.transformer import TransformerOpParallelConfig
    ms.set_context(device_target="CPU")
    init("mccl")
    ms.set_auto_parallel_context(parallel_mode="semi_auto_parallel", device_num=world, global_rank=rank)
    pc = TransformerOpParallelConfig(data_parallel=dp, model_parallel=mp, vocab_emb_dp=False)
    cfg = GPTConfig(parallel_config=pc, **BASE)
    net = GPTForCausalLM(cfg)
    g = pc.groups()
    shard_w = shard_full_weights(init_w, cfg, mp, g["tp"].rank)
    for p in net.get_parameters():
        p.set_data(shard_w[p.name])
    opt = nn.AdamWeightDecay(net.trainable_params(), learning_rate=1e-2, weight_decay=0.0, use_arena=True,
                             max_grad_norm=1.0)
    if mp > 1:
        opt.set_model_parallel_group(g["tp"].name)
    if dp > 1:
        opt.set_data_parallel_group(g["dp"], mean=True, shard=shard)
    step = nn.TrainOneStepCell(net, opt)
    tok = _tokens()
    n = tok.shape[0] // dp
    d = rank // mp
    losses = [float(step(ms.Tensor(tok[d * n:(d + 1) * n]))) for _ in range(steps)]
    torch.distributed.barrier()
    return g["tp"].rank, d, losses, {p.name: p.detach().clone() for p in net.get_parameters()}


@pytest.mark.parametrize("dp,mp,shard", [(1, 2, False), (2, 2, True), (2, 1, True)])
def test_gpt_dp_mp_matches_single_process(dp, mp, shard):
    from mindspore_b200.models.gpt import GPTConfig, shard_full_weights
    from mindspore_b200.parallel.transformer import TransformerOpParallelConfig
    steps = 3
    init_w, ref_losses, ref_final = _single(steps)
    res = run_ranks(_worker, dp * mp, dp, mp, shard, init_w, steps, timeout=600)
    cfg = GPTConfig(parallel_config=TransformerOpParallelConfig(model_parallel=mp, vocab_emb_dp=False), **BASE)
    by_dp = {}
    for tp_rank, d, losses, params in res:
        by_dp.setdefault(d, losses)
        want = shard_full_weights(ref_final, cfg, mp, tp_rank)
        for name, value in params.items():
            torch.testing.assert_close(value, want[name], rtol=2e-4, atol=2e-5)
    mean_losses = [sum(by_dp[d][i] for d in by_dp) / len(by_dp) for i in range(steps)]
    assert mean_losses == pytest.approx(ref_losses, rel=1e-4)
