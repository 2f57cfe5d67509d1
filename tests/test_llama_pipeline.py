"""Config "pipeline_stages = 2 x model_parallel": the strategy-driven Llama split into two pipeline stages of
model-parallel ranks (1F1B, activations with their layouts handed over by point-to-point sends) must give the loss
and the gradients of the single-device model run with the same micro-batches.  CPU ranks over gloo here; the GPU
variant runs the same over NCCL point-to-point and the fused NVLink kernels inside each stage."""
import pytest
import torch

from _mp import run_ranks


def _worker(rank, world, device, stages, micro):
    import mindspore_b200 as ms
    from mindspore_b200 import nn
    from mindspore_b200.communication import init
    from mindspore_b200.models import llama, llama_tp
    from mindspore_b200.parallel.layout import slice_for_rank
    from mindspore_b200.parallel.pipeline import run_pipeline_step
    cuda = device == "cuda"
    if cuda:
        torch.cuda.set_device(rank)
    ms.set_context(device_target="GPU" if cuda else "CPU", device_id=rank if cuda else 0)
    init("nccl" if cuda else "mccl")
    mp = world // stages
    dt = torch.bfloat16 if cuda else torch.float32
    base = dict(vocab_size=512, hidden_size=256, num_layers=4, num_heads=2, num_kv_heads=2, ffn_hidden_size=512,
                seq_length=128, dtype=dt)
    if cuda:
        base.update(hidden_size=512, num_heads=4, num_kv_heads=4, ffn_hidden_size=1024, seq_length=256)
    ms.set_seed(7)
    tokens = torch.randint(0, 512, (2 * micro, base["seq_length"] + 1),
                           generator=torch.Generator().manual_seed(3)).to(torch.int32)
    if cuda:
        tokens = tokens.cuda()
    full = llama.LlamaForCausalLM(llama.LlamaConfig(model_parallel=1, **base))
    losses = []
    n = tokens.shape[0] // micro
    for i in range(micro):
        l = full(ms.Tensor(tokens[i * n:(i + 1) * n]))
        (l / micro).backward()
        losses.append(float(l))
    loss_ref = sum(losses) / micro
    full_w = {p.name: p.detach().clone() for p in full.get_parameters()}
    full_g = {p.name: p.grad.detach().clone() for p in full.get_parameters()}

    ms.set_auto_parallel_context(parallel_mode="semi_auto_parallel", device_num=world, global_rank=rank,
                                 full_batch=True, pipeline_stages=stages)
    cfg = llama.LlamaConfig(model_parallel=mp, **base)
    net = llama.LlamaForCausalLM(cfg)
    packed = llama.pack_full_weights(full_w, cfg, mp)
    for p in net.get_parameters():
        w = packed[p.name].to(p.device)
        if p.param_layout is not None:
            w = slice_for_rank(w, p.param_layout, rank % mp).contiguous()
        p.set_data(w, slice_shape=True)
    cell = nn.PipelineCell(net, micro)
    loss = run_pipeline_step(cell, (ms.Tensor(tokens),), 1.0 / micro)
    stage = rank // mp
    per = cfg.num_layers // stages
    g_ref = llama_tp.shard_full_weights(full_g, cfg, mp, rank % mp)
    worst, checked = 0.0, 0
    for p in net.get_parameters():
        name = p.name
        if ".layers." in name:
            own = int(name.split(".layers.")[1].split(".")[0]) // per == stage
        elif "tok_embeddings" in name:
            own = stage == 0
        else:
            own = stage == stages - 1
        if not own:
            assert p.grad is None or float(p.grad.abs().max()) == 0.0, name
            continue
        g = p.grad.detach().float()
        r = g_ref[name].float().to(g.device)
        worst = max(worst, float((g - r).abs().max() / (r.abs().max() + 1e-8)))
        checked += 1
    torch.distributed.barrier()
    return stage, float(loss), loss_ref, worst, checked


@pytest.mark.parametrize("world,stages", [(4, 2), (2, 2), (4, 4)])
def test_pipeline_llama_matches_single_cpu(world, stages):
    """pp2 x mp2, and pure pipelines (one rank per stage) of 2 and 4 stages."""
    res = run_ranks(_worker, world, "cpu", stages, 2, timeout=420)
    for stage, loss, ref, worst, checked in res:
        if stage == stages - 1:
            assert abs(loss - ref) < 1e-4, (loss, ref)
        assert worst < 1e-3 and checked > 0, (stage, worst, checked)


@pytest.mark.gpu
def test_pp2_mp2_llama_matches_single_gpu():
    if torch.cuda.device_count() < 4:
        pytest.skip("needs 4 GPUs")
    res = run_ranks(_worker, 4, "cuda", 2, 2, timeout=420)
    for stage, loss, ref, worst, checked in res:
        if stage == 1:
            assert abs(loss - ref) < 3e-2, (loss, ref)
        assert worst < 8e-2 and checked > 0, (stage, worst, checked)
