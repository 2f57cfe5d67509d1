"""The strategy-driven Llama (``models/llama.py``: primitives + ``shard`` only, communication inserted by the
dispatcher) must give the loss and gradients of (a) the single-device model and (b) the hand-placed tensor-parallel
formulation (``models/llama_tp.py``).  CPU ranks over gloo check the inserted redistribution / forward communication
/ mirrors; the GPU variant checks that the same strategies run through the fused NVLink kernels.
Reference behaviour: frontend/parallel/step_parallel.cc:2738-2793, ops_info/matmul_info.cc:290-403."""
import pytest
import torch

from _mp import run_ranks

BASE = dict(vocab_size=512, hidden_size=256, num_layers=2, num_heads=2, num_kv_heads=2, ffn_hidden_size=512,
            seq_length=128)


def _worker(rank, world, device, sp):
    import mindspore_b200 as ms
    from mindspore_b200.communication import init
    from mindspore_b200.models import llama, llama_tp
    from mindspore_b200.parallel import spmd, tp as TP
    from mindspore_b200.parallel.layout import slice_for_rank
    cuda = device == "cuda"
    if cuda:
        torch.cuda.set_device(rank)
    ms.set_context(device_target="GPU" if cuda else "CPU", device_id=rank if cuda else 0)
    init("nccl" if cuda else "mccl")
    dt = torch.bfloat16 if cuda else torch.float32
    base = dict(BASE, dtype=dt, sequence_parallel=sp)
    if cuda:
        base.update(hidden_size=512, num_heads=4, num_kv_heads=4, ffn_hidden_size=1024, seq_length=256)
    torch.manual_seed(7)
    ms.set_seed(7)
    tokens = torch.randint(0, 512, (2, base["seq_length"] + 1), generator=torch.Generator().manual_seed(3)).to(torch.int32)
    if cuda:
        tokens = tokens.cuda()

    # (a) one device
    full = llama.LlamaForCausalLM(llama.LlamaConfig(model_parallel=1, **base))
    loss_ref = full(ms.Tensor(tokens))
    loss_ref.backward()
    full_w = {p.name: p.detach().clone() for p in full.get_parameters()}
    full_g = {p.name: p.grad.detach().clone() for p in full.get_parameters()}

    # (b) hand-placed tensor parallelism
    ms.set_auto_parallel_context(parallel_mode="semi_auto_parallel", device_num=world, global_rank=rank,
                                 full_batch=True)
    cfg = llama.LlamaConfig(model_parallel=world, **base)
    net_tp = llama_tp.LlamaForCausalLM(cfg, TP.TPGroup())
    shard = llama_tp.shard_full_weights(full_w, cfg, world, rank)
    for p in net_tp.get_parameters():
        p.set_data(shard[p.name].to(p.device))
    loss_tp = net_tp(ms.Tensor(tokens))
    loss_tp.backward()
    g_tp = {}
    for p in net_tp.get_parameters():
        g = p.grad.detach().float()
        if getattr(p, "tp_grad_reduce", False):
            torch.distributed.all_reduce(g)
        g_tp[p.name] = g

    # (c) strategies only
    net = llama.LlamaForCausalLM(cfg)
    packed = llama.pack_full_weights(full_w, cfg, world)
    sliced = 0
    for p in net.get_parameters():
        w = packed[p.name].to(p.device)
        if p.param_layout is not None:
            w = slice_for_rank(w, p.param_layout, rank).contiguous()
            sliced += 1
        p.set_data(w, slice_shape=True)
    records = []
    from mindspore_b200.ops import primitive as prim_mod
    orig = spmd.dispatch

    def spy(prim, args, kwargs):
        out = orig(prim, args, kwargs)
        if spmd.last_dispatch is not None:
            records.append((prim.name, dict(spmd.last_dispatch)))
        return out
    spmd.dispatch = spy
    try:
        loss = net(ms.Tensor(tokens))
    finally:
        spmd.dispatch = orig
    loss.backward()
    worst_tp = worst_full = 0.0
    g_ref = llama_tp.shard_full_weights(full_g, cfg, world, rank)
    for p in net.get_parameters():
        g = p.grad.detach().float()
        worst_tp = max(worst_tp, float((g - g_tp[p.name]).abs().max() / (g_tp[p.name].abs().max() + 1e-8)))
        r = g_ref[p.name].float().to(g.device)
        worst_full = max(worst_full, float((g - r).abs().max() / (r.abs().max() + 1e-8)))
    fused = sorted({r["fused"] for _, r in records if r.get("fused")})
    comm = sorted({(n, r["forward_comm"][0]) for n, r in records if r.get("forward_comm")})
    redis = sorted({(n, tuple(r["redistribution"])) for n, r in records if r.get("redistribution")})
    from mindspore_b200 import _native
    status = _native.device_status() if cuda else 0
    torch.distributed.barrier()
    return dict(loss=float(loss), loss_tp=float(loss_tp), loss_ref=float(loss_ref), worst_tp=worst_tp,
                worst_full=worst_full, sliced=sliced, fused=fused, comm=comm, redis=redis, status=status,
                nparams=len(list(net.get_parameters())))


@pytest.mark.parametrize("sp", [True, False])
def test_strategy_driven_llama_matches_tp_and_single_cpu(sp):
    for r in run_ranks(_worker, 2, "cpu", sp):
        assert abs(r["loss"] - r["loss_ref"]) < 1e-4 and abs(r["loss"] - r["loss_tp"]) < 1e-5, r
        assert r["worst_tp"] < 1e-4 and r["worst_full"] < 1e-3, r
        # wqkv, wo, w_gate_up, w_down per layer + embedding + lm_head are sliced at construction
        assert r["sliced"] == 2 * 4 + 2, r
        names = dict(r["comm"])
        if sp:
            assert names.get("MatMul") == "ReduceScatter" and names.get("Gather") == "ReduceScatter", r
            assert ("MatMul", ("AllGather",)) in r["redis"], r
        else:
            assert names.get("MatMul") == "AllReduce" and names.get("Gather") == "AllReduce", r
        assert "VocabParallelCrossEntropy" in r["fused"], r


@pytest.mark.gpu
def test_strategy_driven_llama_uses_the_fused_kernels_gpu():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    for r in run_ranks(_worker, 2, "cuda", True):
        assert abs(r["loss"] - r["loss_ref"]) < 3e-2 and abs(r["loss"] - r["loss_tp"]) < 2e-2, r
        assert r["worst_tp"] < 8e-2 and r["worst_full"] < 8e-2, r
        assert "MatMulReduceScatter" in r["fused"] and "AllGatherMatMul" in r["fused"], r
        assert r["status"] == 0, r
