"""GRAPH_MODE with the flat-arena optimizer: the micro-batch forward + backward of the strategy-driven Llama is traced
into one graph (fused primitives, reverse-mode nodes that accumulate into the fp32 gradient arena), goes through the
pass pipeline and trains to the same numbers as PYNATIVE_MODE."""
import os

import torch

import mindspore_b200 as ms
from mindspore_b200 import nn
from mindspore_b200.models.llama import LlamaConfig, LlamaForCausalLM


def _train(mode, tmp_path=None, accumulate=True, steps=3):
    kw = dict(save_graphs=2, save_graphs_path=str(tmp_path)) if tmp_path is not None else {}
    ms.set_context(mode=mode, device_target="CPU", **kw)
    ms.set_seed(0)
    cfg = LlamaConfig(vocab_size=256, hidden_size=64, ffn_hidden_size=128, num_layers=2, num_heads=4, num_kv_heads=4,
                      seq_length=32, dtype=ms.float32)
    net = LlamaForCausalLM(cfg)
    opt = nn.AdamWeightDecay(net.trainable_params(), learning_rate=1e-3, use_arena=True, max_grad_norm=1.0)
    step = nn.TrainOneStepCell(nn.GradAccumulationCell(net, 2) if accumulate else net, opt)
    step.set_train()
    assert step.use_arena
    g = torch.Generator().manual_seed(1)
    losses = []
    for _ in range(steps):
        tokens = ms.Tensor(torch.randint(0, 256, (4, 33), generator=g))
        losses.append(float(step(tokens)))
    return losses, [p.detach().clone().float() for p in net.get_parameters()], step


def test_compiled_micro_batch_trains_like_eager(tmp_path):
    try:
        ref_l, ref_p, _ = _train(ms.PYNATIVE_MODE)
        l, p, step = _train(ms.GRAPH_MODE, tmp_path)
    finally:
        ms.set_context(mode=ms.PYNATIVE_MODE, save_graphs=0)
    assert l == ref_l
    for a, b in zip(p, ref_p):
        torch.testing.assert_close(a, b, rtol=0, atol=1e-6)
    cg = step._runner._compiled
    names = [getattr(n.target, "name", getattr(n.target, "__name__", "")) for n in cg.fg.graph.nodes
             if n.op == "call_function"]
    assert "AddRmsNorm" in names and "SwiGLU" in names and "RotaryFlashAttention" in names and "vjp" in names
    assert not any(o.op == "call_function" and getattr(o.target, "__name__", "") == "vjp"
                   for o in cg.fg.output_node.all_input_nodes), "weight gradients must not be graph outputs"
    dumped = sorted(os.listdir(tmp_path))
    assert any(f.endswith("_00_trace.ir") for f in dumped) and any("cse" in f for f in dumped), dumped
    assert cg.memory_report()["tensors"] > 0


def test_compiled_step_without_accumulation():
    try:
        ref_l, ref_p, _ = _train(ms.PYNATIVE_MODE, accumulate=False)
        l, p, _ = _train(ms.GRAPH_MODE, accumulate=False)
    finally:
        ms.set_context(mode=ms.PYNATIVE_MODE)
    assert l == ref_l
    for a, b in zip(p, ref_p):
        torch.testing.assert_close(a, b, rtol=0, atol=1e-6)
