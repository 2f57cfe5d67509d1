"""Elementwise clusters -> one generated kernel: clustering rules, the expression oracle, the generated CUDA text
(compiled for sm_100a here, run on a GPU in the gpu-marked test)."""
import numpy as np
import pytest
import torch

import mindspore_b200 as ms
from mindspore_b200 import nn, ops
from mindspore_b200.graph import graph_kernel as GK
from mindspore_b200.graph.jit import trace_cell


class Chain(nn.Cell):
    def construct(self, x, y):
        a = ops.Add()(x, y)
        b = ops.Mul()(a, 2.0)
        c = ops.Tanh()(b)
        d = ops.Sub()(1.5, c)
        return ops.Maximum()(d, x), ops.ReLU()(a)


def _fused_nodes(fg):
    return [n for n in fg.graph.nodes if n.op == "call_function" and isinstance(n.target, GK.FusedElementwise)]


def test_chain_becomes_one_node_with_two_outputs():
    net = Chain()
    x = ms.Tensor(np.random.RandomState(0).randn(4, 8).astype(np.float32))
    y = ms.Tensor(np.random.RandomState(1).randn(4, 8).astype(np.float32))
    fg = trace_cell(net, (x, y))
    assert GK.fuse_elementwise(fg) == 1
    (node,) = _fused_nodes(fg)
    fused = node.target
    assert [s[0] for s in fused.steps] == ["Add", "Mul", "Tanh", "Sub", "Maximum", "ReLU"]
    assert fused.n_inputs == 2 and len(fused.outputs) == 2
    assert fg.count("Add") == 0 and fg.count("Tanh") == 0
    want = net(x, y)
    got = fused.reference(x.as_subclass(torch.Tensor), y.as_subclass(torch.Tensor))
    for g, w in zip(got, want):
        assert torch.allclose(g, w.as_subclass(torch.Tensor), atol=1e-6)
    from mindspore_b200.graph.executor import GraphExecutor
    out = GraphExecutor(fg).run([x, y])
    for g, w in zip(out, want):
        assert torch.allclose(g.as_subclass(torch.Tensor), w.as_subclass(torch.Tensor), atol=1e-6)


def test_clustering_respects_order_shapes_and_the_context_flag():
    class Mixed(nn.Cell):
        def __init__(self):
            super().__init__()
            self.fc = nn.Dense(8, 8)

        def construct(self, x, bias):
            a = ops.Exp()(x)                      # used by the matmul below: an outside user in the middle
            h = self.fc(a)
            b = ops.Mul()(a, 0.5)
            c = ops.Add()(b, h)
            d = ops.Add()(c, bias)                # bias broadcasts ([8] vs [4, 8]): not part of a cluster
            return ops.Sigmoid()(ops.Neg()(d))

    net = Mixed()
    x = ms.Tensor(np.random.RandomState(2).randn(4, 8).astype(np.float32))
    bias = ms.Tensor(np.random.RandomState(3).randn(8).astype(np.float32))
    fg = trace_cell(net, (x, bias))
    made = GK.fuse_elementwise(fg)
    names = [tuple(s[0] for s in n.target.steps) for n in _fused_nodes(fg)]
    assert made == len(names) and ("Neg", "Sigmoid") in names
    assert all("Exp" not in n or n.index("Exp") == 0 for n in names)
    from mindspore_b200.graph.executor import GraphExecutor
    got = GraphExecutor(fg).run([x, bias])
    assert torch.allclose(got.as_subclass(torch.Tensor), net(x, bias).as_subclass(torch.Tensor), atol=1e-5)

    ms.set_context(mode=ms.GRAPH_MODE, enable_graph_kernel=True)
    try:
        chain = Chain()
        y = ms.Tensor(np.ones((4, 8), np.float32))
        out = chain(x, y)
        cg = next(iter(chain._compiled.values()))
        assert len(_fused_nodes(cg.fg if hasattr(cg, "fg") else cg.executor.fg)) == 1
    finally:
        ms.set_context(mode=ms.PYNATIVE_MODE, enable_graph_kernel=False)
    ref = Chain()(x, y)
    assert torch.allclose(out[0].as_subclass(torch.Tensor), ref[0].as_subclass(torch.Tensor), atol=1e-6)


def test_generated_source_compiles_for_sm_100a(tmp_path, monkeypatch):
    monkeypatch.setenv("MSB200_KERNEL_CACHE", str(tmp_path))
    steps = [("Add", [("in", 0), ("in", 1)]), ("Mul", [("tmp", 0), ("const", 0.5)]), ("Sigmoid", [("tmp", 1)]),
             ("Sub", [("const", 1.0), ("tmp", 2)]), ("Maximum", [("tmp", 3), ("in", 0)])]
    for dtype in (torch.bfloat16, torch.float32):
        src = GK.kernel_source(steps, [4, 0], 2, dtype)
        assert "fmaxf(t3, x0)" in src and "(1.0f) - t2" in src and "expf(-t1)" in src
        lib = GK.compile_source(src)
        assert lib.endswith(".so") and (tmp_path / lib.split("/")[-1]).stat().st_size > 0
        assert GK.compile_source(src) == lib                       # cached by the hash of the source


@pytest.mark.gpu
def test_generated_kernel_matches_the_expression_on_the_gpu():
    steps = [("Add", [("in", 0), ("in", 1)]), ("Mul", [("tmp", 0), ("const", 0.5)]), ("Sigmoid", [("tmp", 1)]),
             ("Sub", [("const", 1.0), ("tmp", 2)]), ("Maximum", [("tmp", 3), ("in", 0)])]
    for dtype, tol in ((torch.float32, 1e-6), (torch.bfloat16, 1e-2), (torch.float16, 2e-3)):
        fused = GK.FusedElementwise(steps, [4, 0], 2, dtype)
        for n in (1, 7, 4096, 8 * 1000 + 3):
            a = torch.randn(n, device="cuda").to(dtype)
            b = torch.randn(n, device="cuda").to(dtype)
            got = fused(a, b)
            want = fused.reference(a, b)
            for g, w in zip(got, want):
                assert torch.allclose(g.float(), w.float(), atol=tol, rtol=tol)
        base = torch.randn(4097, device="cuda").to(dtype)
        odd = base[1:]                                             # not 16-byte aligned: the scalar path
        got = fused(odd, odd)
        assert torch.allclose(got[0].float(), fused.reference(odd, odd)[0].float(), atol=tol, rtol=tol)
    x = torch.randn(64, 64, device="cuda", requires_grad=True)
    y = torch.randn(64, 64, device="cuda", requires_grad=True)
    fused = GK.FusedElementwise(steps, [4], 2, torch.float32)
    out = fused(x, y)
    out.sum().backward()
    gx, gy = x.grad.clone(), y.grad.clone()
    x.grad = y.grad = None
    fused.reference(x, y).sum().backward()
    assert torch.allclose(gx, x.grad, atol=1e-6) and torch.allclose(gy, y.grad, atol=1e-6)
