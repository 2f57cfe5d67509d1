"""Cell-level ``shard``: strategies given once for a cell's inputs / outputs and a parameter plan drive the
un-annotated primitives inside by propagation; 2 gloo ranks must reproduce the single-device loss and gradients.
Reference: python/mindspore/parallel/shard.py:129-345, tests/ut/python/parallel/test_shard*.py."""
import torch

from _mp import run_ranks


def _build(ms, nn, ops):
    class Block(nn.Cell):
        def __init__(self):
            super().__init__()
            torch.manual_seed(5)
            self.w1 = ms.Parameter(ms.Tensor(torch.randn(32, 64) * 0.1), name="w1")
            self.w2 = ms.Parameter(ms.Tensor(torch.randn(64, 16) * 0.1), name="w2")
            self.m1, self.m2 = ops.MatMul(), ops.MatMul()      # no strategies on the primitives
            self.relu, self.sum, self.mul = ops.ReLU(), ops.ReduceSum(), ops.Mul()

        def construct(self, x):
            h = self.relu(self.m1(x, self.w1))
            y = self.m2(h, self.w2)
            return self.sum(self.mul(y, y), ())
    return Block()


def _worker(rank, world, mode):
    import mindspore_b200 as ms
    from mindspore_b200 import nn, ops
    from mindspore_b200.communication import init
    from mindspore_b200.parallel import spmd
    from mindspore_b200.parallel.layout import Layout, slice_for_rank
    ms.set_context(device_target="CPU")
    x = torch.randn(8, 32, generator=torch.Generator().manual_seed(1))
    ref = _build(ms, nn, ops)
    lr = ref(ms.Tensor(x))
    gr = torch.autograd.grad(lr, [ref.w1, ref.w2])
    init("mccl")
    ms.set_auto_parallel_context(parallel_mode="semi_auto_parallel", device_num=world, global_rank=rank,
                                 full_batch=True)
    net = _build(ms, nn, ops)
    if mode == "dp":
        fn = net.shard(in_strategy=((world, 1),))
    elif mode == "mp":
        fn = net.shard(in_strategy=((1, 1),), parameter_plan={"w1": (1, world), "w2": (world, 1)})
    else:
        lay = Layout((world,), ("mp",))
        fn = ms.shard(net, in_strategy=(None,), parameter_plan={"w1": lay("None", "mp"), "w2": lay("mp", "None")})
    loss = fn(ms.Tensor(x))
    full = float(spmd.to_full(loss))
    g = torch.autograd.grad(spmd.virtual_div_loss(loss), [net.w1, net.w2])
    errs = []
    for p, gi, gf in zip([net.w1, net.w2], g, gr):
        want = slice_for_rank(gf, p.param_layout, rank) if p.param_layout is not None else gf
        errs.append(float((gi - want).abs().max()))
    lays = {k: v.tensor_strategy() for k, v in spmd.parameter_layouts.items()}
    torch.distributed.barrier()
    return full, float(lr), max(errs), lays


def test_cell_shard_drives_unannotated_primitives():
    for mode, want in (("dp", {"w1": (1, 1), "w2": (1, 1)}), ("mp", {"w1": (1, 2), "w2": (2, 1)}),
                       ("layout", {"w1": (1, 2), "w2": (2, 1)})):
        for full, ref, gerr, lays in run_ranks(_worker, 2, mode):
            assert abs(full - ref) < 1e-3 * max(1.0, abs(ref)), (mode, full, ref)
            assert gerr < 1e-4, (mode, gerr)
            assert lays == want, (mode, lays)
