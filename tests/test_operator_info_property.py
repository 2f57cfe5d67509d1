"""Property test of the distributed operator semantics: for every primitive family, random legal shard strategies
on 4 or 8 virtual ranks must reproduce the unsharded operator - slices cut by the inferred input layouts, the local
operator run with localised shape arguments / attributes, the forward communication applied over the inferred rank
groups, outputs re-assembled with the inferred output layouts (``parallel.simulate.run_sharded``).
Reference tests of the same rules: tests/ut/python/parallel/test_{strided_slice,split,concat,tile,conv2d,batchnorm,
topk,cumsum,gather_v2,unsorted_segment_sum}.py and tests/ut/cpp/parallel/ops_info/*."""
import itertools
import random

import pytest
import torch

import mindspore_b200 as ms
from mindspore_b200 import ops
from mindspore_b200.parallel import operator_info as OI
from mindspore_b200.parallel.simulate import run_sharded


def _divs(n):
    return [d for d in range(1, n + 1) if n % d == 0]


def _splits(shape, device_num, frozen=()):
    """All ways to split ``shape`` (dims in ``frozen`` stay whole) using exactly or fewer than ``device_num``."""
    out = []
    for st in itertools.product(*[[1] if i in frozen else [d for d in _divs(device_num) if s % d == 0]
                                  for i, s in enumerate(shape)]):
        p = 1
        for s in st:
            p *= s
        if device_num % p == 0:
            out.append(tuple(st))
    return out


def _check(prim, args, strategy, device_num, out_strategy=None, tol=1e-4):
    want = prim._run(*args)
    want = list(want) if isinstance(want, (tuple, list)) else [want]
    got, info = run_sharded(prim, args, strategy, out_strategy, device_num)
    assert len(got) >= 1
    for g, w in zip(got, want):
        if isinstance(w, torch.Tensor) and isinstance(g, torch.Tensor):
            assert tuple(g.shape) == tuple(w.shape), (prim.name, strategy, g.shape, w.shape)
            torch.testing.assert_close(g.float(), w.float(), rtol=tol, atol=tol)
    return info


def _sample(cands, k, rng):
    cands = list(cands)
    rng.shuffle(cands)
    return cands[:k]


@pytest.mark.parametrize("device_num", [4, 8])
def test_array_ops_random_strategies(device_num):
    rng = random.Random(device_num)
    g = torch.Generator().manual_seed(0)
    x = torch.randn(8, 16, 24, generator=g)
    # StridedSlice: dim 1 is cut, dims 0 / 2 taken whole -> they may be split
    ss = ops.StridedSlice()
    for st in _sample(_splits(x.shape, device_num, frozen=(1,)), 6, rng):
        _check(ss, (x, (0, 2, 0), (8, 10, 24), (1, 2, 1)), (st,), device_num)
    with pytest.raises(OI.StrategyError):
        run_sharded(ss, (x, (0, 2, 0), (8, 10, 24), (1, 2, 1)), ((1, 2, 1),), device_num)
    sl = ops.Slice()
    for st in _sample(_splits(x.shape, device_num, frozen=(2,)), 4, rng):
        _check(sl, (x, (0, 0, 4), (8, -1, 8)), (st,), device_num)
    sp = ops.Split(axis=1, output_num=4)
    for st in _sample(_splits(x.shape, device_num, frozen=(1,)), 4, rng):
        info = _check(sp, (x,), (st,), device_num)
        assert len(info.outputs_tensor_map) == 4
    cat = ops.Concat(axis=2)
    y = torch.randn(8, 16, 8, generator=g)
    for st in _sample(_splits((8, 16), device_num), 4, rng):
        _check(cat, ((x, y),), (st + (1,), st + (1,)), device_num)
    stack = ops.Stack(axis=1)
    z = torch.randn(8, 16, 24, generator=g)
    for st in _sample(_splits(x.shape, device_num), 4, rng):
        info = _check(stack, ((x, z),), (st, st), device_num)
        assert info.outputs_tensor_map[0][1] == -1
    ex = ops.ExpandDims()
    for st in _sample(_splits(x.shape, device_num), 3, rng):
        _check(ex, (x, 1), (st,), device_num)
    sq = ops.Squeeze(axis=1)
    w = torch.randn(8, 1, 24, generator=g)
    for st in _sample(_splits(w.shape, device_num, frozen=(1,)), 3, rng):
        _check(sq, (w,), (st,), device_num)
    # Tile: strategy over the output dims; a split of a tiled dim divides the multiple
    tile = ops.Tile()
    t = torch.randn(8, 1, 6, generator=g)
    for st in [(2, 2, 1), (device_num, 1, 1), (1, device_num, 1), (2, device_num // 2, 1)]:
        _check(tile, (t, (1, device_num, 1)), (st,), device_num)
    bt = ops.BroadcastTo((4, 8, 16, 24))
    for st in _sample(_splits(x.shape, device_num), 3, rng):
        _check(bt, (x,), (st,), device_num)


@pytest.mark.parametrize("device_num", [4, 8])
def test_axis_bound_ops(device_num):
    rng = random.Random(100 + device_num)
    g = torch.Generator().manual_seed(1)
    x = torch.randn(8, 16, 32, generator=g)
    for st in _sample(_splits(x.shape, device_num, frozen=(2,)), 5, rng):
        _check(ops.TopK(), (x, 4), (st,), device_num)
        _check(ops.CumSum(), (x, 2), (st,), device_num)
        _check(ops.Sort(axis=-1), (x,), (st,), device_num)
        _check(ops.ArgMaxWithValue(axis=2), (x,), (st,), device_num)
    with pytest.raises(OI.StrategyError):
        run_sharded(ops.CumSum(), (x, 2), ((1, 1, 2),), device_num)
    idx = torch.randint(0, 16, (8, 5, 32), generator=g)
    for st in _sample(_splits((8, 1, 32), device_num, frozen=(1,)), 3, rng):
        _check(ops.GatherD(), (x, 1, idx), (st, st), device_num)
    # segment sum: id rows split -> partial sums all-reduced
    seg = torch.randint(0, 5, (8,), generator=g)
    for d0 in [d for d in _divs(device_num) if 8 % d == 0]:
        info = _check(ops.UnsortedSegmentSum(), (x, seg, 5), ((d0, 1, device_num // d0 if 32 % (device_num // d0) == 0 else 1),
                                                             (d0,)), device_num)
        assert (info.forward_comm is not None) == (d0 > 1)


@pytest.mark.parametrize("device_num", [4, 8])
def test_conv_bn_pool(device_num):
    g = torch.Generator().manual_seed(2)
    x = torch.randn(8, 8, 10, 10, generator=g)
    w = torch.randn(16, 8, 3, 3, generator=g) * 0.2
    conv = ops.Conv2D(16, 3, pad_mode="same")
    for sx, sw in [((device_num, 1, 1, 1), (1, 1, 1, 1)), ((1, 1, 1, 1), (device_num, 1, 1, 1)),
                   ((2, 1, 1, 1), (device_num // 2, 1, 1, 1)), ((1, device_num // 2, 1, 1), (2, device_num // 2, 1, 1)),
                   ((1, 2, 1, 1), (1, 2, 1, 1))]:
        info = _check(conv, (x, w), (sx, sw), device_num, tol=2e-4)
        assert (info.forward_comm is not None) == (sx[1] > 1)
    with pytest.raises(OI.StrategyError):
        run_sharded(conv, (x, w), ((1, 1, 2, 1), (1, 1, 1, 1)), device_num)
    scale, bias = torch.rand(8, generator=g) + 0.5, torch.randn(8, generator=g)
    bn = ops.BatchNorm(is_training=True)
    for st in [(device_num, 1, 1, 1), (1, device_num, 1, 1), (2, device_num // 2, 1, 1)]:
        mean, var = torch.zeros(8), torch.ones(8)
        want = torch.nn.functional.batch_norm(x, None, None, scale, bias, True, 0.1, 1e-5)
        got, info = run_sharded(bn, (x, scale, bias, mean, var), (st, (st[1],), (st[1],), (st[1],), (st[1],)), None,
                                device_num)
        torch.testing.assert_close(got[0], want, rtol=1e-4, atol=1e-4)
        assert info.needs_sync_stats() == (st[0] > 1)
    ba = ops.BiasAdd()
    for st in [(2, device_num // 2, 1, 1), (1, device_num, 1, 1)]:
        _check(ba, (x, bias), (st, (st[1],)), device_num)
    with pytest.raises(OI.StrategyError):
        run_sharded(ba, (x, bias), ((1, 2, 1, 1), (1,)), device_num)
    for st in [(device_num, 1, 1, 1), (2, device_num // 2, 1, 1)]:
        _check(ops.MaxPool(kernel_size=2, strides=2), (x,), (st,), device_num)
        _check(ops.AvgPool(kernel_size=2, strides=2), (x,), (st,), device_num)


@pytest.mark.parametrize("device_num", [4, 8])
def test_fused_decoder_primitives(device_num):
    g = torch.Generator().manual_seed(3)
    T, Hd = 64, 32
    x, r, gamma = torch.randn(T, Hd, generator=g), torch.randn(T, Hd, generator=g), torch.rand(Hd, generator=g) + 0.5
    _check(ops.AddRmsNorm(1e-5), (x, r, gamma), ((device_num, 1), (device_num, 1), (1,)), device_num)
    gu = torch.randn(T, 2 * 16 * device_num, generator=g)
    sw = ops.SwiGLU(groups=device_num)
    for st in [(1, device_num), (2, device_num // 2), (device_num, 1)]:
        _check(sw, (gu,), (st,), device_num)
    heads, d, seq = device_num, 16, 16
    qkv = torch.randn(2 * seq, 3 * heads * d, generator=g)
    ang = torch.outer(torch.arange(seq, dtype=torch.float32), 1.0 / (10000 ** (torch.arange(0, d, 2) / d)))
    att = ops.RotaryFlashAttention(heads, heads, d, groups=device_num)
    for st in [(1, device_num), (2, device_num // 2)]:
        _check(att, (qkv, ang.cos(), ang.sin()), (st, (1, 1), (1, 1)), device_num, tol=2e-4)
    # vocabulary-split embedding with reduce-scatter output, and the matmul pair of a transformer block
    table = torch.randn(8 * device_num, Hd, generator=g)
    ids = torch.randint(0, 8 * device_num, (T,), generator=g)
    info = _check(ops.Gather(), (table, ids, 0), ((device_num, 1), (1,)), device_num, out_strategy=((device_num, 1),))
    assert info.forward_comm[0] == "ReduceScatter"
    w = torch.randn(48, Hd, generator=g)
    _check(ops.MatMul(transpose_b=True), (x, w), ((1, 1), (device_num, 1)), device_num)
    w2 = torch.randn(Hd, 16 * device_num, generator=g)
    a = torch.randn(T, 16 * device_num, generator=g)
    info = _check(ops.MatMul(transpose_b=True), (a, w2), ((1, device_num), (1, device_num)), device_num,
                  out_strategy=((device_num, 1),), tol=1e-3)
    assert info.forward_comm[0] == "ReduceScatter"
