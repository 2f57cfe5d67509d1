"""Top-level helpers: sparse containers, Symbol, mutable / recompute / vmap / hessian, scipy routines, torch-style
optimizers and schedulers, boost."""
import numpy as np
import pytest
import torch

import mindspore_b200 as ms
from mindspore_b200 import nn


def test_sparse_containers():
    coo = ms.COOTensor([[0, 1], [1, 2], [0, 1]], [1.0, 2.0, 3.0], (2, 3))
    dense = coo.to_dense().numpy()
    assert dense.tolist() == [[0, 4, 0], [0, 0, 2]]
    csr = coo.to_csr()
    assert csr.indptr.tolist() == [0, 1, 2] and csr.indices.tolist() == [1, 2] and csr.values.tolist() == [4.0, 2.0]
    assert csr.to_dense().numpy().tolist() == dense.tolist()
    assert csr.mv(torch.tensor([1.0, 2.0, 3.0])).reshape(-1).tolist() == [8.0, 6.0]
    assert csr.mm(torch.eye(3)).numpy().tolist() == dense.tolist()
    assert (csr * 2.0).to_coo().to_dense().numpy().tolist() == (dense * 2).tolist()
    row = ms.RowTensor([0, 2, 0], torch.ones(3, 2), (3, 2))
    assert row.to_dense().numpy().tolist() == [[2, 2], [0, 0], [1, 1]]
    with pytest.raises(ValueError):
        ms.CSRTensor([0, 1], [0], [1.0], (3, 3))


def test_symbol_and_hints():
    s = ms.Symbol(max=64, min=8, divisor=8)
    assert s.admits(16) and not s.admits(12) and not s.admits(128)
    with pytest.raises(ValueError):
        ms.Symbol(divisor=4, remainder=4)
    m = ms.mutable((1, 2.0))
    assert isinstance(m[0], ms.Tensor) and float(m[1]) == 2.0
    with pytest.raises(TypeError):
        ms.mutable("text")

    @ms.jit_class
    class Cfg:
        pass
    assert Cfg.__ms_class__
    ms.set_algo_parameters(fully_use_devices=False)
    assert ms.get_algo_parameters("fully_use_devices") is False
    ms.reset_algo_parameters()
    assert ms.get_algo_parameters("fully_use_devices") is True
    with pytest.raises(ValueError):
        ms.set_algo_parameters(nonsense=1)


def test_recompute_vmap_hessian():
    net = nn.SequentialCell([nn.Dense(4, 8), nn.Tanh(), nn.Dense(8, 1)])
    x = ms.Tensor(torch.randn(3, 4)).requires_grad_(True)
    a = net(x).sum()
    a.backward()
    g_ref = [p.grad.clone() for p in net.trainable_params()]
    for p in net.trainable_params():
        p.grad = None
    ms.recompute(net, x).sum().backward()
    for p, g in zip(net.trainable_params(), g_ref):
        torch.testing.assert_close(p.grad, g)
    out = ms.vmap(lambda a, b: (a * b).sum(), (0, None))(ms.Tensor(torch.arange(6.0).reshape(3, 2)),
                                                         ms.Tensor(torch.tensor([1.0, 10.0])))
    assert out.tolist() == [10.0, 32.0, 54.0]
    h = ms.hessian(lambda v: (v ** 3).sum())(ms.Tensor(torch.tensor([1.0, 2.0])))
    np.testing.assert_allclose(np.asarray(h.detach().numpy()), np.diag([6.0, 12.0]), atol=1e-5)
    g = ms.Generator().manual_seed(5)
    assert g.initial_seed() == 5
    st = g.get_state()
    g.seed()
    g.set_state(st)
    assert g.initial_seed() == 5


def test_scipy_namespace():
    import mindspore_b200.scipy as sp
    torch.manual_seed(0)
    A = torch.randn(8, 8)
    A = A @ A.t() + 8 * torch.eye(8)
    b = torch.randn(8)
    for solver in (sp.sparse.linalg.cg, sp.sparse.linalg.bicgstab, sp.sparse.linalg.gmres):
        x, info = solver(A, b, tol=1e-6)
        assert info == 0 and float((A @ torch.as_tensor(x) - b).norm()) < 1e-4
    csr = ms.COOTensor(torch.nonzero(A), A[A != 0], (8, 8)).to_csr()
    x, info = sp.sparse.linalg.cg(csr, b, tol=1e-6)
    assert info == 0 and float((A @ torch.as_tensor(x) - b).norm()) < 1e-4
    c = sp.linalg.cho_factor(A, lower=True)
    assert float((A @ torch.as_tensor(sp.linalg.cho_solve(c, b)) - b).norm()) < 1e-4
    L = torch.tril(A)
    y = sp.linalg.solve_triangular(L, b, lower=True)
    assert float((L @ torch.as_tensor(y) - b).norm()) < 1e-4
    p, l, u = sp.linalg.lu(A)
    torch.testing.assert_close(torch.as_tensor(p) @ torch.as_tensor(l) @ torch.as_tensor(u), A, rtol=1e-4, atol=1e-4)
    assert sp.linalg.block_diag(torch.ones(2, 2), torch.ones(1, 3)).shape == (3, 5)

    def rosen(v):
        return 100 * (v[1] - v[0] ** 2) ** 2 + (1 - v[0]) ** 2
    for method in ("BFGS", "LBFGS"):
        r = sp.optimize.minimize(rosen, torch.tensor([-1.2, 1.0]), method=method, options={"maxiter": 300})
        assert r.success and np.allclose(r.x.numpy(), [1, 1], atol=1e-3)


def test_experimental_optim_and_schedulers():
    from mindspore_b200.experimental import optim
    ms.set_seed(0)
    net = nn.Dense(4, 2)
    ref = torch.nn.Linear(4, 2)
    with torch.no_grad():
        ref.weight.copy_(net.weight)
        ref.bias.copy_(net.bias)
    ours = optim.AdamW(net.trainable_params(), lr=0.1, weight_decay=0.05)
    theirs = torch.optim.AdamW(ref.parameters(), lr=0.1, weight_decay=0.05)
    sched = optim.lr_scheduler.MultiStepLR(ours, milestones=[2], gamma=0.1)
    tsched = torch.optim.lr_scheduler.MultiStepLR(theirs, milestones=[2], gamma=0.1)
    for i in range(4):
        grads = [torch.full_like(p, 0.1 * (i + 1)) for p in ref.parameters()]
        for p, g in zip(ref.parameters(), grads):
            p.grad = g.clone()
        theirs.step()
        tsched.step()
        ours(tuple(ms.Tensor(g) for g in grads))
        sched.step()
    torch.testing.assert_close(net.weight.detach().as_subclass(torch.Tensor), ref.weight.detach())
    assert ours.lrs == [g["lr"] for g in theirs.param_groups] and abs(ours.lrs[0] - 0.01) < 1e-12
    assert sched.get_last_lr() == tsched.get_last_lr()


def test_boost_less_bn_and_freeze():
    from mindspore_b200 import boost
    net = nn.SequentialCell([nn.Conv2d(1, 2, 3), nn.BatchNorm2d(2), nn.Conv2d(2, 2, 3), nn.BatchNorm2d(2),
                             nn.Conv2d(2, 2, 3), nn.BatchNorm2d(2), nn.Conv2d(2, 2, 3), nn.BatchNorm2d(2)])
    wrapped = boost.LessBN(net, keep=3)
    assert wrapped.frozen == 1
    opt = nn.SGD(net.trainable_params(), 0.1)
    fz = boost.FreezeOpt(opt, freeze_p=0.5, total_steps=2)
    n = len(net.trainable_params())
    before = [p.detach().clone() for p in net.trainable_params()]
    grads = tuple(ms.Tensor(torch.ones_like(p)) for p in net.trainable_params())
    fz(grads)                      # t = 0: nothing frozen
    fz(grads)                      # t = 1: a quarter frozen
    fz(grads)                      # t = 2: half frozen
    moved = [float((p.detach() - b).abs().max()) for p, b in zip(net.trainable_params(), before)]
    assert abs(moved[0] - 0.1) < 1e-6 and abs(moved[-1] - 0.3) < 1e-6
    assert fz.frozen_count() == n // 2
    ab = boost.AutoBoost("O1")
    assert ab.cfg["less_bn"] and ab.cfg["grad_freeze"] and not ab.cfg["adasum"]
    with pytest.raises(ValueError):
        boost.AutoBoost("O9")


def test_composite_functions():
    from mindspore_b200 import ops
    x = ms.Tensor(torch.tensor([[0, 1, 2], [0, 0, 3]]))
    assert ops.count_nonzero(x, axis=1).tolist() == [2, 1] and int(ops.count_nonzero(x)) == 3
    assert ops.sequence_mask(ms.Tensor(torch.tensor([1, 3])), 4).tolist() == [[True, False, False, False],
                                                                               [True, True, True, False]]
    a, b = torch.randn(2, 3, 4), torch.randn(5, 4, 6)
    np.testing.assert_allclose(ops.dot(ms.Tensor(a), ms.Tensor(b)).numpy(), np.dot(a.numpy(), b.numpy()), rtol=1e-5,
                               atol=1e-5)
    assert ops.repeat_elements(ms.Tensor(torch.tensor([1, 2])), 2).tolist() == [1, 1, 2, 2]
    assert ops.ZipOperation()((1, 2), (3, 4)) == ((1, 3), (2, 4))
    assert ops.UnpackCall()(lambda p, q, r=0: p + q + r, (1, 2), {"r": 3}) == 6
    assert torch.equal(ops.poisson((4,), 3.0, seed=2), ops.poisson((4,), 3.0, seed=2))
    g = ops.gamma((2000,), 3.0, 2.0, seed=0)
    assert abs(float(g.mean()) - 1.5) < 0.1
    lp = ops.laplace((4000,), 1.0, 2.0, seed=0)
    assert abs(float(lp.mean()) - 1.0) < 0.2 and abs(float(lp.std()) - 2 * 2 ** 0.5) < 0.3
    idx, mask = ops.choice_with_mask(ms.Tensor(torch.tensor([1, 0, 1, 1])), 4, seed=0)
    assert mask.tolist() == [True, True, True, False] and sorted(idx[:3, 0].tolist()) == [0, 2, 3]


def test_mindspore_only_tensor_methods():
    t = ms.Tensor(torch.tensor([[1., 5., 3.], [4., 2., 6.]]))
    assert t.ptp(1).tolist() == [4.0, 4.0] and float(t.ptp()) == 5.0
    assert float(t.itemset((0, 1), 9.0)[0, 1]) == 9.0 and float(t[0, 1]) == 5.0
    assert t.gather_nd(ms.Tensor(torch.tensor([[0, 1], [1, 2]]))).tolist() == [5.0, 6.0]
    a = ms.Tensor(torch.tensor([1, 3, 5]))
    assert a.searchsorted(ms.Tensor(torch.tensor([0, 3, 6]))).tolist() == [0, 1, 3]
    assert a.searchsorted(ms.Tensor(torch.tensor([0, 3, 6])), side="right").tolist() == [0, 2, 3]
    ch = [ms.Tensor(torch.tensor(v)) for v in ([1, 2, 3], [4, 5, 6], [7, 8, 9])]
    assert ms.Tensor(torch.tensor([2, 0, 1])).choose(ch).tolist() == [7, 2, 6]
    assert float(t.scatter_mul(ms.Tensor(torch.tensor([[0, 0]])), ms.Tensor(torch.tensor([10.0])))[0, 0]) == 10.0
    u, idx = ms.Tensor(torch.tensor([3, 1, 3, 2])).unique_with_pad(0)
    assert u.tolist() == [3, 1, 2, 0] and idx.tolist() == [0, 1, 0, 2]
    assert ms.Tensor(torch.tensor([0, 2])).one_hot(3).tolist() == [[1, 0, 0], [0, 0, 1]]
    assert t.unsorted_segment_sum(ms.Tensor(torch.tensor([0, 0])), 2).tolist() == [[5.0, 7.0, 9.0], [0.0, 0.0, 0.0]]
    assert t.to_csr().to_dense().tolist() == t.tolist() and t.to_coo().size == 6
    assert ms.Tensor.from_numpy(np.arange(3)).tolist() == [0, 1, 2]
    assert len(t.get_bytes()) == 24 and t.fills(2.0).tolist() == [[2.0] * 3] * 2
    assert ms.Tensor(torch.tensor([0.1, 2.5, 7.0])).bucketize([1.0, 3.0]).tolist() == [0, 1, 2]
    with pytest.raises(ValueError):
        t.move_to("TPU")


def test_mint_namespace():
    import mindspore_b200.mint as mint
    out = mint.addmm(torch.ones(2, 2), torch.ones(2, 3), torch.ones(3, 2))
    assert isinstance(out, ms.Tensor) and out.tolist() == [[4.0, 4.0], [4.0, 4.0]]
    assert mint.randn(2, 3).shape == (2, 3) and mint.transpose(ms.Tensor(torch.ones(2, 3)), 0, 1).shape == (3, 2)
    assert float(mint.special.erfc(torch.tensor(0.0))) == 1.0 and float(mint.linalg.det(torch.eye(3))) == 1.0
    for name in ("all_reduce", "barrier", "get_rank", "get_world_size", "init_process_group", "new_group"):
        assert hasattr(mint.distributed, name)
    assert mint.nn.functional.relu(torch.tensor([-1.0, 1.0])).tolist() == [0.0, 1.0]
    layer = mint.nn.Linear(3, 2)
    assert layer(ms.Tensor(torch.ones(4, 3))).shape == (4, 2)
    opt = mint.optim.AdamW(layer.trainable_params(), 1e-3)
    assert opt is not None and mint.nn.Fold is not None and mint.nn.Unfold is not None


def test_numpy_namespace_wide_coverage():
    import mindspore_b200.numpy as mnp
    x = ms.Tensor(torch.tensor([[1., float("nan"), 3.], [4., 5., 6.]]))
    assert float(mnp.nanmax(x)) == 6.0 and mnp.nansum(x, axis=1).tolist() == [4.0, 15.0]
    assert mnp.percentile(ms.Tensor(torch.arange(5.)), 50) == 2.0
    assert mnp.interp(ms.Tensor(torch.tensor([1.5])), ms.Tensor(torch.tensor([1., 2.])),
                      ms.Tensor(torch.tensor([10., 20.]))).tolist() == [15.0]
    hist, edges = mnp.histogram(ms.Tensor(torch.tensor([1., 2., 2., 3.])), bins=3)
    assert hist.tolist() == [1, 2, 1] and len(edges) == 4
    assert mnp.polyval([1, 2, 3], ms.Tensor(torch.tensor([2.]))).tolist() == [11.0]
    c = mnp.cbrt(ms.Tensor(torch.tensor([27., -8.])))
    assert isinstance(c, ms.Tensor) and np.allclose(c.numpy(), [3, -2], atol=1e-5)
    assert float(mnp.average(ms.Tensor(torch.tensor([1., 3.])), weights=ms.Tensor(torch.tensor([3., 1.])))) == 1.5
    a = ms.Tensor(torch.arange(6.).reshape(2, 3))
    assert mnp.flip(a, 0).tolist() == [[3, 4, 5], [0, 1, 2]] and mnp.vstack([a, a]).shape == (4, 3)
    assert mnp.take_along_axis(a, ms.Tensor(torch.tensor([[2], [0]])), 1).tolist() == [[2.0], [3.0]]
    q, r = mnp.divmod(ms.Tensor(torch.tensor([7, -7])), ms.Tensor(torch.tensor([2, 2])))
    assert q.tolist() == [3, -4] and r.tolist() == [1, 1]
    assert mnp.unravel_index(5, (2, 3)) == (1, 2) and np.allclose(mnp.hanning(4).numpy(), np.hanning(4))
    assert mnp.array_equal(a, a) and not mnp.array_equal(a, a + 1)


def test_map_parameter_custom_registration_and_reshard():
    import numpy as np
    import torch
    import mindspore_b200 as ms
    from mindspore_b200 import ops
    from mindspore_b200.experimental import MapParameter
    from mindspore_b200.parallel import Layout
    m = MapParameter(key_dtype=ms.int32, value_dtype=ms.float32, value_shape=(3,), default_value="zeros")
    m.put(ms.Tensor(torch.tensor([5, 9])), ms.Tensor(torch.tensor([[1., 2., 3.], [4., 5., 6.]])))
    got = m.get(ms.Tensor(torch.tensor([9, 7, 5])))
    assert got.tolist() == [[4., 5., 6.], [0., 0., 0.], [1., 2., 3.]] and len(m) == 3      # 7 was inserted
    m.scatter_update(ms.Tensor(torch.tensor([5, 5])), ms.Tensor(torch.ones(2, 3)), lr=0.5)
    assert m[ms.Tensor(torch.tensor([5]))].tolist() == [[0., 1., 2.]]
    m.erase(ms.Tensor(torch.tensor([7])))
    keys, values, status = m.export_data()
    assert keys.tolist() == [5, 9] and values.shape == (2, 3) and status.shape == (2,)
    m2 = MapParameter(value_shape=(3,)).import_data((keys, values))
    assert np.allclose(m2.get_values().numpy(), values)
    # registration records of a custom operator
    info = (ops.CustomRegOp("axpy").input(0, "x").input(1, "y").output(0, "z").attr("alpha", "required", "float")
            .dtype_format(ops.DataType.F32_Default, ops.DataType.F32_Default, ops.DataType.F32_Default)
            .target("GPU").get_op_info())
    assert info["op_name"] == "axpy" and len(info["inputs"]) == 2 and info["dtype_format"][0][0] == ("float32", "DefaultFormat")

    @ops.custom_info_register(info)
    def axpy(x, y):
        return x + y
    assert axpy.reg_info[0]["target"] == "GPU" and float(axpy(1.0, 2.0)) == 3.0
    assert ops.get_vm_impl_fn(ops.ReLU()) is not None
    # reshard outside a parallel mode is the identity; the layout is still checked against the tensor
    lay = Layout((2, 2), ("dp", "mp"))
    x = ms.Tensor(torch.randn(4, 6))
    assert ops.reshard(x, lay("dp", "None")) is x
    import pytest
    with pytest.raises(ValueError):
        ops.reshard(x, lay("dp", "None", "mp"))
    with pytest.raises(TypeError):
        ops.reshard(x, "dp")
