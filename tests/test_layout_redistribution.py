"""Layout algebra and redistribution inference (native C++), checked against brute-force NumPy slicing and the
operator sequences the reference's tensor_redistribution tests expect."""
import numpy as np
import pytest

from mindspore_b200.parallel import redistribution as RD
from mindspore_b200.parallel.layout import Layout, TensorLayout, assemble_full, ranks_along_dims, slice_for_rank


def test_layout_class_and_errors():
    lay = Layout((2, 4), ("dp", "mp"))
    d = lay("dp", "None").to_dict()
    assert d["device_matrix"] == (2, 4) and d["tensor_map"] == (1, -1)
    assert lay(("dp", "mp"), "None").to_dict()["tensor_map"] == ((1, 0), -1)
    with pytest.raises(ValueError):
        lay("dp", "dp")
    with pytest.raises(ValueError):
        lay("xx")
    with pytest.raises(ValueError):
        Layout((2, 2), ("a", "a"))
    with pytest.raises(ValueError):
        Layout((2, 2), ("interleaved_parallel", "a"))


def test_slice_index_matches_manual():
    lay = TensorLayout((2, 4), (1, 0), (8, 8))         # dim0 over the left axis (2), dim1 over the right axis (4)
    assert lay.slice_shape() == (4, 2)
    full = np.arange(64).reshape(8, 8)
    for rank in range(8):
        r, c = rank // 4, rank % 4
        np.testing.assert_array_equal(slice_for_rank(full, lay, rank), full[r * 4:(r + 1) * 4, c * 2:(c + 1) * 2])
    rep = TensorLayout((2, 4), (-1, 0), (8, 8))
    assert rep.repeat_num() == 2 and rep.replica_group(5) == [1, 5]


def test_group_ranks_native_matches_python():
    dm = (2, 2, 4)
    for rank in range(16):
        for dims in ([0], [1], [2], [0, 2], [0, 1, 2]):
            assert RD.group_ranks(dm, rank, dims) == ranks_along_dims(dm, rank, dims)
    assert RD.group_ranks((2, 4), 1, [1], base_rank=8) == [9, 13]


@pytest.mark.parametrize("src_map,dst_map,expect", [
    ((1, -1), (-1, -1), ["AllGather"]),
    ((-1, -1), (1, 0), ["StridedSlice", "StridedSlice"]),
    ((1, -1), (-1, 1), ["AllGather", "StridedSlice"]),
    ((-1, 0), (-1, -1), ["AllGather", "Split", "Concat"]),
    ((1, 0), (0, 1), None),
])
def test_redistribution_sequences_and_values(src_map, dst_map, expect):
    dm, shape = (2, 4), (8, 16)
    src, dst = TensorLayout(dm, src_map, shape), TensorLayout(dm, dst_map, shape)
    ops = RD.infer(src, dst, enable_alltoall=False)
    if expect is not None:
        assert RD.lowered_names(ops) == expect
    full = np.random.RandomState(0).randn(*shape)
    slices = {r: np.ascontiguousarray(slice_for_rank(full, src, r)) for r in range(8)}
    out = RD.apply_virtual(slices, src, dst)
    for r in range(8):
        np.testing.assert_array_equal(out[r], slice_for_rank(full, dst, r))
    np.testing.assert_array_equal(assemble_full(out, dst), full)


def test_alltoall_used_when_enabled_and_cheaper():
    dm, shape = (8,), (16, 16)
    src, dst = TensorLayout(dm, (0, -1), shape), TensorLayout(dm, (-1, 0), shape)
    a2a = RD.infer(src, dst, enable_alltoall=True)
    plain = RD.infer(src, dst, enable_alltoall=False)
    assert [o.name for o in a2a] == ["AlltoAll"] and [o.name for o in plain] == ["AllGather", "StridedSlice"]
    assert RD.cost(a2a, 32) < RD.cost(plain, 32) * 2


def test_different_device_matrices_fall_back_to_gather_slice():
    src, dst = TensorLayout((2, 4), (1, -1), (8, 8)), TensorLayout((4, 2), (1, 0), (8, 8))
    assert RD.infer(src, dst) is None
    full = np.arange(64.0).reshape(8, 8)
    out = RD.apply_virtual({r: slice_for_rank(full, src, r) for r in range(8)}, src, dst)
    for r in range(8):
        np.testing.assert_array_equal(out[r], slice_for_rank(full, dst, r))


def test_random_layout_pairs_property():
    rng = np.random.RandomState(1)
    dm, shape = (2, 2, 2), (8, 8, 8)
    for _ in range(40):
        def rand_map():
            dims = list(rng.permutation(3))
            return tuple(int(dims.pop()) if rng.rand() < 0.6 and dims else -1 for _ in range(3))
        src, dst = TensorLayout(dm, rand_map(), shape), TensorLayout(dm, rand_map(), shape)
        full = rng.randn(*shape)
        out = RD.apply_virtual({r: np.ascontiguousarray(slice_for_rank(full, src, r)) for r in range(8)}, src, dst)
        for r in range(8):
            np.testing.assert_array_equal(out[r], slice_for_rank(full, dst, r))
