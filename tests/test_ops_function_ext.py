"""The wider functional API: values against numpy / torch formulas, and the name coverage of the reference's
``ops.function`` modules."""
import math

import numpy as np
import pytest
import torch

import mindspore_b200 as ms
from mindspore_b200 import ops

T = lambda *a, **k: ms.Tensor(torch.tensor(*a, **k))
N = lambda t: t.detach().as_subclass(torch.Tensor).numpy()


def test_array_functions():
    x = T(np.arange(12, dtype=np.float32).reshape(3, 4))
    assert N(ops.matrix_band_part(T(np.ones((4, 4), np.float32)), 1, 0)).sum() == 7
    assert N(ops.mirror_pad(x, [[1, 1], [2, 0]], "REFLECT")).tolist()[0] == [6, 5, 4, 5, 6, 7]
    assert N(ops.mirror_pad(x, [[0, 0], [1, 1]], "SYMMETRIC")).tolist()[0] == [0, 0, 1, 2, 3, 3]
    sb = ops.space_to_batch_nd(T(np.arange(16, dtype=np.float32).reshape(1, 1, 4, 4)), [2, 2], [[0, 0], [0, 0]])
    assert sb.shape == (4, 1, 2, 2) and N(sb)[1].reshape(-1).tolist() == [1, 3, 9, 11]
    back = ops.batch_to_space_nd(sb, [2, 2], [[0, 0], [0, 0]])
    assert N(back).reshape(-1).tolist() == list(range(16))
    np.testing.assert_array_equal(N(ops.unsorted_segment_max(x, T([0, 1, 0]), 2)), [[8, 9, 10, 11], [4, 5, 6, 7]])
    np.testing.assert_array_equal(N(ops.unsorted_segment_prod(T([1., 2., 3.]), T([0, 0, 1]), 2)), [2, 3])
    np.testing.assert_array_equal(N(ops.scatter_nd_add(T(np.zeros(4, np.float32)), T([[1], [1], [3]]),
                                                       T([1., 2., 3.]))), [0, 3, 0, 3])
    np.testing.assert_array_equal(N(ops.tensor_scatter_max(T(np.zeros((2, 2), np.float32)), T([[0, 0], [0, 0]]),
                                                           T([1., 5.]))), [[5, 0], [0, 0]])
    np.testing.assert_array_equal(N(ops.tensor_scatter_elements(T(np.zeros((2, 3), np.float32)), T([[0, 2]]),
                                                                T([[7., 8.]]), axis=1, reduction="add")),
                                  [[7, 0, 8], [0, 0, 0]])
    v, i = ops.top_k(x, 2)
    assert N(v)[0].tolist() == [3, 2] and i.dtype == torch.int32
    y, idx = ops.unique_with_pad(T([1, 1, 5, 5, 4]), 0)
    assert N(y).tolist() == [1, 5, 4, 0, 0] and N(idx).tolist() == [0, 0, 1, 1, 2]
    assert N(ops.reverse_sequence(T([[1, 2, 3], [4, 5, 6]]), T([2, 3]), seq_dim=1)).tolist() == [[2, 1, 3], [6, 5, 4]]
    assert N(ops.population_count(T([7, 8], dtype=torch.int16))).tolist() == [3, 1]
    assert ops.is_nonzero(T([0.5])) and not ops.is_nonzero(T([0]))
    with pytest.raises(ValueError):
        ops.is_nonzero(T([1, 2]))
    assert ops.tensor_slice(x, (1, 1), (2, -1)).shape == (2, 3)
    assert N(ops.matrix_diag(T([1., 2.]), k=1)).tolist() == [[0, 1, 0], [0, 0, 2], [0, 0, 0]]
    assert ops.col2im(T(np.ones((1, 2, 4, 9), np.float32)), [4, 4], [2, 2], [1, 1], [0, 0], [1, 1]).shape == (1, 2, 4, 4)


def test_math_linalg_fft_windows():
    a = T([[4., 1.], [1., 3.]])
    np.testing.assert_allclose(N(ops.cholesky(a)) @ N(ops.cholesky(a)).T, N(a), rtol=1e-6)
    s, u, v = ops.svd(T(np.random.RandomState(0).randn(4, 3).astype(np.float32)))
    assert s.shape == (3,) and u.shape == (4, 3) and v.shape == (3, 3)
    sign, logdet = ops.log_matrix_determinant(a)
    assert float(sign) == 1 and abs(float(logdet) - math.log(11)) < 1e-5
    np.testing.assert_allclose(N(ops.matrix_solve(a, T([[1.], [2.]]))), np.linalg.solve(N(a), [[1.], [2.]]), rtol=1e-5)
    np.testing.assert_allclose(N(ops.pinv(a)), np.linalg.inv(N(a)), rtol=1e-4)
    x = np.random.RandomState(1).randn(8).astype(np.float32)
    np.testing.assert_allclose(N(ops.fft(T(x))), np.fft.fft(x), rtol=1e-4, atol=1e-5)
    np.testing.assert_allclose(N(ops.irfft(ops.rfft(T(x)))), x, rtol=1e-4, atol=1e-5)
    np.testing.assert_allclose(N(ops.hann_window(6, periodic=False)), np.hanning(6), atol=1e-6)
    np.testing.assert_allclose(N(ops.bartlett_window(5, periodic=False)), np.bartlett(5), atol=1e-6)
    np.testing.assert_allclose(N(ops.floordiv(T([7., -7.]), 2)), [3, -4])
    np.testing.assert_allclose(N(ops.truncate_div(T([7., -7.]), 2)), [3, -3])
    np.testing.assert_allclose(N(ops.truncate_mod(T([7., -7.]), 3)), [1, -1])
    np.testing.assert_allclose(N(ops.logspace(0, 2, 3)), [1, 10, 100])
    np.testing.assert_allclose(N(ops.iou(T([[0., 0, 9, 9]]), T([[0., 0, 4, 9]]))), [[0.5]])
    np.testing.assert_allclose(N(ops.bessel_i0(T([0., 1.]))), [1.0, 1.2660659], rtol=1e-5)
    np.testing.assert_allclose(float(N(ops.clip_by_norm(T(np.full(4, 3., np.float32)), 1.0) ** 2).sum()) ** 0.5, 1.0,
                               rtol=1e-4)
    a2, b2 = ops.clip_by_norm([T([3., 0.]), T([0., 4.])], 1.0)
    np.testing.assert_allclose(N(a2), [0.6, 0], rtol=1e-4)
    assert ops.cov(T(np.random.RandomState(2).randn(3, 10).astype(np.float32))).shape == (3, 3)
    np.testing.assert_allclose(N(ops.sparse_segment_mean(T([[1., 2.], [3., 4.], [5., 6.]]), T([0, 2]), T([0, 0]))),
                               [[3, 4]])


def test_nn_functions():
    x = T(np.random.RandomState(3).randn(2, 3, 10).astype(np.float32))
    w = T(np.random.RandomState(4).randn(4, 3, 3).astype(np.float32))
    assert ops.conv1d(x, w, pad_mode="same").shape == (2, 4, 10)
    assert ops.conv1d(x, w, pad_mode="valid", stride=2).shape == (2, 4, 4)
    np.testing.assert_allclose(N(ops.conv1d(x, w, pad_mode="pad", padding=1)),
                               torch.nn.functional.conv1d(torch.tensor(N(x)), torch.tensor(N(w)), padding=1).numpy(),
                               rtol=1e-5, atol=1e-5)
    assert ops.conv3d(T(np.ones((1, 2, 4, 4, 4), np.float32)), T(np.ones((3, 2, 3, 3, 3), np.float32)),
                      pad_mode="same").shape == (1, 3, 4, 4, 4)
    assert N(ops.intopk(T([[0.1, 0.9, 0.0], [0.3, 0.2, 0.5]]), T([1, 1]), 1)).tolist() == [True, False]
    np.testing.assert_allclose(N(ops.bias_add(T(np.zeros((1, 2, 3), np.float32)), T([1., 2.])))[0, :, 0], [1, 2])
    assert ops.pixel_unshuffle(ops.pixel_shuffle(T(np.ones((1, 8, 2, 2), np.float32)), 2), 2).shape == (1, 8, 2, 2)
    np.testing.assert_allclose(N(ops.softmin(T([1., 2.]))), torch.softmax(torch.tensor([-1., -2.]), 0).numpy(),
                               rtol=1e-6)
    np.testing.assert_allclose(float(ops.huber_loss(T([0., 3.]), T([0., 0.]), delta=1.0)), 1.25)
    np.testing.assert_allclose(float(ops.margin_ranking_loss(T([1.]), T([2.]), T([1.]), margin=0.5)), 1.5)
    out, idx = ops.max_pool3d(T(np.arange(8, dtype=np.float32).reshape(1, 1, 2, 2, 2)), 2, return_indices=True)
    assert float(out) == 7 and ops.max_unpool3d(out, idx, 2).shape == (1, 1, 2, 2, 2)
    ind, vals, shp, neg = ops.ctc_greedy_decoder(T(np.log(np.array(
        [[[0.6, 0.3, 0.1]], [[0.6, 0.3, 0.1]], [[0.1, 0.1, 0.8]], [[0.1, 0.8, 0.1]]], np.float32))), T([4]))
    assert N(vals).tolist() == [0, 1] and N(shp).tolist() == [1, 2]
    # deformable convolution with zero offsets and unit masks is a plain convolution
    xi = T(np.random.RandomState(5).randn(1, 2, 6, 6).astype(np.float32))
    wi = T(np.random.RandomState(6).randn(3, 2, 3, 3).astype(np.float32))
    off = torch.zeros(1, 3 * 9, 4, 4)
    off[:, 18:] = 1.0
    got = ops.deformable_conv2d(xi, wi, ms.Tensor(off), (3, 3), (1, 1, 1, 1), (0, 0, 0, 0))
    np.testing.assert_allclose(N(got), torch.nn.functional.conv2d(torch.tensor(N(xi)), torch.tensor(N(wi))).numpy(),
                               rtol=1e-4, atol=1e-4)


def test_image_and_random_functions():
    anchors = T([[10., 10, 29, 29]])
    gt = T([[12., 14, 33, 31]])
    enc = ops.bounding_box_encode(anchors, gt)
    dec = ops.bounding_box_decode(anchors, enc, max_shape=(100, 100))
    np.testing.assert_allclose(N(dec), N(gt), atol=1e-3)
    assert N(ops.check_valid(T([[0., 0, 5, 5], [0, 0, 50, 5]]), T([10., 10, 1.0]))).tolist() == [True, False]
    img = T(np.arange(16, dtype=np.float32).reshape(1, 4, 4, 1))
    crop = ops.crop_and_resize(img, T([[0., 0., 1., 1.]]), T([0]), (4, 4))
    np.testing.assert_allclose(N(crop), N(img), atol=1e-5)
    s, t_e, s_e = ops.uniform_candidate_sampler(T([[1, 3]]), 2, 4, True, 10, seed=7)
    assert len(set(N(s).tolist())) == 4 and t_e.shape == (1, 2) and s_e.shape == (4,)
    assert ops.random_poisson((3,), T([2., 5.]), seed=1).shape == (3, 2)
    assert ops.random_gamma((3,), T([2., 5.]), seed=1).shape == (3, 2)
    assert ops.standard_laplace((100,), seed=3).shape == (100,)
    assert ops.random_categorical(T([[0., 0., 9.]]), 5, seed=2).shape == (1, 5)
    assert ops.multinomial_with_replacement(T([[0.1, 0.9]]), 1, 0, 4, True).shape == (1, 4)


def test_sparse_functions():
    d = torch.tensor([[0., 2., 0.], [3., 0., 4.]])
    coo, csr = ops.dense_to_sparse_coo(ms.Tensor(d)), ops.dense_to_sparse_csr(ms.Tensor(d))
    np.testing.assert_allclose(N(ops.csr_to_dense(ops.csr_sqrt(csr))), d.sqrt().numpy())
    np.testing.assert_allclose(N(ops.coo_neg(coo).to_dense()), -d.numpy())
    np.testing.assert_allclose(N(ops.csr_softmax(csr).values), [1, 1 / (1 + math.e), math.e / (1 + math.e)], rtol=1e-5)
    np.testing.assert_allclose(N(ops.csr_mm(csr, ms.Tensor(torch.ones(3, 2)))), [[2, 2], [7, 7]])
    np.testing.assert_allclose(N(ops.csr_mv(csr, ms.Tensor(torch.ones(3, 1)))), [[2], [7]])
    np.testing.assert_allclose(N(ops.csr_add(csr, csr, 1.0, 2.0).to_dense()), 3 * d.numpy())
    np.testing.assert_allclose(N(ops.csr_div(csr, 2.0).to_dense()), d.numpy() / 2)
    np.testing.assert_allclose(N(ops.csr_gather(csr.indptr, csr.indices, ms.Tensor(d + 1), csr.shape)), [3, 4, 5])
    assert ops.coo_concat([coo, coo], 0).shape == (4, 3)
    assert N(ops.coo2csr(T([0, 1, 1]), 2)).tolist() == [0, 1, 3] and N(ops.csr2coo(csr.indptr, 3)).tolist() == [0, 1, 1]
    assert ops.csr_tensor_get_dense_shape(csr) == (2, 3) and ops.coo_tensor_get_values(coo).shape == (3,)
    i, v, s = ops.coalesce(T([[0, 0], [1, 1]]), T([1., 2.]), (2, 2))
    assert N(v).tolist() == [3] and N(i).tolist() == [[0], [1]]
    row = ops.make_row_tensor(T([0, 2]), T([[1., 1.], [2., 2.]]), (3, 2))
    np.testing.assert_allclose(N(ops.row_tensor_add(row, ms.Tensor(torch.ones(3, 2)))), [[2, 2], [1, 1], [3, 3]])
    with pytest.raises(TypeError):
        ops.csr_abs(coo)


# the public names (``__all__``) of the reference's ops/function/*.py modules
_FUNCTION_NAMES = """
abs absolute accumulate_n acos acosh adaptive_avg_pool1d adaptive_avg_pool2d adaptive_avg_pool3d adaptive_max_pool1d
adaptive_max_pool2d adaptive_max_pool3d add addbmm addcdiv addcmul addmm addmv addn addr adjoint affine_grid all
amax amin aminmax angle any approximate_equal arange arccos arccosh arcsin arcsinh arctan arctan2 arctanh argmax
argmin argsort argwhere asin asinh assign assign_add assign_sub atan atan2 atanh atleast_1d atleast_2d atleast_3d
avg_pool1d avg_pool2d avg_pool3d baddbmm bartlett_window batch_dot batch_norm batch_to_space_nd bernoulli bessel_i0
bessel_i0e bessel_i1 bessel_i1e bessel_j0 bessel_j1 bessel_k0 bessel_k0e bessel_k1 bessel_k1e bessel_y0 bessel_y1
bias_add bidense binary_cross_entropy binary_cross_entropy_with_logits bincount bitwise_and bitwise_left_shift
bitwise_or bitwise_right_shift bitwise_xor blackman_window block_diag bmm bounding_box_decode bounding_box_encode
broadcast_to bucketize cartesian_prod cat cdist ceil celu channel_shuffle check_valid choice_with_mask cholesky
cholesky_inverse cholesky_solve chunk clamp clip clip_by_global_norm clip_by_norm clip_by_value coalesce col2im
column_stack combinations concat cond conj conv1d conv2d conv3d conv3d_transpose conv_transpose2d coo2csr coo_abs
coo_acos coo_acosh coo_add coo_asin coo_asinh coo_atan coo_atanh coo_ceil coo_concat coo_cos coo_cosh coo_exp
coo_expm1 coo_floor coo_inv coo_isfinite coo_isinf coo_isnan coo_log coo_log1p coo_neg coo_relu coo_relu6 coo_round
coo_sigmoid coo_sin coo_sinh coo_softsign coo_sqrt coo_square coo_tan coo_tanh coo_tensor_get_dense_shape
coo_tensor_get_indices coo_tensor_get_values copysign cos cosh cosine_embedding_loss cosine_similarity count_nonzero
cov crop_and_resize cross cross_entropy csr2coo csr_abs csr_acos csr_acosh csr_add csr_asin csr_asinh csr_atan
csr_atanh csr_ceil csr_cos csr_cosh csr_div csr_exp csr_expm1 csr_floor csr_gather csr_inv csr_isfinite csr_isinf
csr_isnan csr_log csr_log1p csr_mm csr_mul csr_mv csr_neg csr_reduce_sum csr_relu csr_relu6 csr_round csr_sigmoid
csr_sin csr_sinh csr_softmax csr_softsign csr_sqrt csr_square csr_tan csr_tanh csr_tensor_get_dense_shape
csr_tensor_get_indices csr_tensor_get_indptr csr_tensor_get_values csr_to_coo csr_to_dense ctc_greedy_decoder
ctc_loss cummax cummin cumprod cumsum deepcopy deformable_conv2d deg2rad dense dense_to_sparse_coo
dense_to_sparse_csr depend det diag diag_embed diagflat diagonal diagonal_scatter diff digamma dist div divide dot
dropout dropout1d dropout2d dropout3d dsplit dstack dyn_shape eig eigvals einsum elu embedding eps eq equal erf erfc
erfinv exp exp2 expand expand_dims expm1 eye fast_gelu fft fft2 fftn fftshift fill fills flatten flip fliplr flipud
float_power floor floor_div floor_divide floor_mod floordiv floormod fmax fmin fmod fold frac fractional_max_pool2d
fractional_max_pool3d full full_like gamma gather gather_d gather_elements gather_nd gaussian_nll_loss gcd ge gelu
geqrf ger glu greater greater_equal grid_sample group_norm gt gumbel_softmax hamming_window hann_window hardshrink
hardsigmoid hardswish hardtanh heaviside hinge_embedding_loss histc hsplit hstack huber_loss hypot i0 ifft ifft2
ifftn ifftshift igamma igammac imag index_add index_fill index_select inner inplace_add inplace_index_add
inplace_sub inplace_update interpolate intopk inv inverse invert iou irfft is_complex is_floating_point is_nonzero
is_tensor isclose isfinite isinf isnan isneginf isposinf isreal kaiser_window kl_div kron l1_loss laplace layer_norm
lcm ldexp le leaky_relu lerp less less_equal lgamma linspace log log10 log1p log2 log_matrix_determinant log_softmax
log_uniform_candidate_sampler logaddexp logaddexp2 logcumsumexp logdet logical_and logical_not logical_or
logical_xor logit logsigmoid logspace logsumexp lp_pool1d lp_pool2d lrn lstsq lt lu_solve lu_unpack make_coo_tensor
make_csr_tensor make_map_parameter make_row_tensor make_row_tensor_inner make_sparse_tensor margin_ranking_loss
masked_fill masked_select matmul matrix_band_part matrix_determinant matrix_diag matrix_diag_part matrix_exp
matrix_norm matrix_power matrix_set_diag matrix_solve max max_pool2d max_pool3d max_unpool1d max_unpool2d
max_unpool3d maximum mean median meshgrid min minimum mirror_pad mish moveaxis movedim mse_loss msort mul
multi_margin_loss multilabel_margin_loss multilabel_soft_margin_loss multinomial multinomial_with_replacement
multiply mv mvlgamma nan_to_num nanmean nanmedian nanquantile nansum narrow ne neg negative nextafter nll_loss
nonzero norm normal not_equal numel one_hot ones ones_like orgqr ormqr outer pad padding partial pdist permute pinv
pixel_shuffle pixel_unshuffle poisson polar polygamma population_count positive pow pows prelu print_ prod qr
quantile rad2deg rand rand_like randint randint_like randn randn_like random_categorical random_gamma random_poisson
randperm range rank ravel real reciprocal relu relu6 remainder renorm repeat_elements repeat_interleave reshape
reshape_ reshard reverse reverse_sequence rfft rms_norm roll rot90 round row_stack row_tensor_add
row_tensor_get_dense_shape row_tensor_get_indices row_tensor_get_values rrelu rsqrt scalar_cast scalar_to_array
scalar_to_tensor scatter scatter_add scatter_div scatter_max scatter_min scatter_mul scatter_nd scatter_nd_add
scatter_nd_div scatter_nd_max scatter_nd_min scatter_nd_mul scatter_nd_sub scatter_update searchsorted select
select_scatter selu sequence_mask sgn shape shape_ shuffle sigmoid sign signbit silu sin sinc sinh size slice
slice_scatter slogdet smooth_l1_loss soft_margin_loss soft_shrink softmax softmin softplus softshrink softsign sort
space_to_batch_nd sparse_segment_mean split sqrt square squeeze stack standard_laplace standard_normal std std_mean
stft strided_slice sub subtract sum svd swapaxes swapdims t tan tanh tanhshrink tensor_add tensor_div tensor_dot
tensor_exp tensor_expm1 tensor_floordiv tensor_ge tensor_gt tensor_le tensor_lt tensor_mod tensor_mul tensor_pow
tensor_scatter_add tensor_scatter_div tensor_scatter_elements tensor_scatter_max tensor_scatter_min
tensor_scatter_mul tensor_scatter_sub tensor_slice tensor_split tensor_sub threshold tile top_k topk trace transpose
trapz tril tril_indices triplet_margin_loss triu triu_indices true_divide trunc truncate_div truncate_mod
tuple_to_array unbind unfold uniform uniform_candidate_sampler unique unique_consecutive unique_with_pad
unsorted_segment_max unsorted_segment_min unsorted_segment_prod unsorted_segment_sum unsqueeze unstack upsample
vander var var_mean vecdot vector_norm view_as_real vmap vsplit vstack where xdivy xlogy zeros zeros_like zeta
""".split()


def test_every_public_name_of_the_reference_function_modules_exists():
    missing = sorted(n for n in _FUNCTION_NAMES if not hasattr(ops, n))
    assert len(_FUNCTION_NAMES) > 600 and not missing, missing
