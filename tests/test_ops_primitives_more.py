"""The long tail of primitive classes: a sample of each family against a formula, and the name coverage of the
reference's ``ops.operations`` modules (what is deliberately absent is listed)."""
import math

import numpy as np
import pytest
import torch

import mindspore_b200 as ms
from mindspore_b200 import ops

T = lambda *a, **k: ms.Tensor(torch.tensor(*a, **k))
N = lambda t: t.detach().as_subclass(torch.Tensor).numpy()


def test_linear_algebra_and_array_primitives():
    a = T([[4., 1.], [1., 3.]])
    u = N(ops.Cholesky(upper=True)(a))
    np.testing.assert_allclose(u.T @ u, N(a), rtol=1e-6)
    np.testing.assert_allclose(N(ops.MatrixInverse()(a)), np.linalg.inv(N(a)), rtol=1e-5)
    vals, idx = ops.Cummax(axis=0)(T([1., 3., 2.]))
    assert N(vals).tolist() == [1, 3, 3] and N(idx).tolist() == [0, 1, 1]
    assert N(ops.SegmentSum()(T([[1., 2.], [3., 4.], [5., 6.]]), T([0, 0, 1]))).tolist() == [[4, 6], [5, 6]]
    assert N(ops.SegmentMean()(T([1., 3., 5.]), T([0, 0, 1]))).tolist() == [2, 5]
    p = ms.Parameter(T(np.zeros(4, np.float32)))
    ops.ScatterNdAdd()(p, T([[1], [1]]), T([1., 2.]))
    assert N(p).tolist() == [0, 3, 0, 0]                       # in place on the Parameter
    q = ms.Parameter(T(np.ones((3, 2), np.float32)))
    ops.ScatterMul()(q, T([0, 2]), T([[2., 2.], [3., 3.]]))
    assert N(q).tolist() == [[2, 2], [1, 1], [3, 3]]
    assert N(ops.Roll(1, 0)(T([1, 2, 3]))).tolist() == [3, 1, 2]
    assert ops.Meshgrid(indexing="ij")((T([1, 2]), T([3, 4, 5])))[0].shape == (2, 3)
    assert N(ops.IsClose()(T([1.0, 2.0]), T([1.0 + 1e-9, 2.1]))).tolist() == [True, False]
    assert N(ops.SearchSorted()(T([1., 3., 5.]), T([2., 5.]))).tolist() == [1, 2]
    assert N(ops.Bucketize([1., 3.])(T([0., 2., 9.]))).tolist() == [0, 1, 2]
    out, argmax = ops.MaxPoolWithArgmax(2, 2)(T(np.arange(16, dtype=np.float32).reshape(1, 1, 4, 4)))
    assert N(argmax).reshape(-1).tolist() == [5, 7, 13, 15]
    assert N(ops.DepthToSpace(2)(ops.SpaceToDepth(2)(T(np.arange(16, dtype=np.float32).reshape(1, 1, 4, 4))))
             ).reshape(-1).tolist() == list(range(16))
    assert float(N(ops.EditDistance()(T([[0, 0], [0, 1]]), T([1, 2]), T([1, 2]), T([[0, 0], [0, 1]]), T([1, 3]),
                                      T([1, 2])))[0]) == 0.5
    assert ops.FFTWithSize(1, False, True)(T([1., 2., 3., 4.])).shape == (3,)
    std, mean = ops.ReduceStd(axis=0)(T([1., 2., 3.]))
    assert float(std) == 1.0 and float(mean) == 2.0
    with pytest.raises(TypeError):
        ops.Cummax()                                            # required attribute
    with pytest.raises(TypeError):
        ops.Cholesky(bogus=1)


def test_detection_and_nn_primitives():
    feat = T(np.arange(16, dtype=np.float32).reshape(1, 1, 4, 4))
    pooled = ops.ROIAlign(2, 2, 1.0, 2)(feat, T([[0., 0., 0., 3., 3.]]))
    assert pooled.shape == (1, 1, 2, 2) and float(N(pooled)[0, 0, 0, 0]) < float(N(pooled)[0, 0, 1, 1])
    boxes = T([[0., 0, 10, 10, 0.9], [1, 1, 10, 10, 0.8], [20, 20, 30, 30, 0.7]])
    _, order, mask = ops.NMSWithMask(0.5)(boxes)
    assert N(mask).tolist() == [True, False, True] and N(order).tolist() == [0, 1, 2]
    keep = ops.NonMaxSuppressionV3()(T([[0., 0, 10, 10], [1, 1, 10, 10], [20, 20, 30, 30]]), T([0.9, 0.8, 0.7]),
                                     T(10), T(0.5), T(0.0))
    assert N(keep).tolist() == [0, 2]
    rgb = T(np.random.RandomState(0).rand(2, 3, 3).astype(np.float32))
    np.testing.assert_allclose(N(ops.HSVToRGB()(ops.RGBToHSV()(rgb))), N(rgb), atol=1e-5)
    assert ops.Dilation2D(1, 1)(T(np.arange(9, dtype=np.float32).reshape(1, 1, 3, 3)),
                                T(np.zeros((1, 2, 2), np.float32))).shape == (1, 1, 3, 3)
    lstm = ops.LSTM(3, 4, 1, True, False, 0.0)
    ref = torch.nn.LSTM(3, 4)
    flat = torch.cat([ref.weight_ih_l0.reshape(-1), ref.weight_hh_l0.reshape(-1), ref.bias_ih_l0, ref.bias_hh_l0])
    x = torch.randn(5, 2, 3)
    out, hn, cn, _, _ = lstm(ms.Tensor(x), T(np.zeros((1, 2, 4), np.float32)), T(np.zeros((1, 2, 4), np.float32)),
                             ms.Tensor(flat.detach()))
    np.testing.assert_allclose(N(out), ref(x)[0].detach().numpy(), rtol=1e-5, atol=1e-6)
    dw = ops.DepthwiseConv2dNative(2, 3, pad_mode="same")(T(np.ones((1, 3, 5, 5), np.float32)),
                                                         T(np.ones((2, 3, 3, 3), np.float32)))
    assert dw.shape == (1, 6, 5, 5) and float(N(dw)[0, 0, 2, 2]) == 9
    dx = ops.Conv2DBackpropInput(4, 3, pad_mode="same")(T(np.ones((1, 4, 6, 6), np.float32)),
                                                        T(np.ones((4, 2, 3, 3), np.float32)), (1, 2, 6, 6))
    assert dx.shape == (1, 2, 6, 6) and float(N(dx)[0, 0, 3, 3]) == 36
    x = T([1., 2., 3.]).requires_grad_(True)
    ops.InsertGradientOf(lambda g: g * 2)(x).sum().backward()
    assert N(x.grad).tolist() == [2, 2, 2]
    with pytest.raises(RuntimeError):
        ops.Assert()(T(False), [T([1, 2, 3])])
    with pytest.raises(RuntimeError):
        ops.CheckNumerics()(T([float("nan")]))


def test_optimizer_update_and_quantisation_primitives():
    var, acc = ms.Parameter(T([1., 2.])), ms.Parameter(T([0.1, 0.1]))
    ops.ApplyAdagrad()(var, acc, 0.1, T([1., 1.]))
    np.testing.assert_allclose(N(acc), [1.1, 1.1], rtol=1e-6)
    np.testing.assert_allclose(N(var), [1 - 0.1 / math.sqrt(1.1), 2 - 0.1 / math.sqrt(1.1)], rtol=1e-6)
    var, ms_, mom = ms.Parameter(T([1.])), ms.Parameter(T([0.])), ms.Parameter(T([0.]))
    ops.ApplyRMSProp()(var, ms_, mom, 0.1, T([2.]), 0.9, 0.0, 1e-10)
    np.testing.assert_allclose(N(ms_), [0.4], rtol=1e-6)
    np.testing.assert_allclose(N(var), [1 - 0.1 * 2 / math.sqrt(0.4)], rtol=1e-5)
    var = ms.Parameter(T([[1., 1.], [2., 2.], [3., 3.]]))
    acc = ms.Parameter(T(np.zeros((3, 2), np.float32)))
    ops.SparseApplyAdagrad(lr=0.5)(var, acc, T([[1., 1.]]), T([2]))
    assert N(var)[:2].tolist() == [[1, 1], [2, 2]] and N(var)[2].tolist() == [2.5, 2.5]
    var, m, v = ms.Parameter(T([1.])), ms.Parameter(T([0.])), ms.Parameter(T([0.]))
    ops.ApplyAdaMax()(var, m, v, T(0.9), 0.1, 0.9, 0.999, 1e-8, T([1.]))
    np.testing.assert_allclose(N(var), [1 - 0.1 / (1 - 0.9) * 0.1 / 1.0], rtol=1e-5)
    fq = N(ops.FakeQuantPerLayer(num_bits=8)(T([0.2, 0.55, 0.83]), T([0.]), T([1.])))
    np.testing.assert_allclose(fq, np.round(np.array([0.2, 0.55, 0.83]) * 255) / 255, atol=1e-6)
    mn, mx = ops.MinMaxUpdatePerLayer()(T([-1., 2.]), T([0.]), T([0.]))
    assert N(mn).tolist() == [-1] and N(mx).tolist() == [2]
    gen = ops.DropoutGenMask(1, 2)((64,), T(0.5))
    kept = N(ops.DropoutDoMask()(T(np.ones(64, np.float32)), gen, T(0.5)))
    assert set(kept.tolist()) <= {0.0, 2.0} and 10 < (kept > 0).sum() < 54


def test_communication_primitives_are_reachable_from_ops():
    from mindspore_b200.ops import comm_ops
    assert ops.AllReduce is comm_ops.AllReduce and ops.operations.ReduceScatter is comm_ops.ReduceScatter
    assert ops.ReduceOp.SUM == "sum"
    from mindspore_b200.ops import AllGather, Send  # noqa: F401


# the public names of the reference's ops/operations/*.py modules that exist here ...
_PRESENT = """
ACos Abs AccumulateNV2 Acosh Adam AdamNoUpdateParam AdamWeightDecay AdaptiveAvgPool2D AdaptiveAvgPool3D
AdaptiveMaxPool2D AdaptiveMaxPool3D Add AddN Addcdiv Addcmul AdjustHue AdjustSaturation AffineGrid AllGather
AllReduce AlltoAll AlltoAllV Angle ApplyAdaMax ApplyAdadelta ApplyAdagrad ApplyAdagradDA ApplyAdagradV2
ApplyAdamWithAmsgrad ApplyAdamWithAmsgradV2 ApplyAddSign ApplyCenteredRMSProp ApplyFtrl ApplyGradientDescent
ApplyKerasMomentum ApplyMomentum ApplyPowerSign ApplyProximalAdagrad ApplyProximalGradientDescent ApplyRMSProp
ApplyRotaryPosEmb ApproximateEqual ArgMaxWithValue ArgMinWithValue Argmax Argmin Asin Asinh Assert Assign AssignAdd
AssignSub Atan Atan2 Atanh AvgPool AvgPool3D BCEWithLogitsLoss Barrier BartlettWindow BatchISendIRecv BatchMatMul
BatchNorm BatchToSpace BatchToSpaceND BatchToSpaceNDV2 Bernoulli BesselI0 BesselI0e BesselI1 BesselI1e BesselJ0
BesselJ1 BesselK0 BesselK0e BesselK1 BesselK1e BesselY0 BesselY1 Betainc BiasAdd BinaryCrossEntropy Bincount
BitwiseAnd BitwiseOr BitwiseXor BlackmanWindow BoundingBoxDecode BoundingBoxEncode Broadcast BroadcastTo Bucketize
CTCGreedyDecoder CTCLoss CTCLossV2 Cast Cauchy Cdist CeLU Ceil ChannelShuffle CheckNumerics CheckValid Cholesky
CholeskyInverse CholeskySolve Coalesce Col2Im CollectiveGather CollectiveScatter CompareAndBitpack Complex
ComplexAbs ComputeAccidentalHits Concat ConfusionMatrix Conj ConjugateTranspose Conv2D Conv2DBackpropInput
Conv2DTranspose Conv3D Conv3DTranspose CopyWithSlice Cos Cosh CountNonZero CropAndResize Cross CumProd CumSum Cummax
Cummin CumulativeLogsumexp Custom DType DataFormatDimMap DataFormatVecPermute Dense Depend DepthToSpace
DepthwiseConv2dNative Diag DiagPart Digamma Dilation2D Div DivNoNan Dropout Dropout2D Dropout3D DropoutDoMask
DropoutGenMask DynamicShape EditDistance Eig Einsum Elu EmbeddingLookup Eps Equal EqualCount Erf Erfc Erfinv
EuclideanNorm Exp Expand ExpandDims Expm1 ExtractGlimpse ExtractImagePatches Eye FFTWithSize FakeQuantParam
FakeQuantPerChannel FakeQuantPerLayer FakeQuantWithMinMaxVars FakeQuantWithMinMaxVarsPerChannel FastGeLU FastGelu
Fill FillDiagonal FillV2 Fills Flatten FloatStatus Floor FloorDiv FloorMod Fmax Fmin FusedCastAdamWeightDecay
FusedSparseAdam FusedSparseFtrl FusedSparseLazyAdam FusedSparseProximalAdagrad FusedWeightScaleApplyMomentum GLU
Gamma Gather GatherD GatherNd GatherV2 Gcd GeLU GeSwitch Gelu Geqrf Ger GetNext Greater GreaterEqual GridSampler2D
GridSampler3D HSVToRGB HShrink HSigmoid HSwish HammingWindow Heaviside Histogram HistogramFixedWidth
HistogramSummary HookBackward Hypot IOU Identity IdentityN Igamma Igammac Im2Col Imag ImageSummary InTopK IndexAdd
IndexFill IndexPut InplaceAdd InplaceIndexAdd InplaceSub InplaceUpdate InplaceUpdateV2 InsertGradientOf Inv Invert
InvertPermutation IsClose IsFinite IsInf IsNan KLDivLoss L2Loss L2Normalize LARSUpdate LRN LSTM LayerNorm Lcm
LeftShift Lerp Less LessEqual Lgamma LinSpace ListDiff Log Log1p LogMatrixDeterminant LogNormalReverse LogSoftmax
LogSpace LogUniformCandidateSampler LogicalAnd LogicalNot LogicalOr LogicalXor Logit LowerBound LpNorm Lstsq LuSolve
LuUnpack MaskedFill MaskedScatter MaskedSelect MatMul MatrixBandPart MatrixDeterminant MatrixDiagPartV3 MatrixDiagV3
MatrixExp MatrixInverse MatrixLogarithm MatrixPower MatrixSetDiagV3 MatrixSolve MatrixSolveLs MatrixTriangularSolve
MaxPool MaxPool3D MaxPool3DWithArgmax MaxPoolWithArgmax MaxPoolWithArgmaxV2 MaxUnpool2D MaxUnpool3D Maximum Merge
Meshgrid MinMaxUpdatePerChannel MinMaxUpdatePerLayer Minimum MirrorPad Mish Mod Mul MulNoNan MultiMarginLoss
MultilabelMarginLoss Multinomial MultinomialWithReplacement Mvlgamma NLLLoss NMSWithMask NPUAllocFloatStatus
NPUClearFloatStatus NPUGetFloatStatus NanToNum Neg NeighborExchange NeighborExchangeV2 NextAfter NoRepeatNGram
NonDeterministicInts NonMaxSuppressionV3 NonZero NotEqual NthElement NuclearNorm OneHot Ones OnesLike Orgqr Ormqr
PReLU Pack Pad PadV3 Padding PagedAttention PagedAttentionMask ParallelConcat ParameterizedTruncatedNormal Partial
Pdist Poisson Polar Polygamma PopulationCount Pow Print PyExecute PyFunc Qr Quantile RGBToHSV ROIAlign RaggedRange
RandomCategorical RandomChoiceWithMask RandomGamma RandomPoisson RandomShuffle Randperm RandpermV2 Range Rank ReLU
ReLU6 Real RealDiv Receive Reciprocal Reduce ReduceAll ReduceAny ReduceMax ReduceMean ReduceMin ReduceOp ReduceProd
ReduceScatter ReduceStd ReduceSum Renorm Reshape ReshapeAndCache Reshard ResizeArea ResizeBicubic ResizeBilinearV2
ResizeLinear1D ResizeNearestNeighbor ResizeNearestNeighborV2 Reusing ReverseSequence ReverseV2 RightShift Rint
RmsNorm Roll Round Rsqrt SGD STFT ScalarCast ScalarSummary ScalarToArray ScalarToTensor ScatterAdd
ScatterAddWithAxis ScatterDiv ScatterMax ScatterMin ScatterMul ScatterNd ScatterNdAdd ScatterNdDiv ScatterNdMax
ScatterNdMin ScatterNdMul ScatterNdSub ScatterNdUpdate ScatterNonAliasingAdd ScatterSub ScatterUpdate SeLU
SearchSorted SegmentMax SegmentMean SegmentMin SegmentProd SegmentSum Select SelectView Send Shape Sigmoid
SigmoidCrossEntropyWithLogits Sign Sin Sinc Sinh Size Slice SmoothL1Loss SoftMarginLoss SoftShrink Softmax
SoftmaxCrossEntropyWithLogits Softplus Softsign Sort SpaceToBatch SpaceToBatchND SpaceToDepth SparseApplyAdadelta
SparseApplyAdagrad SparseApplyAdagradV2 SparseApplyFtrl SparseApplyFtrlV2 SparseApplyProximalAdagrad
SparseApplyRMSProp SparseGatherV2 SparseSoftmaxCrossEntropyWithLogits SparseTensorDenseAdd SparseTensorDenseMatmul
SparseToDense Split SplitV Sqrt Square SquareSumAll SquaredDifference Squeeze Stack StandardLaplace StandardNormal
StopGradient StridedSlice Sub Svd Tan Tanh TensorAdd TensorDump TensorScatterAdd TensorScatterDiv
TensorScatterElements TensorScatterMax TensorScatterMin TensorScatterMul TensorScatterSub TensorScatterUpdate
TensorShape TensorSummary Tile TopK Trace Transpose TridiagonalMatMul Tril TrilIndices TripletMarginLoss Triu
TriuIndices Trunc TruncateDiv TruncateMod TruncatedNormal TupleToArray UniformCandidateSampler UniformInt
UniformReal Unique UniqueConsecutive UniqueWithPad Unpack UnravelIndex UnsortedSegmentMax UnsortedSegmentMin
UnsortedSegmentProd UnsortedSegmentSum Unstack UpdateState UpperBound UpsampleNearest3D UpsampleTrilinear3D Xdivy
Xlogy Zeros ZerosLike Zeta identity
""".split()

# ... and the ones that do not: Ascend quantisation-aware-training and THOR kernels (ActsULQ*, BatchNormFold*, Cus*,
# CorrectionMul*, FakeLearnedScale*, IFMR, WtsARQ, LoadIm2Col), gradient-only classes, parameter-server / embedding
# cache plumbing (Push, Pull, MapCacheIdx, MapUniform, SubAndFilter), reinforcement-learning buffers (Buffer*),
# Ascend recurrent kernels (DynamicRNN, DynamicGRUV2, BasicLSTMCell) and a few image / pooling variants
_ABSENT = """
ActULQClampMaxGrad ActULQClampMinGrad ActsULQ ActsULQInputGrad BasicLSTMCell BatchNormFold BatchNormFold2
BatchNormFold2D BatchNormFold2Grad BatchNormFold2GradD BatchNormFold2GradReduce BatchNormFoldD BatchNormFoldGrad
BatchNormFoldGradD BufferAppend BufferGetItem BufferSample CombinedNonMaxSuppression CorrectionMul CorrectionMulGrad
CorrectionMulGradReduce CusBatchMatMul CusCholeskyTrsm CusFusedAbsMax1 CusImg2Col CusMatMulCube
CusMatMulCubeDenseLeft CusMatMulCubeDenseRight CusMatMulCubeFraczLeftCast CusMatMulCubeFraczRightMul
CusMatrixCombine CusTranspose02314 DeformableOffsets DynamicGRUV2 DynamicRNN ExtractVolumePatches
FakeLearnedScaleQuantPerChannel FakeLearnedScaleQuantPerChannelGrad FakeLearnedScaleQuantPerChannelGradD
FakeLearnedScaleQuantPerChannelGradDReduce FakeLearnedScaleQuantPerLayer FakeLearnedScaleQuantPerLayerGrad
FakeLearnedScaleQuantPerLayerGradD FakeLearnedScaleQuantPerLayerGradDReduce FakeQuantPerChannelGrad
FakeQuantPerLayerGrad FakeQuantWithMinMaxVarsGradient FakeQuantWithMinMaxVarsPerChannelGradient FractionalAvgPool
FractionalMaxPool FractionalMaxPool3DWithFixedKsize FractionalMaxPoolWithFixedKsize FusedAdaFactor
FusedAdaFactorWithGlobalNorm IFMR LoadIm2Col MapCacheIdx MapUniform NonMaxSuppressionWithOverlaps Pull Push RNNTLoss
SampleDistortedBoundingBoxV2 ScaleAndTranslate SparseSlice SubAndFilter WtsARQ
""".split()


def test_primitive_name_coverage():
    missing = sorted(n for n in _PRESENT if not hasattr(ops, n))
    assert len(_PRESENT) > 520 and not missing, missing
    assert len(_ABSENT) < 80
