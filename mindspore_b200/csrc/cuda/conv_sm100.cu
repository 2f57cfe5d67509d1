// Implicit-GEMM convolution kernels for bf16 tensors; the fp16 build of the same text is conv_sm100_fp16.cu.
#include "conv_sm100_impl.cuh"
