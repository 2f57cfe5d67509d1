// Implicit-GEMM convolution kernels for fp16 tensors: the text of conv_sm100.cu with fp16 element types; every entry point carries the
// suffix _fp16.
#define MSB_ELEM_FP16 1
#include "conv_sm100_impl.cuh"
