// BatchNorm / pooling kernels for bf16 tensors; the fp16 build of the same text is bn_pool_fp16.cu.
#include "bn_pool_impl.cuh"
